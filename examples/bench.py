"""The benchmark tool with InfiniLM's option names (its `examples/bench.py`): sweeps --input-len x --output-len at
--batch-size and prints time to first token, prefill and decode throughput.

    python examples/bench.py --model DIR --batch-size 8 --input-len 256,1024 --output-len 256,1024 --block-size 16 --enable-graph
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from infinilm_b200.cli import bench_main  # noqa: E402

if __name__ == "__main__":
    sys.exit(bench_main())
