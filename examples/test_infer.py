"""Generate for a prompt, as InfiniLM's `examples/test_infer.py` does:

    python examples/test_infer.py --model DIR --enable-paged-attn --batch-size 2 --max-new-tokens 32
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from infinilm_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
