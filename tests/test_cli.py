"""The command line on the CPU: InfiniLM's option names parse, and the random-weights mode writes a
model folder that loads back (no GPU needed for either)."""
import json
import os
import subprocess
import sys

import pytest

from infinilm_b200.cli import build_parser, main
from infinilm_b200.config import load_config
from infinilm_b200.weights import FolderSource, check_against
from tiny_configs import tiny_b

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_option_names_of_infinilm_parse():
    a = build_parser().parse_args(["--model", "/m", "--device", "nvidia", "--attn", "paged-attn", "--enable-graph", "--enable-paged-attn",
                                   "--disable-prefix-caching", "--num-blocks", "64", "--block-size", "16", "--skip-load",
                                   "--batch-size", "3", "--max-batch-size", "4", "--max-new-tokens", "7", "--prompt", "hi",
                                   "--top-k", "5", "--top-p", "0.9", "--temperature", "0.7", "--ignore-eos", "--warmup",
                                   "--log-level", "DEBUG", "--dtype", "bfloat16"])
    assert (a.model, a.attn, a.enable_graph, a.enable_paged_attn, a.num_blocks, a.block_size) == ("/m", "paged-attn", True, True, 64, 16)
    assert (a.batch_size, a.max_batch_size, a.max_new_tokens, a.top_k, a.top_p, a.temperature) == (3, 4, 7, 5, 0.9, 0.7)
    assert a.skip_load and a.ignore_eos and a.warmup and a.enable_prefix_caching is False
    d = build_parser().parse_args(["--model", "/m"])           # InfiniLM's defaults
    assert (d.num_blocks, d.block_size, d.max_new_tokens, d.top_k, d.top_p, d.temperature, d.batch_size) == (512, 256, 512, 1, 1.0, 1.0, 1)
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--model", "/m", "--attn", "other"])


def test_length_lists_of_the_benchmark_tool_parse_as_infinilm_spells_them():
    from infinilm_b200.cli import parse_list
    assert parse_list("7") == 7 and parse_list("[1,2,4]") == [1, 2, 4] and parse_list("256, 1024") == [256, 1024]
    import argparse
    with pytest.raises(argparse.ArgumentTypeError):
        parse_list("a,b")
    a = build_parser().parse_args(["--model", "/m", "--input-len", "256,1024", "--output-len", "[16]", "--batch-size", "8"])
    assert a.input_len == [256, 1024] and a.output_len == [16]
    d = build_parser().parse_args(["--model", "/m"])
    assert (d.input_len, d.output_len) == (10, 20)              # InfiniLM's defaults


def test_write_random_model_and_missing_arguments(tmp_path, capsys):
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(tiny_b()))
    out = tmp_path / "m"
    assert main(["--write-random-model", str(out), "--config", str(cfg_path), "--seed", "5"]) == 0
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    cfg = load_config(str(out))
    from infinilm_b200.config import describe_model
    from infinilm_b200.models.causal_lm import CausalLM
    import torch
    src = FolderSource(str(out))
    check_against(CausalLM(describe_model(cfg), torch.float32), src)
    src.close()
    assert main(["--write-random-model", str(out)]) == 2       # --config is needed
    assert main([]) == 2                                        # --model is needed


def test_trace_run_help_runs_without_a_gpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--help"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "--max-tokens" in p.stdout and "--dtype" in p.stdout


def _bench(*args):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return subprocess.run([sys.executable, os.path.join(root, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_bench_answers_without_a_gpu_where_it_runs_nothing():
    """More than one GPU: one line that says so and exit code 2. The reference arm: its `unavailable` line and exit code 0."""
    p = _bench("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2 and len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout
    p = _bench("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]
