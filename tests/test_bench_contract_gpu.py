"""The benchmark's one JSON line, on two layers of the benchmark's sizes so that it takes seconds: the keys the contract
names, a flat `config` of at most twenty keys that gives both layer counts, and figures that hang together."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_bench_line_has_the_contract_keys(cuda_device):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--layers", "2", "--steps", "6", "--warmup", "3", "--points", "1"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1, "one JSON line"
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "prefill", "roofline", "points"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 6 and d["warmup"] == 3 and d["dtype"] == "bf16" and d["higher_is_better"] is True
    cfg = d["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values()), "config is flat, at most twenty keys"
    assert cfg["layers"] == 2 and cfg["layers_of_config"] == 32 and cfg["global_batch"] == 8 and cfg["hidden"] == 4096
    assert abs(d["value"] - 8 / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
    assert set(d["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} and d["e2e"]["h2d_bytes_per_step"] > 0
    assert 0.5 * d["value"] < d["e2e"]["value"] < 1.1 * d["value"], "end to end is its own measurement, near the device-timed one"
    assert set(d["prefill"]) >= {"value", "tokens", "ms", "frac"} and d["prefill"]["tokens"] == 2048 and 0 < d["prefill"]["frac"] < 1.2
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9 and 0 < r["frac"] < 1.2
    assert d["gpu_launches"] > 0 and "decode_b1" in d["points"]
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
