"""Generation through the Python entry point and the command line tools: greedy against the plain
implementation, seeded temperature sampling (repeatable, independent of what else is in the
batch, equal to the plain sampler), CUDA-graph replay against eager steps, preemption by
recomputation, and `bin/trace_run` as a separate process."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model
from replay_util import TOL, check_greedy, plain_logits, rel_err
from tiny_configs import TINY, make_weights, random_ids, tiny_a, tiny_b

pytestmark = pytest.mark.gpu

from infinilm_b200.config import config_from_json  # noqa: E402
from infinilm_b200.llm import LLM, SamplingParams  # noqa: E402
from infinilm_b200.sampling import uniform01  # noqa: E402
from infinilm_b200.weights import write_model_folder  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_greedy_generation_matches_plain(cuda_device):
    raw = tiny_a()
    w = make_weights(raw, 0)
    prompts = [random_ids(n, raw["vocab_size"], 20 + n) for n in (5, 17, 33)]
    llm = LLM.from_tensors(config_from_json(raw), w, dtype="float32", num_blocks=16, block_size=16, max_batch_size=3)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(top_k=1, max_tokens=16, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == plain_model.greedy_generate(raw, w, p, 16)
        assert o.finished and o.finish_reason.value == "length" and o.prompt_token_ids == p
    assert llm.stats()["free_pages"] == 16
    # bfloat16: the same tokens as long as the plain top-2 margin is wide enough to survive rounding
    llm16 = LLM.from_tensors(config_from_json(raw), w, dtype="bfloat16", num_blocks=16, block_size=16, max_batch_size=3)
    outs16 = llm16.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(top_k=1, max_tokens=16, ignore_eos=True))
    for p, o in zip(prompts, outs16):
        ids = list(p)
        for t in o.outputs[0].token_ids:
            lg = plain_logits(raw, w, ids, "bfloat16")[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 4 * TOL["bfloat16"] * float(lg.abs().max()):
                assert t == int(torch.argmax(lg))
            ids.append(t)


def test_sampling_parameters_may_differ_from_prompt_to_prompt(cuda_device):
    raw = tiny_a()
    w = make_weights(raw, 0)
    prompts = [random_ids(n, raw["vocab_size"], 40 + n) for n in (7, 21, 4)]
    llm = LLM.from_tensors(config_from_json(raw), w, dtype="float32", num_blocks=16, block_size=16, max_batch_size=3)
    sps = [SamplingParams(top_k=1, max_tokens=m, ignore_eos=True) for m in (3, 11, 6)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=sps)
    for p, o, m in zip(prompts, outs, (3, 11, 6)):
        assert o.outputs[0].token_ids == plain_model.greedy_generate(raw, w, p, m)


def test_eos_stops_generation(cuda_device):
    raw = tiny_a()
    w = make_weights(raw, 0)
    p = random_ids(9, raw["vocab_size"], 3)
    ref = plain_model.greedy_generate(raw, w, p, 12)
    raw2 = dict(raw, eos_token_id=ref[4])
    first = ref.index(ref[4])
    llm = LLM.from_tensors(config_from_json(raw2), w, dtype="float32", num_blocks=8, block_size=16, max_batch_size=2)
    o = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(top_k=1, max_tokens=12))[0]
    assert o.outputs[0].token_ids == ref[:first + 1] and o.finish_reason.value == "eos_token"
    o = llm.generate(prompt_token_ids=[p], sampling_params=SamplingParams(top_k=1, max_tokens=12, ignore_eos=True))[0]
    assert o.outputs[0].token_ids == ref


def _plain_sampled(raw, w, prompt, n_new, sp, seed, stream):
    ids, out = list(prompt), []
    for i in range(n_new):
        lg = plain_model.forward(raw, w, ids)[-1]
        t = plain_model.sample_plain(lg, sp.temperature, sp.top_k, sp.top_p, uniform01(seed, stream, i))
        out.append(t)
        ids.append(t)
    return out


def test_temperature_sampling_mixed_batch(cuda_device):
    """Four requests with prompts of 3, 40, 70 and 100 tokens under chunked prefill (portions of 16),
    temperature 0.7 with a fixed seed: repeatable, the same whether a request runs alone or with the
    others, and equal to the plain sampler on plain logits."""
    raw = tiny_b()
    w = make_weights(raw, 1)
    cfg = config_from_json(raw)
    prompts = [random_ids(n, raw["vocab_size"], 30 + n) for n in (3, 40, 70, 100)]
    sp = SamplingParams(temperature=0.7, top_k=0, top_p=0.9, max_tokens=12, ignore_eos=True)

    def run(batch, **kw):
        llm = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=40, block_size=16, max_batch_size=4,
                               chunk_size=16, max_num_batched_tokens=40, seed=5, **kw)
        return [o.outputs[0].token_ids for o in llm.generate(prompt_token_ids=batch, sampling_params=sp)]
    together = run(prompts)
    assert together == run(prompts)
    assert len({tuple(t) for t in together}) == 4
    for i, p in enumerate(prompts):
        # alone, the request is the engine's first (stream 0); give it the stream it had in the batch
        llm = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=40, block_size=16, max_batch_size=4, chunk_size=16,
                               max_num_batched_tokens=40, seed=5)
        llm._n_requests = i
        assert llm.generate(prompt_token_ids=[p], sampling_params=sp)[0].outputs[0].token_ids == together[i]
        assert together[i] == _plain_sampled(raw, w, p, 12, sp, 5, i)
    other = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=40, block_size=16, max_batch_size=4, seed=6)
    assert [o.outputs[0].token_ids for o in other.generate(prompt_token_ids=prompts, sampling_params=sp)] != together


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager(cuda_device, dtype):
    raw = tiny_b()
    w = make_weights(raw, 2)
    cfg = config_from_json(raw)
    prompts = [random_ids(n, raw["vocab_size"], 60 + n) for n in (7, 30, 18)]
    sp = SamplingParams(top_k=1, max_tokens=40, ignore_eos=True)
    outs = []
    for graph, pipelined in ((False, True), (True, True), (True, False), (False, False)):
        llm = LLM.from_tensors(cfg, w, dtype=dtype, num_blocks=32, block_size=16, max_batch_size=4, enable_graph=graph,
                               pipelined=pipelined)
        outs.append([o.outputs[0].token_ids for o in llm.generate(prompt_token_ids=prompts, sampling_params=sp)])
        if graph:
            assert any(g.graph is not None for g in llm.engine.runner._graphs.values())
            # most decode steps followed the same requests' step before them and were made from it
            assert llm.engine.runner.fast_steps > 20
    # reading a step's tokens one step late (the next step gets them on the device) changes nothing
    assert outs[0] == outs[1] == outs[2] == outs[3]
    # and the four are the plain implementation's tokens, not just one another's
    for p, toks in zip(prompts, outs[1]):
        check_greedy(raw, w, p, toks, dtype)


def test_sampling_parameters_of_a_step_survive_the_next_step(cuda_device):
    """Pipelined stepping fills the sampling parameters of step k+1 on the host before the GPU has copied those of
    step k (here the GPU is held back on purpose, as it is by a large model): every step must still draw with its own
    uniform numbers. Eight temperature requests with eight live requests at most, so that the rows fill the buffer."""
    raw = tiny_b()
    w = make_weights(raw, 4)
    cfg = config_from_json(raw)
    prompts = [random_ids(9, raw["vocab_size"], 70 + i) for i in range(8)]
    sp = SamplingParams(temperature=0.9, top_k=0, top_p=0.95, max_tokens=10, ignore_eos=True)

    def run(pipelined, hold_back):
        llm = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=40, block_size=16, max_batch_size=8, seed=11,
                               pipelined=pipelined)
        assert llm.sampler.max_rows == 8
        if hold_back:
            step = llm.engine.step

            def slow_step(entries, device_tokens=None):
                torch.cuda._sleep(30_000_000)       # some 15 ms of GPU time in front of every step
                return step(entries, device_tokens)
            llm.engine.step = slow_step
        outs = [o.outputs[0].token_ids for o in llm.generate(prompt_token_ids=prompts, sampling_params=sp)]
        llm.close()
        return outs
    ref = run(False, False)
    assert run(True, True) == ref
    assert run(True, False) == ref
    for i in (0, 7):
        assert ref[i] == _plain_sampled(raw, w, prompts[i], 10, sp, 11, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("block_size", [None, 16])
def test_command_line_generates_the_plain_tokens(cuda_device, tmp_path, capsys, dtype, block_size):
    """`python -m infinilm_b200 --model DIR ...` as a user runs it: a folder written by --write-random-model, the
    default block size (256, InfiniLM's) and 16, both precisions; the printed token ids are the plain implementation's."""
    import warnings

    from infinilm_b200.cli import main
    raw = TINY["d"]()
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(raw))
    model_dir = str(tmp_path / "model")
    assert main(["--write-random-model", model_dir, "--config", str(cfg_path), "--seed", "3"]) == 0
    from infinilm_b200.weights import random_tensors
    w = random_tensors(config_from_json(raw), 3, "cpu")
    prompt = random_ids(70, raw["vocab_size"], 5)
    argv = ["--model", model_dir, "--dtype", dtype, "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "12",
            "--batch-size", "2", "--ignore-eos", "--num-blocks", "8" if block_size is None else "64", "--log-level", "ERROR"]
    if block_size is not None:
        argv += ["--block-size", str(block_size)]
    capsys.readouterr()
    with warnings.catch_warnings():
        warnings.filterwarnings("error", message="attention:")    # the fast kernels take both page sizes: no fallback
        assert main(argv) == 0
    printed = capsys.readouterr().out
    answers = [json.loads(ln) for ln in printed.splitlines() if ln.startswith("[") and ln.endswith("]")]
    answers = [a for a in answers if a != prompt]
    assert len(answers) == 2 and answers[0] == answers[1] and len(answers[0]) == 12
    check_greedy(raw, w, prompt, answers[0], dtype)
    assert "total_time" in printed and "finish_reason: length" in printed


def test_benchmark_tool_sweeps_lengths(cuda_device, tmp_path, capsys):
    """`examples/bench.py` (InfiniLM's benchmark tool): lists of input and output lengths at a batch size, one record a case."""
    from infinilm_b200.cli import bench_main
    raw = TINY["d"]()
    model_dir = write_model_folder(config_from_json(raw), 4, str(tmp_path / "model"))
    capsys.readouterr()
    assert bench_main(["--model", model_dir, "--batch-size", "3", "--input-len", "20,150", "--output-len", "[5,9]", "--block-size", "16",
                       "--num-blocks", "64", "--enable-graph", "--log-level", "ERROR"]) == 0
    out = capsys.readouterr().out
    recs = json.loads([ln for ln in out.splitlines() if ln.startswith('{"bench"')][0])["bench"]
    assert [(r["input_len"], r["output_len"], r["batch_size"]) for r in recs] == [(20, 5, 3), (20, 9, 3), (150, 5, 3), (150, 9, 3)]
    assert all(r["prefill_tok_s"] > 0 and r["decode_tok_s"] > 0 and r["ttft_ms"] > 0 for r in recs)
    assert out.count("Prefill TTFT:") == 4 and out.count("Decode  Avg ITL:") == 4


def test_entry_point_loads_a_folder_at_the_default_block_size(cuda_device, tmp_path):
    """`LLM(model_path=...)` with every default (pages of 256 tokens): the bfloat16 path stays on its fast attention
    kernels, and a page is a run of sixteen kernel pages."""
    import warnings
    raw = TINY["d"]()
    cfg = config_from_json(raw)
    model_dir = write_model_folder(cfg, 9, str(tmp_path / "model"))
    from infinilm_b200.weights import random_tensors
    w = random_tensors(cfg, 9, "cpu")
    with warnings.catch_warnings():
        warnings.filterwarnings("error", message="attention:")
        llm = LLM(model_dir, num_blocks=6, max_batch_size=4)
        assert llm.engine.cache.page_size == 256 and llm.engine.cache.kernel_page == 16 and llm.engine.cache.sub == 16
        assert llm.engine.dtype_name == "bfloat16"
        prompts = [random_ids(n, raw["vocab_size"], 80 + n) for n in (3, 120, 260)]
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(top_k=1, max_tokens=20, ignore_eos=True))
    for p, o in zip(prompts, outs):
        check_greedy(raw, w, p, o.outputs[0].token_ids, "bfloat16")
    assert llm.stats()["free_pages"] == 6
    llm.close()


def test_preemption_recomputes_to_the_same_tokens(cuda_device):
    """With so few pages that the younger request is preempted and recomputed, greedy outputs are
    those of a roomy run."""
    raw = tiny_a()
    w = make_weights(raw, 3)
    cfg = config_from_json(raw)
    prompts = [random_ids(20, raw["vocab_size"], 1), random_ids(20, raw["vocab_size"], 2)]
    sp = SamplingParams(top_k=1, max_tokens=60, ignore_eos=True)
    roomy = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=32, block_size=16, max_batch_size=2)
    ref = [o.outputs[0].token_ids for o in roomy.generate(prompt_token_ids=prompts, sampling_params=sp)]
    tight = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=8, block_size=16, max_batch_size=2, admission="optimistic")
    got = [o.outputs[0].token_ids for o in tight.generate(prompt_token_ids=prompts, sampling_params=sp)]
    assert tight.scheduler.n_preemptions >= 1 and got == ref
    waits = LLM.from_tensors(cfg, w, dtype="float32", num_blocks=8, block_size=16, max_batch_size=2)   # worst_case
    assert [o.outputs[0].token_ids for o in waits.generate(prompt_token_ids=prompts, sampling_params=sp)] == ref
    assert waits.scheduler.n_preemptions == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_process(cuda_device, tmp_path, dtype):
    raw = tiny_b()
    cfg = config_from_json(raw)
    model_dir = write_model_folder(cfg, 7, str(tmp_path / "model"))
    from infinilm_b200.weights import random_tensors
    w = random_tensors(cfg, 7, "cpu")
    a, b = random_ids(50, raw["vocab_size"], 1), random_ids(21, raw["vocab_size"], 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},          # nothing wanted: no file
        {"step": 2, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[2:21], "want": [18, 0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[31:50], "want": list(range(19))}], "end": ["a"]},
    ]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(out_dir)) == ["0.f32", "2.f32", "3.f32"]
    V = raw["vocab_size"]
    la, lb = plain_logits(raw, w, a, dtype), plain_logits(raw, w, b, dtype)
    want = {0: torch.stack([la[0], la[29]]), 2: torch.stack([la[30], lb[20], lb[2]]), 3: la[31:50]}
    for s, ref in want.items():
        got = torch.from_numpy(np.fromfile(out_dir / f"{s}.f32", dtype="<f4").reshape(-1, V))
        assert rel_err(got, ref) <= TOL[dtype], f"step {s}"
