"""Benchmark: decode tokens/s at batch 8 (and 1, 64) and prefill tokens/s at 2,048 tokens, MiniCPM4-8B
layer sizes with random weights in bfloat16 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

Prints ONE JSON line. A step is one decode step (forward of one token per request over the paged
cache, plus sampling). `value` is timed on the device with CUDA events; `e2e` is the same number
through the Python entry point (`LLM.step`: descriptors copied from pinned host memory every
step, sampled ids read back every step). The definitions are InfiniLM's own
(`python/infinilm/infer_engine.py:720-726`): prefill tok/s = tokens / time of the prompt step,
decode tok/s = batch * steps / time of the decode steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# MiniCPM4-8B layer sizes (the benchmark configuration).
CONFIG_8B = {
    "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 16384, "vocab_size": 73448,
    "rope_theta": 10000.0, "max_position_embeddings": 32768,
    "rope_scaling": {"rope_type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(64)],
                     "long_factor": [1.0 + 0.25 * i for i in range(64)], "original_max_position_embeddings": 32768},
    "scale_emb": 12, "dim_model_base": 256, "scale_depth": 1.4, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "eos_token_id": [2, 73440],
}
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE = 16


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except Exception:
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(cfg, n_layers):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim * H
    o = H * cfg.num_attention_heads * cfg.head_dim
    per_layer = qkv + o + 3 * H * I + 2 * H
    return 2 * (per_layer * n_layers + V * H + H), per_layer


def profile_step(args) -> int:
    """One decode step (batch --batch, --prompt-len tokens cached) or one prefill step (the last 2,048 tokens of a
    --prompt-len prompt) of the benchmark model with --layers layers, bracketed by cudaProfilerStart/Stop; nothing is timed or printed but 'profiled'."""
    import torch

    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    from infinilm_b200.weights import random_tensors
    raw = dict(CONFIG_05B if args.sizes == "0.5b" else CONFIG_8B)
    raw["num_hidden_layers"] = args.layers or 2
    cfg = config_from_json(raw)
    B, P = args.batch, args.prompt_len
    if P % PROMPT_LEN or P <= 0 or P + 16 > cfg.max_position_embeddings:
        print(f"--prompt-len must be a positive multiple of {PROMPT_LEN} below the model's maximum")
        return 2
    eng = Engine.from_tensors(cfg, random_tensors(cfg, 0, "cuda:0"), dtype="bfloat16", page_size=PAGE,
                              num_pages=B * (P // PAGE + 4) + 8, max_seqs=max(B, 2), max_batch_tokens=4096)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (P,), generator=g).tolist() for _ in range(B)]

    def feed(seq, ids, upto):                     # a prompt's tokens [0, upto) in portions of 2,048, nothing wanted
        for a in range(0, upto, PROMPT_LEN):
            eng.step([StepEntry(seq, ids[a:a + PROMPT_LEN], [])])
    if args.profile_step == "decode":
        seqs = [eng.open(i) for i in range(B)]
        for s, p in zip(seqs, prompts):
            feed(s, p, P)
        for _ in range(2):
            eng.step([StepEntry(s, [5], [0]) for s in seqs])
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.step([StepEntry(s, [5], [0]) for s in seqs])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:                                         # the last portion of the prompt, over the cache of the others
        for i in range(2):
            s = eng.open(("w", i))
            feed(s, prompts[0], P)
            eng.close(s)
        s = eng.open("p")
        feed(s, prompts[0], P - PROMPT_LEN)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        eng.step([StepEntry(s, prompts[0][P - PROMPT_LEN:], [PROMPT_LEN - 1])])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print("profiled")
    return 0


def timeline_step(args) -> int:
    """The kernels of one replayed decode step (batch --batch, --prompt-len tokens cached, --layers layers) with their start
    and duration as the profiler of the framework underneath (CUPTI activity records) sees them inside the replayed
    graph: kernels overlap their predecessors there, which a serialising profiler cannot show. Prints a table; nothing
    here is a benchmark value."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    from infinilm_b200.weights import random_tensors
    raw = dict(CONFIG_05B if args.sizes == "0.5b" else CONFIG_8B)
    raw["num_hidden_layers"] = args.layers or 4
    cfg = config_from_json(raw)
    B, P = args.batch, args.prompt_len
    eng = Engine.from_tensors(cfg, random_tensors(cfg, 0, "cuda:0"), dtype="bfloat16", page_size=PAGE,
                              num_pages=B * (P // PAGE + 4) + 8, max_seqs=max(B, 2), max_batch_tokens=4096)
    eng.enable_graphs()
    g = torch.Generator().manual_seed(1)
    seqs = [eng.open(i) for i in range(B)]
    for s in seqs:
        ids = torch.randint(0, cfg.vocab_size, (P,), generator=g).tolist()
        for a in range(0, P, PROMPT_LEN):
            eng.step([StepEntry(s, ids[a:a + PROMPT_LEN], [])])
    for _ in range(6):
        eng.step([StepEntry(s, [5], [0]) for s in seqs])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            eng.step([StepEntry(s, [5], [0]) for s in seqs])
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "emcpy" not in e.name and "emset" not in e.name),
                key=lambda e: e.time_range.start)
    last = ev[-(len(ev) // 3):]
    t0 = last[0].time_range.start
    print("| start us | duration us | start of the next - start us | kernel |")
    print("|---|---|---|---|")
    for e, nxt in zip(last, last[1:] + [None]):
        a = e.time_range.start - t0
        gap = f"{nxt.time_range.start - e.time_range.start:.1f}" if nxt is not None else ""
        print(f"| {a:.1f} | {e.time_range.end - e.time_range.start:.1f} | {gap} | {e.name[:64]} |")
    print(f"\nstep: {last[-1].time_range.end - t0:.1f} us, {len(last)} kernels, {raw['num_hidden_layers']} layers, batch {B}, {P} tokens cached")
    return 0


CONFIG_05B = dict(CONFIG_8B, num_hidden_layers=24, hidden_size=1024, num_attention_heads=16, num_key_value_heads=2, head_dim=64,
                  intermediate_size=4096, tie_word_embeddings=True,
                  rope_scaling={"rope_type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(32)],
                                "long_factor": [1.0 + 0.25 * i for i in range(32)], "original_max_position_embeddings": 32768})


def run_workload(args) -> int:
    """The two serving workloads of the baseline beside the headline: both go through `LLM.generate`
    (scheduler, chunked prefill mixed with decoding, paged cache, sampling), host tokens in and out."""
    import torch

    from infinilm_b200.config import config_from_json
    from infinilm_b200.llm import LLM, SamplingParams
    from infinilm_b200.weights import random_tensors
    long_ctx = args.workload == "long_context"
    raw = dict(CONFIG_8B if long_ctx else CONFIG_05B)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_json(raw)
    g = torch.Generator().manual_seed(2)
    if long_ctx:
        n_req, new = 8, 512
        lens = [16384] * n_req
        max_b, chunk, budget = 8, 2048, 2048 + 8
    else:
        n_req, new = 256, 256
        lens = torch.randint(16, 4097, (n_req,), generator=g).tolist()
        max_b, chunk, budget = 256, 2048, 4096
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    pages = sum((n + new + PAGE - 1) // PAGE + 1 for n in lens) + 16
    t0 = time.perf_counter()
    llm = LLM.from_tensors(cfg, random_tensors(cfg, 0, "cuda:0"), dtype="bfloat16", num_blocks=pages, block_size=PAGE,
                           max_batch_size=max_b, max_num_batched_tokens=budget, chunk_size=chunk, enable_graph=not args.no_graph)
    sp = SamplingParams(top_k=1, max_tokens=new, ignore_eos=True)
    warm = llm.generate(prompt_token_ids=[prompts[0][:64]], sampling_params=SamplingParams(top_k=1, max_tokens=4, ignore_eos=True))
    assert len(warm[0].outputs[0].token_ids) == 4
    torch.cuda.synchronize()
    steps0, toks0 = llm.engine.runner.steps_run, llm.engine.runner.tokens_run
    t1 = time.perf_counter()
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=sp)
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    n_new = sum(len(o.outputs[0].token_ids) for o in outs)
    assert n_new == n_req * new and all(o.finish_reason.value == "length" for o in outs)
    st = llm.stats()
    rec = {"workload": args.workload, "impl": "ours", "dtype": "bf16", "n_gpus": 1,
           "config": {"model": "MiniCPM4-8B sizes" if long_ctx else "MiniCPM4-0.5B sizes", "layers": cfg.num_hidden_layers,
                      "requests": n_req, "prompt_tokens": sum(lens), "new_tokens_each": new, "chunk": chunk, "page_size": PAGE,
                      "max_live": max_b, "token_budget": budget},
           "seconds": t2 - t1, "steps": llm.engine.runner.steps_run - steps0,
           "tokens_run": llm.engine.runner.tokens_run - toks0,
           "total_tok_per_s": (sum(lens) + n_new) / (t2 - t1), "new_tok_per_s": n_new / (t2 - t1),
           "preemptions": st["preemptions"], "free_pages_after": st["free_pages"], "pool_pages": st["pool_pages"],
           "setup_s": round(t1 - t0, 1)}
    print(json.dumps(rec))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--sizes", choices=["8b", "0.5b"], default="8b",
                    help="layer sizes: MiniCPM4-8B (the benchmark's) or MiniCPM4-0.5B (hidden 1024, head_dim 64; not the headline)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="tokens cached per request before decoding (a multiple of 2,048; default: the configuration's 2,048). "
                         "With more, prompts go in portions of 2,048 and `prefill` times the LAST portion, over the cache of the others")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-graph", action="store_true", help="do not replay decode steps as CUDA graphs")
    ap.add_argument("--points", type=str, default="1,64", help="batch sizes of the extra decode points")
    ap.add_argument("--workload", choices=["default", "long_context", "continuous"], default="default",
                    help="default: the benchmark line. long_context: 8 requests x 16,384-token prompts at 8B sizes, prompt "
                         "portions of 2,048 interleaved with the others' decoding, 512 new tokens each. continuous: 256 requests "
                         "at 0.5B sizes, prompts of 16..4096 tokens, 256 new tokens each. Both print their own JSON line.")
    ap.add_argument("--profile-step", choices=["decode", "prefill"], default=None,
                    help="run one step of this kind between cudaProfilerStart/Stop and exit (for ncu --profile-from-start off); "
                         "use with --layers 2 to keep the capture small")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one replayed decode step with start and duration inside the graph "
                         "(--batch, --layers, --sizes, --prompt-len apply) and exit")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "InfiniLM needs InfiniCore (infinicore Python package, infiniop/infinirt libraries, xmake); "
                          "none is in the image or the wheelhouse, so it cannot be installed offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this engine has no multi-GPU path); --gpus {args.gpus} is not run")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from infinilm_b200 import ops
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    from infinilm_b200.llm import LLM, SamplingParams
    from infinilm_b200.weights import random_tensors

    if args.profile_step:
        return profile_step(args)
    if args.timeline:
        return timeline_step(args)
    if args.workload != "default":
        return run_workload(args)
    raw = dict(CONFIG_05B if args.sizes == "0.5b" else CONFIG_8B)
    full_layers = raw["num_hidden_layers"]
    n_layers = args.layers or full_layers
    raw["num_hidden_layers"] = n_layers
    # the branch scale is scale_depth / sqrt(layers): with fewer layers than the configuration has, scale_depth is
    # lowered so that each branch keeps the scale it has in the full model
    raw["scale_depth"] = raw["scale_depth"] * (n_layers / full_layers) ** 0.5
    cfg = config_from_json(raw)
    hbm_peak, tf_peak, peak_src = load_peaks()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    K, W = args.steps, args.warmup
    P = args.prompt_len
    if P % PROMPT_LEN or P <= 0 or P + 2 * (K + W) + 8 > cfg.max_position_embeddings:
        print(f"--prompt-len must be a positive multiple of {PROMPT_LEN} that leaves room for the decoded tokens")
        return 2
    max_b = max([args.batch] + ([] if args.no_points else [int(b) for b in args.points.split(',') if b]))
    pages_per_req = (P + 2 * (K + W) + (args.batch * P + 4095) // 4096 + args.batch + 16 + PAGE - 1) // PAGE + 1
    num_pages = max_b * pages_per_req + 8

    t_setup = time.time()
    tensors = random_tensors(cfg, 0, dev)
    llm = LLM.from_tensors(cfg, tensors, dtype="bfloat16", num_blocks=num_pages, block_size=PAGE,
                           max_batch_size=max_b, max_num_batched_tokens=4096, chunk_size=PROMPT_LEN,
                           enable_graph=not args.no_graph)
    del tensors
    eng = llm.engine
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (P,), generator=g).tolist() for _ in range(max_b)]
    wbytes, _ = weight_bytes(cfg, n_layers)
    kv_per_token = eng.cache.bytes_per_token(2)

    def flops_prefill(T, before=0):
        _, per_layer = weight_bytes(cfg, n_layers)
        lin = 2.0 * T * (per_layer - 2 * cfg.hidden_size) * n_layers + 2.0 * cfg.vocab_size * cfg.hidden_size
        attn = 4.0 * (T * before + T * (T + 1) / 2) * cfg.num_attention_heads * cfg.head_dim * n_layers
        return lin + attn

    def feed(seq, ids, upto):                     # a prompt's tokens [0, upto) in portions of 2,048, nothing wanted
        for a in range(0, upto, PROMPT_LEN):
            eng.step([StepEntry(seq, ids[a:a + PROMPT_LEN], [])])

    # ---- prefill: one portion of 2,048 tokens, one step (the whole prompt at the default length) ------
    def time_prefill(reps):
        times = []
        for i in range(reps):
            seq = eng.open(("pf", i))
            feed(seq, prompts[0], P - PROMPT_LEN)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            eng.step([StepEntry(seq, prompts[0][P - PROMPT_LEN:], [PROMPT_LEN - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.close(seq)
        return times
    time_prefill(4)                               # warm-up: by its fourth coming the step is captured and replayed as a graph
    pf_ms = statistics.median(time_prefill(3))
    prefill = {"value": PROMPT_LEN / (pf_ms / 1e3), "tokens": PROMPT_LEN, "ms": pf_ms,
               "frac": flops_prefill(PROMPT_LEN, P - PROMPT_LEN) / (pf_ms / 1e3) / (tf_peak * 1e12)}
    if P != PROMPT_LEN:
        prefill["cached_before"] = P - PROMPT_LEN

    # ---- decode on the device: B requests with 2,048 tokens cached, K timed steps -----------------
    def time_decode(B, clocks=None):
        seqs = [eng.open(("d", B, i)) for i in range(B)]
        for i, s in enumerate(seqs):
            feed(s, prompts[i], P)
        toks = [[(7 * i + 3) % cfg.vocab_size] for i in range(B)]

        def one():
            logits = eng.step([StepEntry(s, t, [0]) for s, t in zip(seqs, toks)])
            llm.sampler.argmax(logits)
        for _ in range(W):
            one()
        torch.cuda.synchronize()
        n0 = ops.launch_count()
        if clocks is not None:
            clocks.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        ck = clocks.stop() if clocks is not None else None
        launches = ops.launch_count() - n0
        ctx = seqs[0].length
        for s in seqs:
            eng.close(s)
        return ms / K, launches, ctx, ck

    ms_step, launches, ctx_end, clocks = time_decode(args.batch, ClockSampler())
    value = args.batch / (ms_step / 1e3)
    ctx_mid = ctx_end - K / 2.0
    bytes_step = wbytes + args.batch * ctx_mid * kv_per_token
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    points = {}
    if not args.no_points:
        for B in [int(b) for b in args.points.split(',') if b]:
            ms_b, _, _, _ = time_decode(B)
            points[f"decode_b{B}"] = B / (ms_b / 1e3)

    # ---- end to end through the Python entry point ------------------------------------------------
    # no request may reach its limit inside the timed steps: those that finish their prompt first decode while the others' prompts go in
    n_prompt_steps = (args.batch * P + 4095) // 4096 + args.batch
    sp = SamplingParams(top_k=1, max_tokens=K + W + n_prompt_steps + 4, ignore_eos=True)
    reqs = [llm.add_request(prompts[i], sp) for i in range(args.batch)]
    while any(len(r.output_token_ids) < 1 for r in reqs):
        llm.step()
    for _ in range(W):
        llm.step()
    torch.cuda.synchronize()
    h2d0, n_out0 = eng.runner.h2d_bytes, sum(len(r.output_token_ids) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(K):
        llm.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n_out = sum(len(r.output_token_ids) for r in reqs) - n_out0
    e2e = {"value": n_out / (t1 - t0), "unit": "tokens/s", "h2d_bytes_per_step": (eng.runner.h2d_bytes - h2d0) / K,
           "d2h_bytes_per_step": 4 * args.batch}
    while llm.scheduler.has_work():
        llm.step()

    rec = {
        "metric": "decode tok/s at batch 8 (MiniCPM4-8B sizes, one B200); prefill at 2,048 tokens and batch 1/64 in extra keys",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids",
        "config": {"model": "MiniCPM4-0.5B sizes" if args.sizes == "0.5b" else "MiniCPM4-8B sizes", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "prompt_len": P, "context": max(CONTEXT, P + 2 * (K + W) + 8),
                   "seq_len": int(ctx_end), "page_size": PAGE, "parallelism": "single GPU",
                   "cuda_graph": not args.no_graph, "l2": "inputs larger than L2 (weights 16 GB per step)",
                   "peaks": peak_src},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak},
        "points": points, "impl": "ours", "setup_s": round(time.time() - t_setup, 1),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
