"""Runs InfiniLM's own Python control plane on the CPU and writes what it decided, step by step, to
`reference_scheduler_traces.json` beside this file. `tests/test_reference_parity.py` replays the same
traces through this package's cache manager and scheduler and compares where the two designs coincide.

    python tests/golden/make_reference_scheduler_traces.py /path/to/InfiniLM

InfiniLM's `python/infinilm/llm/{prefix_cache,sampling_params,cache_manager,request,scheduler}.py` are loaded by
file path under empty stand-in parent packages (importing the real `infinilm` package pulls in `infinicore`, which
is not installed), with a small stand-in for `janus.Queue` (the scheduler only uses `sync_q.put / get / get_nowait /
qsize`). No model runs: a step 'samples' token 5 for every scheduled request, and the loop around the scheduler is
that of `python/infinilm/llm/llm.py:143-176,178-276` (schedule, append one token per request, finish at max_tokens,
`complete_requests`).
"""
import importlib.util
import json
import logging
import os
import queue
import sys
import types


def load_reference(root):
    llm_dir = os.path.join(root, "python", "infinilm", "llm")

    class _SyncQ:
        def __init__(self):
            self.q = queue.Queue()

        def put(self, x):
            self.q.put(x)

        def get(self):
            return self.q.get()

        def get_nowait(self):
            return self.q.get_nowait()

        def qsize(self):
            return self.q.qsize()

    class _JanusQueue:
        def __init__(self):
            self.sync_q = _SyncQ()
            self.async_q = self.sync_q

    janus = types.ModuleType("janus")
    janus.Queue = _JanusQueue
    sys.modules["janus"] = janus
    for pkg in ("infinilm", "infinilm.llm"):
        m = types.ModuleType(pkg)
        m.__path__ = []
        sys.modules[pkg] = m
    mods = {}
    for name in ("prefix_cache", "sampling_params", "cache_manager", "request", "scheduler"):
        spec = importlib.util.spec_from_file_location(f"infinilm.llm.{name}", os.path.join(llm_dir, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"infinilm.llm.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def run_trace(mods, num_blocks, block_size, max_batch_size, max_num_batched_tokens, requests, arrivals=None, max_steps=400):
    """requests: list of (id, prompt_len, max_tokens); arrivals: step at which each is added (default 0)."""
    Scheduler = mods["scheduler"].Scheduler
    InferenceRequest = mods["request"].InferenceRequest
    FinishReason = mods["request"].FinishReason
    SamplingParams = mods["sampling_params"].SamplingParams
    s = Scheduler(max_batch_size=max_batch_size, num_blocks=num_blocks, block_size=block_size,
                  max_num_batched_tokens=max_num_batched_tokens, enable_prefix_caching=False)
    arrivals = arrivals or [0] * len(requests)
    reqs = {}
    steps = []
    for step in range(max_steps):
        for (rid, n_prompt, max_tokens), at in zip(requests, arrivals):
            if at == step:
                r = InferenceRequest(rid, prompt_token_ids=list(range(1, n_prompt + 1)),
                                     sampling_params=SamplingParams(max_tokens=max_tokens, ignore_eos=True))
                reqs[rid] = r
                s.add_request(r)
        out = s.schedule()
        if out is None:
            if all(r.is_finished() for r in reqs.values()) and len(reqs) == len(requests):
                break
            steps.append({"step": step, "scheduled": [], "usable_blocks": s.cache_manager.get_total_usable_blocks()})
            continue
        rec = {"step": step, "is_prefill": bool(out.is_prefill),
               "scheduled": [r.request_id for r in out.scheduled_requests],
               "block_tables": {r.request_id: list(r.block_table) for r in out.scheduled_requests},
               "slots": {r.request_id: list(r.slot_mapping) for r in out.scheduled_requests},
               "cached_before": {r.request_id: int(r.num_local_cached_tokens) for r in out.scheduled_requests}}
        # llm.py:190-276 without a model: one token per scheduled request, finish at max_tokens, complete_requests
        for r in out.scheduled_requests:
            r.append_generated_token_id(5)
            if r.get_num_generated_tokens() >= r.sampling_params.max_tokens:
                r.mark_finished(FinishReason.LENGTH)
        s.complete_requests(out.scheduled_requests)
        rec["finished"] = [r.request_id for r in out.scheduled_requests if r.is_finished()]
        rec["usable_blocks"] = s.cache_manager.get_total_usable_blocks()
        rec["waiting"] = s.waiting_queue.sync_q.qsize()
        steps.append(rec)
    return steps


TRACES = {
    # three prompts of 5, 17 and 33 tokens in 16 pages of 16: one prefill step, then decode steps
    "three_prompts": dict(num_blocks=16, block_size=16, max_batch_size=8, max_num_batched_tokens=1024,
                          requests=[("a", 5, 16), ("b", 17, 16), ("c", 33, 16)]),
    # 8 pages: each request can need 5, so the second one is deferred at admission until the first has finished
    "defer_at_admission": dict(num_blocks=8, block_size=16, max_batch_size=8, max_num_batched_tokens=1024,
                               requests=[("a", 20, 60), ("b", 20, 60)]),
    # pages of 4, a request that arrives while others decode, pages of a finished request handed out again
    "arrival_and_reuse": dict(num_blocks=24, block_size=4, max_batch_size=4, max_num_batched_tokens=1024,
                              requests=[("a", 6, 3), ("b", 9, 12), ("c", 14, 5), ("d", 30, 4)], arrivals=[0, 0, 2, 6]),
    # the token budget of a step defers the third prompt
    "token_budget": dict(num_blocks=32, block_size=16, max_batch_size=8, max_num_batched_tokens=48,
                         requests=[("a", 20, 4), ("b", 20, 4), ("c", 20, 4)]),
}


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    root = sys.argv[1]
    logging.disable(logging.WARNING)               # the scheduler logs every deferral
    mods = load_reference(root)
    out = {}
    for name, kw in TRACES.items():
        out[name] = {"setup": {k: v for k, v in kw.items()}, "steps": run_trace(mods, **kw)}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_scheduler_traces.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print(f"wrote {path}")


if __name__ == "__main__":
    main()
