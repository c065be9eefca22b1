"""This package's cache manager and scheduler against InfiniLM's own Python classes (`BlockManager`, `Scheduler`),
where the two designs coincide: which pages a request gets and in what order, which requests a step holds, when a
request is deferred at admission, and how many pages are free after every step.

InfiniLM's classes were run on the CPU by `tests/golden/make_reference_scheduler_traces.py` (which loads
`python/infinilm/llm/{cache_manager,scheduler,request,...}.py` by file path; the script says how); what they decided is
in `tests/golden/reference_scheduler_traces.json`. Where the designs differ on purpose the comparison says so: InfiniLM
runs a step of prompts OR a step of decodes and never cuts a prompt (`scheduler.py:295-306`), here a step mixes both
and cuts prompts under the token budget, so step numbers shift while page tables do not.
"""
import json
import os

import pytest

from infinilm_b200.cache import CacheManager
from infinilm_b200.engine.scheduler import Request, Scheduler
from infinilm_b200.parts.spec import CacheNeed
from infinilm_b200.sampling import SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_scheduler_traces.json")) as f:
    GOLDEN = json.load(f)


def run_ours(setup, chunk_size=4096):
    """The same requests and arrivals through this package's scheduler (worst-case admission, InfiniLM's rule) and
    cache manager, with the step function replaced by page bookkeeping and token 5 'sampled' for every request."""
    cache = CacheManager([CacheNeed("paged_kv", n_kv_heads=1, head_dim=16)], page_size=setup["block_size"],
                         num_pages=setup["num_blocks"], max_seqs=setup["max_batch_size"])
    sched = Scheduler(cache, max_batch_size=setup["max_batch_size"], max_num_batched_tokens=setup["max_num_batched_tokens"],
                      chunk_size=chunk_size, admission="worst_case")
    arrivals = setup.get("arrivals") or [0] * len(setup["requests"])
    reqs, steps = {}, []
    for step in range(400):
        for (rid, n_prompt, max_tokens), at in zip(setup["requests"], arrivals):
            if at == step:
                reqs[rid] = Request(rid, list(range(1, n_prompt + 1)), SamplingParams(max_tokens=max_tokens, ignore_eos=True))
                sched.add_request(reqs[rid])
        if len(reqs) == len(setup["requests"]) and not sched.has_work():
            break
        out = sched.schedule()
        rec = {"step": step, "scheduled": [e.request.request_id for e in out.entries],
               "n_tokens": {e.request.request_id: len(e.tokens) for e in out.entries},
               "cached_before": {e.request.request_id: e.request.n_cached for e in out.entries}}
        for e in out.entries:
            cache.reserve(e.request.seq, e.request.n_cached + len(e.tokens))
        rec["block_tables"] = {e.request.request_id: list(e.request.seq.tables[0]) for e in out.entries}
        for e in out.entries:
            cache.commit(e.request.seq, e.request.n_cached + len(e.tokens))
        fin = sched.update(out, {e.request.request_id: 5 for e in out.entries if e.samples})
        cache.check_invariants()
        rec["finished"] = [r.request_id for r in fin]
        rec["free_pages"] = cache.free_pages()[0]
        steps.append(rec)
    return steps, reqs


def last_tables(steps):
    out = {}
    for s in steps:
        out.update(s.get("block_tables", {}))
    return out


def first_step_of(steps, rid):
    return next(s["step"] for s in steps if rid in s["scheduled"])


def test_three_prompts_step_by_step():
    """Prompts of 5, 17 and 33 tokens, 16 pages of 16: one step of whole prompts, then decode steps. Here the two
    designs make the same steps, so everything is compared step by step."""
    g = GOLDEN["three_prompts"]
    ours, _ = run_ours(g["setup"])
    ref = g["steps"]
    assert len(ours) == len(ref)
    for o, r in zip(ours, ref):
        assert o["scheduled"] == r["scheduled"]
        assert o["block_tables"] == r["block_tables"]
        assert o["cached_before"] == r["cached_before"]
        assert o["finished"] == r["finished"]
        assert o["free_pages"] == r["usable_blocks"]
    assert ref[0]["block_tables"] == {"a": [0], "b": [1, 2], "c": [3, 4, 5]}
    # slots: InfiniLM keeps a slot mapping (block * block_size + offset, `cache_manager.py:186-190`); here a token's
    # slot follows from the block table and its position - the same number
    bs = g["setup"]["block_size"]
    for r in ref:
        for rid, slots in r["slots"].items():
            first = r["cached_before"][rid]
            assert slots == [r["block_tables"][rid][(first + i) // bs] * bs + (first + i) % bs for i in range(len(slots))]


def test_deferred_at_admission_until_the_first_request_has_finished():
    g = GOLDEN["defer_at_admission"]
    ours, reqs = run_ours(g["setup"])
    ref = g["steps"]
    # the second request waits while the first can still need the pages, in both; it starts in the same step
    assert first_step_of(ours, "b") == first_step_of(ref, "b") == 60
    assert all(s["scheduled"] == ["a"] for s in ours[:60]) and all(s["scheduled"] == ["a"] for s in ref[:60])
    # pages come back first-in first-out in both: b starts on the pages a never used, then takes a's first ones
    assert last_tables(ours) == last_tables(ref)
    assert last_tables(ref)["b"] == [5, 6, 7, 0, 1]
    assert [s["free_pages"] for s in ours] == [s["usable_blocks"] for s in ref]
    assert len(ours) == len(ref)


def test_arrivals_while_others_decode_get_the_same_pages():
    """InfiniLM gives a newly arrived prompt a step of its own and lets the decoding requests wait; here they decode
    in the same step. The step numbers shift, the pages each request ends up with do not."""
    g = GOLDEN["arrival_and_reuse"]
    ours, reqs = run_ours(g["setup"])
    ref = g["steps"]
    mine, theirs = last_tables(ours), last_tables(ref)
    assert mine["a"] == theirs["a"] and mine["c"] == theirs["c"]
    # b and d both grow after d has arrived; since the steps have shifted by then, which of the two asks first for a
    # page differs. What each got at admission, and how many pages each holds in the end, is the same.
    assert mine["d"][:8] == theirs["d"][:8] == list(range(11, 19)) and len(mine["d"]) == len(theirs["d"])
    assert mine["b"][:4] == theirs["b"][:4] == [2, 3, 4, 9] and len(mine["b"]) == len(theirs["b"])
    ref_mixed = [s for s in ref if s["scheduled"]]
    assert any(s["is_prefill"] and s["step"] > 0 for s in ref_mixed)          # InfiniLM: a prefill-only step mid-run
    assert any(len(s["scheduled"]) > 1 and max(s["n_tokens"].values()) > 1 and min(s["n_tokens"].values()) == 1 for s in ours)
    assert len(ours) < len(ref)                                               # nobody waits for a prompt here
    assert ours[-1]["free_pages"] == ref[-1]["usable_blocks"] == g["setup"]["num_blocks"]
    for rid, r in reqs.items():
        assert len(r.output_token_ids) == r.params.max_tokens


def test_token_budget():
    """InfiniLM defers the prompt that would pass the budget whole (`scheduler.py:111-127`); here it is cut and its
    first portion fills what is left. Neither passes the budget; the pages are the same."""
    g = GOLDEN["token_budget"]
    budget = g["setup"]["max_num_batched_tokens"]
    ours, _ = run_ours(g["setup"])
    ref = g["steps"]
    assert ref[0]["scheduled"] == ["a", "b"] and ref[1]["scheduled"] == ["c"]
    assert ours[0]["scheduled"] == ["a", "b", "c"] and ours[0]["n_tokens"] == {"a": 20, "b": 20, "c": 8}
    assert all(sum(s["n_tokens"].values()) <= budget for s in ours)
    assert last_tables(ours) == last_tables(ref) == {"a": [0, 1], "b": [2, 3], "c": [4, 5]}
