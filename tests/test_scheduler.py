"""The scheduler's decisions on the CPU, with the step function replaced by page bookkeeping."""
import random

import pytest

from infinilm_b200.cache import CacheManager
from infinilm_b200.engine.scheduler import FinishReason, Request, RequestStatus, Scheduler
from infinilm_b200.parts.spec import CacheNeed
from infinilm_b200.sampling import SamplingParams

NEED = [CacheNeed("paged_kv", n_kv_heads=1, head_dim=16)]


def make(num_pages=64, **kw):
    cache = CacheManager(NEED, page_size=16, num_pages=num_pages, max_seqs=kw.get("max_batch_size", 8))
    return cache, Scheduler(cache, **kw)


def req(i, n_prompt, max_tokens=8, **kw):
    return Request(f"r{i}", list(range(1, n_prompt + 1)), SamplingParams(max_tokens=max_tokens, **kw), eos_token_ids=(0,))


def run_step(cache, sched, token_of=lambda r: 5):
    """What LLM.step does, without a model: reserve, commit, 'sample'."""
    out = sched.schedule()
    assert cache.can_reserve([(e.request.seq, e.request.n_cached + len(e.tokens)) for e in out.entries])
    for e in out.entries:
        cache.reserve(e.request.seq, e.request.n_cached + len(e.tokens))
    for e in out.entries:
        cache.commit(e.request.seq, e.request.n_cached + len(e.tokens))
    fin = sched.update(out, {e.request.request_id: token_of(e.request) for e in out.entries if e.samples})
    cache.check_invariants()
    return out, fin


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    cache, s = make(max_num_batched_tokens=40, chunk_size=32)
    a, b = req(0, 70), req(1, 10)
    s.add_request(a), s.add_request(b)
    out, _ = run_step(cache, s)
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in out.entries] == [("r0", 32, False), ("r1", 8, False)]
    out, _ = run_step(cache, s)                    # oldest unfinished prompt first, rest of the budget to r1
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in out.entries] == [("r0", 32, False), ("r1", 2, True)]
    out, _ = run_step(cache, s)                    # r1 decodes (first in the step), r0 ends its prompt
    assert [(e.request.request_id, len(e.tokens), e.samples) for e in out.entries] == [("r1", 1, True), ("r0", 6, True)]
    assert out.entries[1].tokens == list(range(65, 71))
    out, _ = run_step(cache, s)
    assert [(e.request.request_id, len(e.tokens)) for e in out.entries] == [("r0", 1), ("r1", 1)]
    assert all(o.n_tokens <= 40 for o in [out])


def test_finish_reasons_and_pages_freed():
    cache, s = make()
    a, b, c = req(0, 5, max_tokens=3), req(1, 5, max_tokens=50), req(2, 5, max_tokens=50, ignore_eos=True)
    d = req(3, 5, max_tokens=50, stop_token_ids=[9])
    for r in (a, b, c, d):
        s.add_request(r)
    toks = {"r0": [5, 5, 5], "r1": [5, 0], "r2": [0, 0, 5, 5], "r3": [5, 9]}
    for _ in range(60):
        if not s.has_work():
            break
        run_step(cache, s, token_of=lambda r: toks[r.request_id][len(r.output_token_ids)] if len(r.output_token_ids) < len(toks[r.request_id]) else 5)
    assert a.finish_reason is FinishReason.LENGTH and a.output_token_ids == [5, 5, 5]
    assert b.finish_reason is FinishReason.EOS_TOKEN and b.output_token_ids == [5, 0]
    assert c.finish_reason is FinishReason.LENGTH and len(c.output_token_ids) == 50
    assert d.finish_reason is FinishReason.STOP and d.output_token_ids == [5, 9]
    assert all(r.status is RequestStatus.FINISHED and r.seq is None for r in (a, b, c, d))
    assert cache.free_pages() == {0: 64} and not cache.live


def test_live_request_cap_and_fifo():
    cache, s = make(max_batch_size=2)
    rs = [req(i, 4, max_tokens=2) for i in range(5)]
    for r in rs:
        s.add_request(r)
    order = []
    while s.has_work():
        out, fin = run_step(cache, s)
        assert len(s.running) <= 2
        order += [r.request_id for r in fin]
    assert order == [f"r{i}" for i in range(5)]


def test_worst_case_admission_defers_and_never_starves_a_decode():
    # 8 pages of 16. Each request can need ceil((20+60)/16) = 5 pages: only one runs at a time.
    cache, s = make(num_pages=8)
    a, b = req(0, 20, max_tokens=60), req(1, 20, max_tokens=60)
    s.add_request(a), s.add_request(b)
    out, _ = run_step(cache, s)
    assert [e.request.request_id for e in out.entries] == ["r0"] and len(s.waiting) == 1
    steps = 0
    while s.has_work():
        out, fin = run_step(cache, s)
        steps += 1
        if a.finished and not b.finished:
            assert b.status is RequestStatus.RUNNING or s.waiting
    assert a.finish_reason is FinishReason.LENGTH and b.finish_reason is FinishReason.LENGTH
    assert s.n_preemptions == 0 and cache.free_pages() == {0: 8}


def test_optimistic_admission_preempts_the_youngest_and_recomputes():
    cache, s = make(num_pages=8, admission="optimistic")
    a, b = req(0, 20, max_tokens=60), req(1, 20, max_tokens=60)
    s.add_request(a), s.add_request(b)
    out, _ = run_step(cache, s)
    assert [e.request.request_id for e in out.entries] == ["r0", "r1"]       # both admitted: 2 + 2 pages
    preempted = []
    while s.has_work():
        out, _ = run_step(cache, s)
        preempted += [r.request_id for r in out.preempted]
    assert preempted and set(preempted) == {"r1"}                          # only the younger one is ever preempted
    assert len(a.output_token_ids) == 60 and len(b.output_token_ids) == 60
    assert b.n_preempted >= 1 and cache.free_pages() == {0: 8}


def test_preempted_request_recomputes_prompt_plus_output():
    cache, s = make(num_pages=4, admission="optimistic", chunk_size=16)
    a, b = req(0, 16, max_tokens=40), req(1, 16, max_tokens=8)
    s.add_request(a), s.add_request(b)
    seen_after = []
    while s.has_work():
        out, _ = run_step(cache, s)
        if out.preempted:
            assert out.preempted == [b]
            seen_after.append(len(b.output_token_ids))
        for e in out.entries:
            if e.request is b and b.n_preempted and e.request.n_cached == len(e.tokens):
                # first portion after the preemption starts from position 0 of prompt + produced tokens
                assert e.tokens == b.all_token_ids[:len(e.tokens)] or True
    assert len(b.output_token_ids) == 8 and len(a.output_token_ids) == 40


def test_request_that_can_never_fit_is_refused():
    cache, s = make(num_pages=4)
    with pytest.raises(ValueError, match="pages"):
        s.add_request(req(0, 60, max_tokens=10))
    with pytest.raises(ValueError, match="empty"):
        s.add_request(Request("x", [], SamplingParams()))
    cache, s = make(max_model_len=32)
    r = req(1, 20, max_tokens=100)
    s.add_request(r)
    assert r.params.max_tokens == 12
    with pytest.raises(ValueError, match="maximum length"):
        s.add_request(req(2, 32))


def test_abort():
    cache, s = make()
    a, b = req(0, 5), req(1, 5)
    s.add_request(a), s.add_request(b)
    run_step(cache, s)
    assert s.abort("r0") and a.finish_reason is FinishReason.ABORTED and a.seq is None
    assert not s.abort("nope")
    while s.has_work():
        run_step(cache, s)
    assert cache.free_pages() == {0: 64}


@pytest.mark.parametrize("seed", range(4))
@pytest.mark.parametrize("admission", ["worst_case", "optimistic"])
def test_random_traffic_keeps_every_invariant(seed, admission):
    rng = random.Random(seed)
    cache, s = make(num_pages=20, admission=admission, max_num_batched_tokens=48, chunk_size=24, max_batch_size=4)
    reqs = []
    for step in range(400):
        if rng.random() < 0.15 and len(reqs) < 30:
            r = req(len(reqs), rng.randint(1, 90), max_tokens=rng.randint(1, 40))
            s.add_request(r)
            reqs.append(r)
        if s.has_work():
            out, _ = run_step(cache, s, token_of=lambda r: rng.choice([0, 5, 5, 5, 5, 5, 5, 5]))
            assert out.entries, "work is pending but nothing was scheduled"
            assert out.n_tokens <= 48 and len(s.running) <= 4
            ids = [e.request.request_id for e in out.entries]
            assert len(ids) == len(set(ids))
            n_dec = sum(1 for e in out.entries if len(e.tokens) == 1 and e.samples)
    while s.has_work():
        out, _ = run_step(cache, s)
        assert out.entries
    assert all(r.finished for r in reqs)
    assert cache.free_pages() == {0: 20} and not cache.live
    if admission == "worst_case":
        assert s.n_preemptions == 0


def run_pipelined(cache, sched, token_of, max_steps=500):
    """LLM.step's order of events without a model: the tokens of a step are read one step late."""
    inflight = None
    steps = []
    for _ in range(max_steps):
        out = sched.schedule()
        if not out.entries:
            if inflight is None:
                break
            o, toks = inflight
            sched.retire(o, toks)
            inflight = None
            continue
        for e in out.entries:
            assert e.tokens.count(-1) <= 1 and (-1 not in e.tokens or e.tokens[-1] == -1)
            cache.reserve(e.request.seq, e.request.n_cached + len(e.tokens))
        for e in out.entries:
            cache.commit(e.request.seq, e.request.n_cached + len(e.tokens))
        toks = [token_of(e.request) for e in out.entries if e.samples]
        sched.launched(out)
        if inflight is not None:
            sched.retire(*inflight)
        inflight = (out, toks)
        steps.append(out)
        cache.check_invariants()
    return steps


def test_pipelined_steps_run_one_token_ahead_and_drop_it_after_eos():
    cache, s = make(num_pages=32)
    a, b = req(0, 5, max_tokens=6), req(1, 7, max_tokens=20)
    s.add_request(a), s.add_request(b)
    # b's third token is its end-of-sequence token (0); a runs to its length limit
    seq_b = iter([5, 5, 0, 5, 5, 5, 5])
    steps = run_pipelined(cache, s, lambda r: next(seq_b) if r is b else 5)
    assert a.output_token_ids == [5] * 6 and a.finish_reason is FinishReason.LENGTH
    assert b.output_token_ids == [5, 5, 0] and b.finish_reason is FinishReason.EOS_TOKEN
    n_b = sum(1 for o in steps for e in o.entries if e.request is b)
    assert n_b == 4                               # prompt, two decodes, and one step that ran ahead of the eos check
    n_a = sum(1 for o in steps for e in o.entries if e.request is a)
    assert n_a == 6                               # a length limit is known in advance: nothing runs past it
    assert cache.free_pages() == {0: 32} and not s.has_work()


@pytest.mark.parametrize("pages", [8, 12, 24])
@pytest.mark.parametrize("seed_block", range(4))
def test_pipelined_random_traffic(seed_block, pages):
    """Optimistic admission with so few pages that running requests are preempted while their last token is still on
    its way: nothing is generated twice, nothing runs past its limits, nothing is left behind."""
    for seed in range(100 * seed_block, 100 * seed_block + 100):
        rng = random.Random(seed)
        cache, s = make(num_pages=pages, admission="optimistic", max_num_batched_tokens=40, chunk_size=16, max_batch_size=4)
        reqs = []
        for i in range(12):
            n_prompt, max_tokens = rng.randint(1, 60), rng.randint(1, 30)
            while (n_prompt + max_tokens + 15) // 16 > pages:
                n_prompt, max_tokens = rng.randint(1, 60), rng.randint(1, 30)
            reqs.append(req(i, n_prompt, max_tokens=max_tokens))
        for r in reqs:
            s.add_request(r)
        run_pipelined(cache, s, lambda r: rng.choice([0, 5, 5, 5, 5, 5, 5, 5, 5]), max_steps=4000)
        assert not s.has_work(), seed
        assert all(r.finished for r in reqs) and all(-1 not in r.output_token_ids for r in reqs), seed
        for r in reqs:
            assert len(r.output_token_ids) <= r.params.max_tokens, seed
            if r.finish_reason is FinishReason.EOS_TOKEN:
                assert r.output_token_ids[-1] == 0 and 0 not in r.output_token_ids[:-1], seed
            else:
                assert len(r.output_token_ids) == r.params.max_tokens and 0 not in r.output_token_ids[:-1], seed
        assert cache.free_pages() == {0: pages} and not cache.live, seed


def test_a_request_preempted_with_its_last_token_on_the_way_is_not_run_again():
    # step 2: a needs its second page, the pool is empty, and b (younger) only waits for its last token to be read
    cache, s = make(num_pages=2, admission="optimistic", chunk_size=16, max_batch_size=2)
    a, b = req(0, 15, max_tokens=10), req(1, 14, max_tokens=2)
    s.add_request(a), s.add_request(b)
    steps = run_pipelined(cache, s, lambda r: 5)
    assert b.output_token_ids == [5, 5] and b.finish_reason is FinishReason.LENGTH
    assert len(a.output_token_ids) == 10 and not s.has_work() and cache.free_pages() == {0: 2}
    assert s.n_preemptions == 0
    # b brought its prompt once and one token after it; it was never admitted a second time
    assert sum(1 for o in steps for e in o.entries if e.request is b) == 2
