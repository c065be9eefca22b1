"""The engine against the plain implementation under every way of cutting the work:
whole prompts; most of it in one step and the last 32 tokens one by one; portions of changing
size down to two tokens; up to four live requests mixed, with so few pages that they are used
again. In float32 and in bfloat16, on tiny configurations that differ in every size and option."""
import pytest
import torch

import plain_model
from replay_util import TOL, build_engine, first_bad_row, plain_logits, rel_err, run_cut, run_schedule
from tiny_configs import TINY, make_weights, random_ids

pytestmark = pytest.mark.gpu

CASES = [("a", 0), ("b", 1), ("c", 2), ("d", 3)]
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"a": [5, 17, 33, 100], "b": [3, 40, 70, 100, 200], "c": [2, 31, 64, 129], "d": [4, 65, 130, 300]}


def _setup(name, seed):
    raw = TINY[name]()
    return raw, make_weights(raw, seed)


def _check(got, ref, dtype, what):
    err = rel_err(got, ref)
    bad = first_bad_row(got, ref, TOL[dtype])
    assert bad is None, f"{what}: first wrong position {bad} of {got.shape[0]}, rel err {err:.3e} > {TOL[dtype]:.1e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_whole_prompts(cuda_device, name, seed, dtype):
    raw, w = _setup(name, seed)
    eng = build_engine(raw, w, dtype)
    for n in LENGTHS[name]:
        ids = random_ids(n, raw["vocab_size"], 100 + n)
        got = run_cut(eng, ids, [n])
        _check(got, plain_logits(raw, w, ids, dtype), dtype, f"{name} whole prompt of {n}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_last_32_one_by_one(cuda_device, name, seed, dtype):
    raw, w = _setup(name, seed)
    eng = build_engine(raw, w, dtype)
    n = LENGTHS[name][-1]
    ids = random_ids(n, raw["vocab_size"], 7)
    got = run_cut(eng, ids, [n - 32] + [1] * 32)
    ref = plain_logits(raw, w, ids, dtype)
    _check(got, ref, dtype, f"{name} prompt {n - 32} then 32 single tokens")
    whole = run_cut(eng, ids, [n])
    # decoding against prefill of the same engine: the same up to rounding
    assert rel_err(got, whole) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_changing_portions(cuda_device, name, seed, dtype):
    raw, w = _setup(name, seed)
    eng = build_engine(raw, w, dtype)
    n = LENGTHS[name][-1]
    ids = random_ids(n, raw["vocab_size"], 11)
    pattern = [16, 7, 2, 5, 3, 17, 2, 1, 31, 2, 9]
    cuts, left, i = [], n, 0
    while left > 0:
        c = min(pattern[i % len(pattern)], left)
        cuts.append(c)
        left -= c
        i += 1
    got = run_cut(eng, ids, cuts)
    _check(got, plain_logits(raw, w, ids, dtype), dtype, f"{name} portions {cuts[:8]}...")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_mixed_requests_pages_reused(cuda_device, name, seed, dtype):
    """Four live requests at most, portions of some beside single tokens of others, and a pool so
    small that pages of finished requests are handed out again (they are not cleared)."""
    raw, w = _setup(name, seed)
    V = raw["vocab_size"]
    lens = {"p": 3, "q": 40, "r": 70, "s": 100, "t": 55, "u": 90}
    reqs = {k: random_ids(n, V, 50 + i) for i, (k, n) in enumerate(lens.items())}
    sched = [
        [("p", 3), ("q", 16)],
        [("q", 16), ("r", 16), ("s", 2)],
        [("q", 7), ("r", 16), ("s", 16)],                       # q: 39 done
        [("q", 1), ("r", 1), ("s", 16), ("t", 16)],              # q ends; t starts beside decodes
        [("r", 1), ("s", 30), ("t", 1), ("u", 5)],
        [("r", 36), ("s", 1), ("t", 2), ("u", 1)],               # r ends (16+16+1+1+36 = 70)
        [("s", 35), ("t", 36), ("u", 20)],                       # s: 100 done; t: 55 done
        [("u", 1)], [("u", 1)], [("u", 30)], [("u", 32)],
    ]
    # pages of 16: at most 14 are held at once, 26 are allocated over the run: a pool of 16 forces reuse
    eng = build_engine(raw, w, dtype, num_pages=16)
    got = run_schedule(eng, reqs, sched)
    for k, ids in reqs.items():
        _check(got[k], plain_logits(raw, w, ids, dtype), dtype, f"{name} mixed request {k}")
    assert not eng.cache.live
    assert eng.cache.free_pages() == {0: 16}


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(cuda_device, dtype):
    """A short prompt and then many single tokens, crossing LongRoPE's original maximum and many pages."""
    raw, w = _setup("b", 5)
    eng = build_engine(raw, w, dtype)
    ids = random_ids(250, raw["vocab_size"], 3)
    got = run_cut(eng, ids, [4] + [1] * 246)
    _check(got, plain_logits(raw, w, ids, dtype), dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(cuda_device, dtype):
    """The first tokens of a sequence: a single token, and two."""
    raw, w = _setup("a", 9)
    eng = build_engine(raw, w, dtype)
    for n in (1, 2):
        ids = random_ids(n, raw["vocab_size"], 40 + n)
        _check(run_cut(eng, ids, [n]), plain_logits(raw, w, ids, dtype), dtype, f"first {n} token(s)")
        _check(run_cut(eng, ids, [1] * n), plain_logits(raw, w, ids, dtype), dtype, f"first {n} token(s) one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", [("b", 1), ("d", 3)])
@pytest.mark.parametrize("page_size,num_pages", [(32, 9), (256, 4), (4, 60)])
def test_mixed_requests_at_other_page_sizes(cuda_device, name, seed, dtype, page_size, num_pages):
    """The mixed schedule with pages of 32 and 256 tokens (runs of kernel pages of 16: the fast kernels stay in use)
    and of 4 (smaller than the kernels' tile: the plain kernels), each with a pool that forces pages to be used again."""
    import warnings
    raw, w = _setup(name, seed)
    V = raw["vocab_size"]
    lens = {"p": 3, "q": 40, "r": 70, "s": 100, "t": 55, "u": 90}
    reqs = {k: random_ids(n, V, 50 + i) for i, (k, n) in enumerate(lens.items())}
    sched = [
        [("p", 3), ("q", 16)],
        [("q", 16), ("r", 16), ("s", 2)],
        [("q", 7), ("r", 16), ("s", 16)],
        [("q", 1), ("r", 1), ("s", 16), ("t", 16)],
        [("r", 1), ("s", 30), ("t", 1), ("u", 5)],
        [("r", 36), ("s", 1), ("t", 2), ("u", 1)],
        [("s", 35), ("t", 36), ("u", 20)],
        [("u", 1)], [("u", 1)], [("u", 30)], [("u", 32)],
    ]
    with warnings.catch_warnings():
        if page_size >= 16:
            warnings.filterwarnings("error", message="attention:")
        else:
            warnings.filterwarnings("ignore", message="attention:")
        eng = build_engine(raw, w, dtype, num_pages=num_pages, page_size=page_size)
        assert eng.cache.kernel_page == min(page_size, 16)
        got = run_schedule(eng, reqs, sched)
    for k, ids in reqs.items():
        _check(got[k], plain_logits(raw, w, ids, dtype), dtype, f"{name} mixed request {k}, pages of {page_size}")
    assert not eng.cache.live and eng.cache.free_pages() == {0: num_pages}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_hidden_states_layer_by_layer(cuda_device, name, seed, dtype):
    """The residual stream after every layer, taken through the step function's tap, against the plain
    implementation's, for a whole prompt and for the same tokens cut into portions: a wrong scale, page or norm in
    one layer is named, not just seen in the logits. (InfiniLM: hooks on intermediate tensors,
    `csrc/debug_utils/hooks.hpp:31-62`, compared layer by layer in `test/models/llama/test_intermediate_validation.py:758-812`.)"""
    raw, w = _setup(name, seed)
    eng = build_engine(raw, w, dtype)
    n = LENGTHS[name][-2]
    ids = random_ids(n, raw["vocab_size"], 21)
    _, hidden = plain_model.forward(raw, w, ids, round_embedding_bf16=(dtype == "bfloat16"), return_hidden=True)
    L = raw["num_hidden_layers"]
    for cuts in ([n], [n - 9, 1, 2, 1, 5]):
        seen = {i: [] for i in range(L)}

        def tap(label, resid, pending):
            assert label.startswith("layer")
            h = resid.float().clone()
            if pending is not None:
                branch, scale = pending
                h += scale * branch.float()
            seen[int(label[5:])].append(h.cpu())
        eng.runner.tap = tap
        try:
            run_cut(eng, ids, cuts)
        finally:
            eng.runner.tap = None
        for i in range(L):
            got = torch.cat(seen[i], 0)
            bad = first_bad_row(got, hidden[i + 1], TOL[dtype])
            assert bad is None, f"{name} layer {i}, cuts {cuts}: first wrong position {bad}, rel err {rel_err(got, hidden[i + 1]):.3e}"


def test_step_refuses_batches_that_cannot_be_run(cuda_device):
    """What the step function checks on the host before anything is launched (these checks stand where a memory checker
    would): a request twice in a step, no token, a token id outside the vocabulary, a token that is said to be on the device
    when nothing is, a wanted place outside the entry's tokens, a step beyond the token budget or the model's maximum
    length, more pages than the pool has. After every refusal the cache is as it was."""
    from infinilm_b200.cache import OutOfPages
    from infinilm_b200.engine import StepEntry
    from infinilm_b200.engine.step import StepError
    raw, w = _setup("a", 0)
    eng = build_engine(raw, w, "float32", num_pages=4, max_batch_tokens=40)
    V = raw["vocab_size"]
    a, b = eng.open("a"), eng.open("b")
    cases = [
        ([StepEntry(a, [1, 2], [0]), StepEntry(a, [3], [0])], StepError, "twice"),
        ([StepEntry(a, [], [])], StepError, "no token"),
        ([StepEntry(a, [1, V], [0])], StepError, "outside"),
        ([StepEntry(a, [1, -1], [0])], StepError, "outside"),
        ([StepEntry(a, [1, 2, 3], [3])], StepError, "wanted place"),
        ([StepEntry(a, [1] * 30, []), StepEntry(b, [2] * 11, [])], StepError, "max_batch_tokens"),
        ([StepEntry(a, [1] * 40, []), ], None, None),                                     # fine: 40 tokens, 3 pages
        ([StepEntry(b, [1] * 33, [])], OutOfPages, "pages"),                              # 3 more pages, 1 is free
    ]
    for entries, exc, word in cases:
        before = (a.length, b.length, eng.cache.free_pages())
        if exc is None:
            eng.step(entries)
            continue
        with pytest.raises(exc, match=word):
            eng.step(entries)
        assert (a.length, b.length, eng.cache.free_pages()) == before
        eng.cache.check_invariants()
    with pytest.raises(StepError, match="device token"):
        eng.step([StepEntry(b, [-5], [0])], device_tokens=torch.zeros(2, dtype=torch.int32, device="cuda"))
    eng.close(a), eng.close(b)
    c = eng.open("c")
    eng2 = build_engine(raw, w, "float32", num_pages=16, max_batch_tokens=200)
    d = eng2.open("d")
    eng2.step([StepEntry(d, [1] * 120, [])])
    with pytest.raises(StepError, match="max_position_embeddings"):
        eng2.step([StepEntry(d, [1] * 9, [])])                                            # 129 > 128
    eng.close(c), eng2.close(d)
