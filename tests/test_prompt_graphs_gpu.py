"""Steps with prompt portions replayed as CUDA graphs: a step whose shape (single tokens, portions, their tokens,
block-table widths) has come back is captured and replayed; what it returns is compared with the plain implementation
and with the eager engine. Equal portions of one long prompt; portions of one request beside single tokens of others,
with so few pages that they are used again; a portion count that changes (another key, another graph)."""
import pytest
import torch

from replay_util import TOL, build_engine, first_bad_row, plain_logits
from tiny_configs import TINY, make_weights, random_ids

pytestmark = pytest.mark.gpu


def _rows(eng, entries):
    return eng.step(entries).clone()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed,portion", [("a", 0, 12), ("b", 1, 16), ("c", 2, 40), ("d", 3, 18)])
def test_equal_portions_are_replayed(cuda_device, name, seed, portion, dtype):
    from infinilm_b200.engine import StepEntry
    raw = TINY[name]()
    w = make_weights(raw, seed)
    eng = build_engine(raw, w, dtype, num_pages=48)
    eng.enable_graphs()
    n = portion * 9 + 5
    for trial in range(2):                        # the second prompt starts on pages the first one gave back
        ids = random_ids(n, raw["vocab_size"], 50 + trial)
        ref = plain_logits(raw, w, ids, dtype)
        seq = eng.open(("p", trial))
        got, at = [], []
        for a in range(0, n, portion):
            c = min(portion, n - a)
            got.append(_rows(eng, [StepEntry(seq, ids[a:a + c], [c - 1])]))
            at.append(a + c - 1)
        eng.close(seq)
        got = torch.cat(got, 0)
        bad = first_bad_row(got, ref[at], TOL[dtype])
        assert bad is None, f"{name} {dtype}: portion {bad} of {len(at)} differs from the plain implementation"
    assert eng.runner.portion_replays >= 8, "the equal portions were not replayed as graphs"
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("b", 4), ("c", 5)])
def test_portions_beside_single_tokens_are_replayed(cuda_device, name, seed, dtype):
    """Three requests decode one token a step while a fourth brings its prompt in equal portions; some portions want a
    row and some none; then two requests bring portions at once (another key). Every returned row against the plain
    implementation, and the whole run against the same engine without graphs, bit for bit in float32."""
    from infinilm_b200.engine import StepEntry
    raw = TINY[name]()
    w = make_weights(raw, seed)
    V = raw["vocab_size"]
    texts = {k: random_ids(n, V, 70 + i) for i, (k, n) in enumerate([("x", 60), ("y", 41), ("z", 23), ("long", 12 * 11 + 3), ("long2", 12 * 9)])}
    refs = {k: plain_logits(raw, w, ids, dtype) for k, ids in texts.items()}

    def run(graphs):
        eng = build_engine(raw, w, dtype, num_pages=40)
        if graphs:
            eng.enable_graphs()
        seqs = {k: eng.open(k) for k in texts}
        done = {k: 0 for k in texts}
        out = []
        for k, n0 in (("x", 30), ("y", 20), ("z", 5)):           # the three decoders' prompts, whole
            eng.step([StepEntry(seqs[k], texts[k][:n0], [])])
            done[k] = n0
        step_no = 0
        while done["long"] < len(texts["long"]) or done["long2"] < len(texts["long2"]):
            entries, who = [], []
            for k in ("long", "x", "long2", "y", "z"):            # portions and single tokens interleaved in the caller's order
                left = len(texts[k]) - done[k]
                if left <= 0:
                    continue
                if k.startswith("long"):
                    if k == "long2" and step_no < 6:
                        continue
                    c = min(12, left)
                    want = [c - 1] if (step_no % 3 != 1 or left <= 12) else []
                else:
                    c, want = 1, [0]
                entries.append(StepEntry(seqs[k], texts[k][done[k]:done[k] + c], want))
                who += [(k, done[k] + j) for j in want]
                done[k] += c
            rows = _rows(eng, entries)
            assert rows.shape[0] == len(who)
            out += [(k, at, rows[i]) for i, (k, at) in enumerate(who)]
            step_no += 1
        for s_ in seqs.values():
            eng.close(s_)
        eng.cache.check_invariants()
        return eng, out

    eng, got = run(True)
    assert eng.runner.portion_replays >= 6, "steps of the same shape were not replayed as graphs"
    for k, at, row in got:
        bad = first_bad_row(row[None], refs[k][at:at + 1], TOL[dtype])
        assert bad is None, f"{name} {dtype}: request {k} position {at} differs from the plain implementation"
    _, eager = run(False)
    assert [(k, at) for k, at, _ in got] == [(k, at) for k, at, _ in eager]
    if dtype == "float32":
        for (k, at, a), (_, _, b) in zip(got, eager):
            assert torch.equal(a, b), f"request {k} position {at}: the replayed step differs from the eager one"
