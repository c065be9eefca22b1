"""The native host code that fills a step's descriptors (`csrc/step_fill.cpp`) against a plain construction in Python,
over random batches: single tokens and portions mixed, tokens that are still on the device, wanted places, block tables
of pages that are runs of kernel pages, padding rows of a replayed step. Runs on the CPU (the code is host code)."""
import random

import numpy as np
import pytest

from infinilm_b200 import ops
from infinilm_b200.cache.manager import PageTable


def _case(rng):
    E, sub = rng.randint(1, 9), rng.choice([1, 2, 16])
    graph = rng.random() < 0.4                    # a step laid out for replay: padding entries, a fixed number of wanted rows
    only_single = graph and rng.random() < 0.5
    n_tok = np.array([1 if only_single or rng.random() < 0.5 else rng.randint(2, 7) for _ in range(E)], dtype=np.int32)
    start = np.array([rng.randint(0, 40) for _ in range(E)], dtype=np.int32)
    slot = np.array(rng.sample(range(1, 20), E), dtype=np.int32)
    fresh = np.array([rng.random() < 0.3 for _ in range(E)], dtype=np.uint8)
    toks = [[rng.choice([rng.randint(0, 99), -1 - rng.randint(0, 5)]) for _ in range(n)] for n in n_tok]
    wants = [([0] if n == 1 else rng.choice([[], [rng.randrange(n)]])) if graph else sorted(rng.sample(range(n), rng.randint(0, n)))
             for n in n_tok]
    tables = []
    for i in range(E):
        t = PageTable(sub=sub)
        for _ in range((int(start[i] + n_tok[i]) + 15) // 16):
            t.append(rng.randint(0, 50))
        tables.append(t)
    return E, sub, graph, n_tok, start, slot, fresh, toks, wants, tables


@pytest.mark.parametrize("seed", range(5))
def test_native_filler_equals_a_plain_construction(seed):
    rng = random.Random(seed)
    for _ in range(60):
        E, sub, graph, n_tok, start, slot, fresh, toks, wants, tables = _case(rng)
        order = np.argsort(n_tok != 1, kind="stable").astype(np.int32)
        T = int(n_tok.sum())
        n_pad = rng.randint(0, 3) if graph else 0
        Ep, Tp = E + n_pad, T + n_pad
        n_single = int((n_tok == 1).sum())        # the padding entries run behind the single tokens
        n_want_fixed = Ep if graph else -1
        tokens = np.array([t for row in toks for t in row], dtype=np.int64)
        tok_off = np.zeros(E + 1, np.int32)
        np.cumsum(n_tok, out=tok_off[1:])
        want_off = np.zeros(E + 1, np.int32)
        np.cumsum(np.array([len(w) for w in wants], np.int32), out=want_off[1:])
        want = np.array([w for row in wants for w in row], dtype=np.int32)
        tbl_len = np.array([[len(t) * sub for t in tables]], dtype=np.int32)
        tbl_ptr = np.array([[t.address() for t in tables]], dtype=np.uint64)
        W = max(1, int(tbl_len.max())) + rng.randint(0, 2)
        n_patch = Tp if graph else int((tokens < 0).sum())
        out = np.full(40000, 777, dtype=np.int32)
        offs, outs = np.zeros(12, np.int32), np.zeros(3, np.int32)
        rc = ops.step_fill(out, out.size, E, Ep, Tp, order, n_tok, start, slot, fresh, tokens, tok_off, np.array([W], np.int32), tbl_ptr,
                           tbl_len, np.array([99 * sub], np.int32), 31, want, want_off, n_single, n_want_fixed, n_patch, offs, outs)
        assert rc == 0
        o = offs.tolist()
        qs, tok, pos, ent, kv, rs, ws, bt, pr, ps, first_row = [0], [], [], [], [], [], [], [], [], [], {}
        running = order.tolist()
        running = running[:n_single] + [None] * n_pad + running[n_single:]
        for k, i in enumerate(running):
            if i is None:                         # a padding entry of a replayed step
                tok.append(0), pos.append(0), ent.append(k), qs.append(qs[-1] + 1), kv.append(1), rs.append(0), ws.append(31)
                bt.append([99 * sub] + [-1] * (W - 1))
                continue
            first_row[i] = qs[-1]
            for j, t in enumerate(toks[i]):
                if t < 0:
                    pr.append(qs[-1] + j)
                    ps.append(-1 - t)
                tok.append(max(t, 0))
                pos.append(int(start[i]) + j)
                ent.append(k)
            qs.append(qs[-1] + int(n_tok[i]))
            kv.append(int(start[i] + n_tok[i]))
            rs.append(0 if fresh[i] else int(slot[i]))
            ws.append(int(slot[i]))
            row = tables[i].array().tolist()
            bt.append(row + [-1] * (W - len(row)))
        wr = [first_row[i] + w for i in range(E) for w in wants[i]]
        if graph:
            wr += [0] * (Ep - len(wr))
        assert out[o[0]:o[0] + Tp].tolist() == tok and out[o[1]:o[1] + Tp].tolist() == pos and out[o[2]:o[2] + Tp].tolist() == ent
        assert out[o[3]:o[3] + Ep + 1].tolist() == qs and out[o[4]:o[4] + Ep].tolist() == kv
        assert out[o[5]:o[5] + len(wr)].tolist() == wr and outs[1] == len(wr)
        assert out[o[6]:o[6] + Ep].tolist() == rs and out[o[7]:o[7] + Ep].tolist() == ws
        assert out[o[8]:o[8] + Ep * W].reshape(Ep, W).tolist() == bt
        assert outs[0] == len(pr) and out[o[9]:o[9] + len(pr)].tolist() == pr and out[o[10]:o[10] + len(pr)].tolist() == ps
        assert o[11] == 3 * Tp + Ep + 1 + Ep + max(len(wr), 1) + 2 * Ep + Ep * W + 2 * n_patch
        assert (out[o[11]:] == 777).all()            # nothing written behind the end


def test_native_filler_reports_what_is_wrong():
    t = PageTable()
    for p in (3, 4):
        t.append(p)
    one = dict(order=np.zeros(1, np.int32), n_tok=np.array([3], np.int32), start=np.array([20], np.int32), slot=np.array([1], np.int32),
               fresh=np.zeros(1, np.uint8), tokens=np.array([5, 6, 7], np.int64), tok_off=np.array([0, 3], np.int32))
    tbl_ptr, tbl_len = np.array([[t.address()]], np.uint64), np.array([[2]], np.int32)
    out, offs, outs = np.zeros(200, np.int32), np.zeros(12, np.int32), np.zeros(3, np.int32)

    def fill(want, widths=(2,), cap=200, n_patch=0, tokens=None):
        a = dict(one)
        if tokens is not None:
            a["tokens"] = np.array(tokens, np.int64)
        return ops.step_fill(out, cap, 1, 1, 3, a["order"], a["n_tok"], a["start"], a["slot"], a["fresh"], a["tokens"], a["tok_off"],
                             np.array(widths, np.int32), tbl_ptr, tbl_len, np.array([9], np.int32), 7, np.array(want, np.int32),
                             np.array([0, len(want)], np.int32), 0, -1, n_patch, offs, outs)
    assert fill([0, 2]) == 0
    assert fill([3]) == -11 and outs[2] == 0         # a wanted place outside the entry's tokens
    assert fill([0], widths=(1,)) == -12 and outs[2] == 0
    assert fill([0], cap=10) == -13
    assert fill([0], tokens=[5, -1, 7], n_patch=0) == -14
    with pytest.raises(ops.KernelError):
        ops.step_fill(out.astype(np.int64), 200, 1, 1, 3, one["order"], one["n_tok"], one["start"], one["slot"], one["fresh"], one["tokens"],
                      one["tok_off"], np.array([2], np.int32), tbl_ptr, tbl_len, np.array([9], np.int32), 7, np.array([0], np.int32),
                      np.array([0, 1], np.int32), 0, -1, 0, offs, outs)
