"""Each part alone against the plain function for the same part: norm, position encoding, attention
mixer (over a real paged cache, with a window too), feed-forward, embedding and head. Sizes differ
from the tiny model configurations. Also an engine-level case where attention is made sharp, so that
single far keys among hundreds decide the output."""
import math

import pytest
import torch

import plain_model
from replay_util import TOL, build_engine, first_bad_row, plain_logits, rel_err, run_cut
from tiny_configs import make_weights, random_ids, tiny_c

pytestmark = pytest.mark.gpu

from infinilm_b200.cache import CacheManager, PagedKVView  # noqa: E402
from infinilm_b200.engine.step import StepContext, Workspace  # noqa: E402
from infinilm_b200.parts import PartSpec, build_part  # noqa: E402

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ctx(dtype, starts, qlens, device="cuda"):
    T, E = sum(qlens), len(qlens)
    order = sorted(range(E), key=lambda i: (qlens[i] != 1, i))
    assert order == list(range(E)), "give single-token entries first"
    tok_pos = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, qlens)]).int().to(device)
    tok_entry = torch.cat([torch.full((q,), e) for e, q in enumerate(qlens)]).int().to(device)
    qstart = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=device)
    kvlen = torch.tensor([s + q for s, q in zip(starts, qlens)], dtype=torch.int32, device=device)
    n_dec = sum(1 for q in qlens if q == 1)
    return StepContext(dtype=DT[dtype], T=T, n_entries=E, n_decode=n_dec, token_ids=torch.zeros(T, dtype=torch.int32, device=device),
                       tok_pos=tok_pos, tok_entry=tok_entry, entry_qstart=qstart, entry_kvlen=kvlen,
                       want_rows=torch.zeros(0, dtype=torch.int32, device=device), n_want=0, ws=Workspace(device, 512),
                       h_qlen=list(qlens), h_kvlen=[s + q for s, q in zip(starts, qlens)], max_qlen=max(qlens),
                       max_kvlen=max(s + q for s, q in zip(starts, qlens)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(cuda_device, dtype):
    H = 328
    norm = build_part("norm", PartSpec("rmsnorm", {"size": H, "eps": 3e-5}, "n"), DT[dtype])
    assert [(w.name, w.shape, w.role) for w in norm.weight_specs()] == [("weight", (H,), "vector")]
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.2 * torch.randn(H, generator=g)
    norm.set_weights({"weight": w.cuda()})
    resid = torch.randn(9, H, generator=g)
    branch = torch.randn(9, H, generator=g).to(DT[dtype])
    r = resid.cuda().clone()
    out = torch.empty(9, H, dtype=DT[dtype], device="cuda")
    norm.add_norm(r, branch.cuda(), 0.5, out)
    x = resid + 0.5 * branch.float()
    ref = plain_model.rms_norm(x, w, 3e-5)
    assert rel_err(out, ref) <= TOL[dtype] and rel_err(r, x) <= 1e-6


def test_position_parts():
    rope = build_part("position", PartSpec("rope", {"rot_dim": 24, "theta": 50000.0}), torch.float32)
    cfg = {"hidden_size": 48, "num_attention_heads": 1, "head_dim": 48, "partial_rotary_factor": 0.5, "rope_theta": 50000.0,
           "max_position_embeddings": 512}
    cos, _ = plain_model.rope_tables(cfg, torch.tensor([1.0]))
    rope.to_device("cpu")
    assert torch.allclose(torch.cos(rope.inv_freq), cos[0], atol=1e-7) and rope.mscale == 1.0 and rope.rot_dim == 24
    sf, lf = [1.0 + 0.1 * i for i in range(8)], [2.0 + 0.3 * i for i in range(8)]
    for mx, orig in ((256, 64), (64, 64)):
        lr = build_part("position", PartSpec("longrope", {"rot_dim": 16, "theta": 1e6, "short_factor": sf, "long_factor": lf,
                                                          "original_max_position_embeddings": orig, "max_position_embeddings": mx}),
                        torch.float32)
        lr.to_device("cpu")
        cfg = {"hidden_size": 16, "num_attention_heads": 1, "head_dim": 16, "rope_theta": 1e6, "max_position_embeddings": mx,
               "rope_scaling": {"rope_type": "longrope", "short_factor": sf, "long_factor": lf, "original_max_position_embeddings": orig}}
        cos, sin = plain_model.rope_tables(cfg, torch.tensor([7.0]))
        assert torch.allclose(torch.cos(7.0 * lr.inv_freq) * lr.mscale, cos[0], atol=1e-6)
        assert torch.allclose(torch.sin(7.0 * lr.inv_freq) * lr.mscale, sin[0], atol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 24])
def test_attention_part_over_a_paged_cache(cuda_device, dtype, window):
    """Two steps through the mixer alone: a prompt portion for two requests, then a single token for one beside a
    further portion of the other; compared with plain attention over the whole sequences."""
    H, nh, nkv, hd = 80, 6, 2, 32
    spec = PartSpec("attention", {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qkv_bias": True, "out_bias": True,
                                  "out_scale": 0.8, "window": window, "position": PartSpec("rope", {"rot_dim": 32, "theta": 10000.0})}, "a")
    att = build_part("mixer", spec, DT[dtype])
    g = torch.Generator().manual_seed(1)
    w = {ws.name: (torch.randn(ws.shape, generator=g) * (0.15 if ws.role == "matrix" else 0.05)).bfloat16().float() for ws in att.weight_specs()}
    att.set_weights({k: v.cuda() for k, v in w.items()})
    need = att.cache_need()
    assert need.kind == "paged_kv" and need.window == window and (need.n_kv_heads, need.head_dim) == (nkv, hd)
    cm = CacheManager([need], 16, 12, 4, device="cuda", dtype=DT[dtype])
    xs = {"a": torch.randn(40, H, generator=g).to(DT[dtype]), "b": torch.randn(21, H, generator=g).to(DT[dtype])}
    seqs = {k: cm.open(k) for k in xs}
    outs = {k: [] for k in xs}

    def step(parts):                               # parts: list of (request, n tokens), single-token entries first
        starts = [seqs[k].length for k, _ in parts]
        qlens = [n for _, n in parts]
        for (k, n) in parts:
            cm.reserve(seqs[k], seqs[k].length + n)
        ctx = _ctx(dtype, starts, qlens)
        W = max(len(seqs[k].tables[0]) for k, _ in parts)
        bt = torch.tensor([seqs[k].tables[0] + [-1] * (W - len(seqs[k].tables[0])) for k, _ in parts], dtype=torch.int32).cuda()
        x = torch.cat([xs[k][seqs[k].length: seqs[k].length + n] for k, n in parts]).cuda()
        y = att.forward(x, ctx, PagedKVView(cm.groups[0].storage[0], bt, 16, True, W)).clone()
        a = 0
        for k, n in parts:
            outs[k].append(y[a:a + n])
            a += n
            cm.commit(seqs[k], seqs[k].length + n)
    step([("a", 30), ("b", 20)])
    step([("b", 1), ("a", 10)])
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H, "rope_theta": 10000.0,
           "max_position_embeddings": 128}
    for k in xs:
        T = xs[k].shape[0]
        wk = {f"p.{n}": v for n, v in w.items()}
        ref = 0.8 * (plain_model.attention_block(cfg, {**wk, "p.o_proj.bias": torch.zeros(H)}, "p", xs[k].float(), torch.arange(T), window)) \
            + w["o_proj.bias"]
        got = torch.cat(outs[k])
        bad = first_bad_row(got, ref, TOL[dtype])
        assert bad is None, f"request {k}: first wrong position {bad}, rel err {rel_err(got, ref):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_with_a_position_encoding_that_is_no_rotary_table(cuda_device, dtype):
    """A position encoding defined here, in the test, that is not a rotation: q and k are scaled, dimension by
    dimension, by 1 + a * cos(position * b_i). It is registered as a part, changes q and k through the `transform` hook
    before the keys go into the cache, and the attention mixer and its kernels are used as they are."""
    from infinilm_b200.parts import PositionEncoding, register_part, unregister_part
    a_amp = 0.4

    def scales(pos, hd):
        b = 0.3 / (1.0 + torch.arange(hd, dtype=torch.float32, device=pos.device))
        return 1.0 + a_amp * torch.cos(pos.float()[:, None] * b[None, :])

    class CosScale(PositionEncoding):
        has_transform = True

        def __init__(self, params, prefix, dtype):
            super().__init__(params, prefix, dtype)
            self.rot_dim, self.mscale, self.inv_freq = 0, 1.0, None

        def transform(self, qkv, ctx, n_heads, n_kv_heads, head_dim):
            T = qkv.shape[0]
            v = qkv.view(T, -1, head_dim)[:, :n_heads + n_kv_heads]
            v.copy_((v.float() * scales(ctx.tok_pos, head_dim)[:, None, :]).to(qkv.dtype))
    register_part("position", "test_cos_scale", CosScale)
    try:
        H, nh, nkv, hd = 64, 4, 2, 32
        att = build_part("mixer", PartSpec("attention", {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd,
                                                        "position": PartSpec("test_cos_scale", {})}, "a"), DT[dtype])
        assert not att.graph_safe and not att.accepts_normed(1)      # the transform says nothing about graph replay
        g = torch.Generator().manual_seed(6)
        w = {ws.name: (torch.randn(ws.shape, generator=g) * 0.15).bfloat16().float() for ws in att.weight_specs()}
        att.set_weights({k: v.cuda() for k, v in w.items()})
        cm = CacheManager([att.cache_need()], 16, 8, 2, device="cuda", dtype=DT[dtype])
        T = 45
        x = torch.randn(T, H, generator=g).to(DT[dtype])
        seq = cm.open("r")
        outs = []
        for n in (30, 1, 14):                      # a portion, a single token, another portion
            start = seq.length
            cm.reserve(seq, start + n)
            bt = torch.tensor([list(seq.tables[0])], dtype=torch.int32).cuda()
            y = att.forward(x[start:start + n].cuda(), _ctx(dtype, [start], [n]),
                            PagedKVView(cm.groups[0].storage[0], bt, 16, True, bt.shape[1]))
            outs.append(y.clone())
            cm.commit(seq, start + n)
        xf = x.float()
        q = plain_model.linear(xf, w["q_proj.weight"]).view(T, nh, hd)
        k = plain_model.linear(xf, w["k_proj.weight"]).view(T, nkv, hd)
        v = plain_model.linear(xf, w["v_proj.weight"]).view(T, nkv, hd)
        sc = scales(torch.arange(T), hd)[:, None, :]
        ref = plain_model.linear(plain_model.attention_scores(q * sc, k * sc, v), w["o_proj.weight"])
        got = torch.cat(outs)
        bad = first_bad_row(got, ref, TOL[dtype])
        assert bad is None, f"first wrong position {bad}, rel err {rel_err(got, ref):.3e}"
    finally:
        unregister_part("position", "test_cos_scale")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [5, 40])
def test_swiglu_part(cuda_device, dtype, T):
    H, I = 72, 200
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden": H, "intermediate": I, "bias": True, "out_scale": 1.0}, "m"), DT[dtype])
    g = torch.Generator().manual_seed(2)
    w = {ws.name: (torch.randn(ws.shape, generator=g) * 0.2).bfloat16().float() for ws in ffn.weight_specs()}
    ffn.set_weights({k: v.cuda() for k, v in w.items()})
    x = torch.randn(T, H, generator=g).to(DT[dtype])
    y = ffn.forward(x.cuda(), _ctx(dtype, [0], [T]))
    ref = plain_model.swiglu_mlp({f"p.{k}": v for k, v in w.items()}, "p", x.float())
    assert rel_err(y, ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(cuda_device, dtype):
    V, H = 211, 88
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab": V, "hidden": H, "scale": 7.0}, "e"), DT[dtype])
    head = build_part("head", PartSpec("linear_head", {"vocab": V, "hidden": H, "scale": 0.25, "tied_to": "e.weight"}, "h"), DT[dtype])
    assert head.weight_specs()[0].fallback == "e.weight"
    g = torch.Generator().manual_seed(3)
    table = (torch.randn(V, H, generator=g) * 0.1).bfloat16().float()
    emb.set_weights({"weight": table.cuda()})
    head.set_weights({"weight": emb.table})
    ids = torch.randint(0, V, (13,), generator=g)
    resid = torch.empty(13, H, device="cuda")
    emb.forward(ids.int().cuda(), resid)
    assert torch.equal(resid.cpu(), plain_model.embed(ids, table, 7.0, dtype == "bfloat16"))
    x = torch.randn(13, H, generator=g).to(DT[dtype])
    logits = torch.empty(13, V, device="cuda")
    head.forward(x.cuda(), logits)
    ref = plain_model.linear(x.float(), table, None, 0.25)
    assert logits.dtype == torch.float32 and rel_err(logits, ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_far_keys(cuda_device, dtype):
    """Query and key projections scaled up so that softmax picks single keys: with 500 tokens and pages of 16,
    a key that is lost, misplaced or read from a stale page changes the logits visibly. The factor is 12 in
    float32 (scores x144). In bfloat16 it is 5: a score of magnitude s carries a rounding error near s/256 from
    the rounded q and k alone, and at x144 that error by itself moves the softmax - the comparison would test
    the conditioning of the problem, not the kernels."""
    raw = tiny_c()
    w = dict(make_weights(raw, 4))
    sharp = 12 if dtype == "float32" else 5
    for k in list(w):
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = (w[k].float() * sharp).bfloat16().to(w[k].dtype)
    ids = random_ids(500, raw["vocab_size"], 5)
    ref = plain_logits(raw, w, ids, dtype)
    eng = build_engine(raw, w, dtype, num_pages=40, max_batch_tokens=512)
    for cuts in ([500], [468] + [1] * 32, [129, 2, 200, 7, 1, 161]):
        got = run_cut(eng, ids, cuts)
        bad = first_bad_row(got, ref, TOL[dtype])
        assert bad is None, f"cuts {cuts[:3]}..: first wrong position {bad}, rel err {rel_err(got, ref):.3e}"


@pytest.mark.parametrize("name", ["c", "d"])
@pytest.mark.parametrize("cuts", [[9, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], [20, 3, 2, 5, 16, 1]])
def test_block_with_and_without_the_norm_in_its_products(cuda_device, cuts, name):
    """The arrangement's two ways through a step of few rows - add+norm as kernels of their own, or the product before
    adding into the residual and the product after dividing by the rms - against the plain model, and the fused way
    with as many launches fewer as there are norms between two parts that can. Portions of 17 rows and more take the
    kernels either way. Configuration c rotates half of a head (its q/k/v product does not take the norm), d all of it."""
    from infinilm_b200 import ops
    from infinilm_b200.parts.blocks import PreNormResidual
    from tiny_configs import TINY
    raw = TINY[name]()
    w = make_weights(raw, 5)
    ids = random_ids(sum(cuts), raw["vocab_size"], 77)
    ref = plain_logits(raw, w, ids, "bfloat16")
    was = PreNormResidual.FUSE_NORM
    got, launches = {}, {}
    try:
        for fuse in (False, True):
            PreNormResidual.FUSE_NORM = fuse
            eng = build_engine(raw, w, "bfloat16")
            n0 = ops.launch_count()
            got[fuse] = run_cut(eng, ids, cuts)
            launches[fuse] = ops.launch_count() - n0
        model, saved = eng.model, 0
        for T in cuts:
            for i, st in enumerate(model.order):
                blk = model.blocks[st.layer]
                nxt = model.blocks[model.order[i + 1].layer] if i + 1 < len(model.order) else None
                saved += int(blk.mixer.fuses_tail(T) and blk.ffn.accepts_normed(T))
                saved += int(nxt is not None and nxt.accepts_normed_input(T) and blk.ffn.fuses_tail(T))
    finally:
        PreNormResidual.FUSE_NORM = was
    for fuse in (False, True):
        bad = first_bad_row(got[fuse], ref, TOL["bfloat16"])
        assert bad is None, f"fuse={fuse}: first wrong position {bad} (rel err {rel_err(got[fuse][bad], ref[bad]):.2e})"
    small = sum(1 for c in cuts if c <= ops.SKINNY_MAX_ROWS)
    L = raw["num_hidden_layers"]
    assert saved == small * (L if name == "c" else 2 * L - 1)
    assert launches[False] - launches[True] == saved
