"""Each kernel alone against a plain float32 reference in torch, at sizes other than the engine's:
head sizes in steps of 16, odd numbers of heads and groups, widths and vocabularies that are no
power of two, and inputs built so that a fault shows (one far key that dominates, a window's
edge, a page's edge)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from infinilm_b200 import ops  # noqa: E402

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def close(got, ref, dtype, scale=None):
    """Row by row (a row = the last dimension): the largest error of a row against the largest magnitude of that row
    of the reference, so that a row of small values that is wrong throughout does not hide behind a large one."""
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    got, ref = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
    denom = ref.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6) if scale is None else scale
    err = ((got - ref).abs() / denom).amax(dim=-1)
    bad = torch.nonzero(~(err <= TOL[dtype]))
    assert bad.numel() == 0, f"row {int(bad[0])}: rel err {float(err[int(bad[0])]):.3e} > {TOL[dtype]:.1e} ({bad.numel()} of {err.numel()} rows)"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,V", [(1, 64, 97), (37, 200, 331), (5, 4096, 1000)])
def test_embedding(cuda_device, dtype, T, H, V):
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(V, H, device="cuda", generator=g).to(DT[dtype])
    ids = torch.randint(0, V, (T,), device="cuda", generator=g, dtype=torch.int32)
    out = torch.empty(T, H, device="cuda")
    ops.embed(ids, table, 12.5, out, round_bf16=(dtype == "bfloat16"))
    ref = table.float()[ids.long()] * 12.5
    if dtype == "bfloat16":
        ref = ref.bfloat16().float()
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 64), (33, 200), (7, 4096), (3, 5120 + 16)])
def test_add_rmsnorm(cuda_device, dtype, T, H):
    g = torch.Generator(device="cuda").manual_seed(1)
    resid = torch.randn(T, H, device="cuda", generator=g) * 3
    branch = torch.randn(T, H, device="cuda", generator=g).to(DT[dtype])
    w32 = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    for w in (w32, w32.bfloat16()):
        r = resid.clone()
        out = torch.empty(T, H, device="cuda", dtype=DT[dtype])
        ops.add_rmsnorm(r, branch, 0.37, w, 1e-5, out)
        x = resid + 0.37 * branch.float()
        ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        assert torch.allclose(r, x, rtol=0, atol=1e-6)
        close(out, ref, dtype)
    # without a branch, and on chosen rows only (the residual stays as it is)
    r = resid.clone()
    rows = torch.tensor([T - 1, 0], device="cuda", dtype=torch.int32)
    out = torch.empty(2, H, device="cuda", dtype=DT[dtype])
    ops.add_rmsnorm(r, branch, 2.0, w32, 1e-6, out, rows)
    x = (resid + 2.0 * branch.float())[rows.long()]
    close(out, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w32, dtype)
    assert torch.equal(r, resid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_and_bias(cuda_device, dtype):
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = (torch.randn(19, 2 * 264, device="cuda", generator=g) * 4).to(DT[dtype])
    out = torch.empty(19, 264, device="cuda", dtype=DT[dtype])
    ops.swiglu(gu, out)
    a, b = gu.float()[:, :264], gu.float()[:, 264:]
    close(out, torch.nn.functional.silu(a) * b, dtype)
    y = torch.randn(19, 331, device="cuda", generator=g).to(DT[dtype])
    bias = torch.randn(331, device="cuda", generator=g)
    ref = y.float() + bias
    ops.add_bias(y, bias)
    close(y, ref, dtype)


@pytest.mark.parametrize("M,N,K", [(1, 97, 64), (5, 331, 200), (16, 256, 264), (17, 300, 48), (64, 129, 1000), (200, 513, 333)])
def test_gemm_f32(cuda_device, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g)
    b = torch.randn(N, device="cuda", generator=g)
    out = torch.empty(M, N, device="cuda")
    ops.gemm_f32(a, w, out, 0.7, b)
    ref = 0.7 * (a.double() @ w.double().t()) + b.double()
    close(out, ref.float(), "float32")
    # a row's result is bit-identical whatever the batch around it (another tile shape)
    out1 = torch.empty(1, N, device="cuda")
    ops.gemm_f32(a[M - 1:M].contiguous(), w, out1, 0.7, b)
    assert torch.equal(out1[0], out[M - 1])


# -- rope + cache write --------------------------------------------------------------------------
def _paged_setup(E, lens, nkv, hd, page, dtype, seed, n_extra_pages=3):
    """Random block tables over shuffled pages for entries with the given kv lengths."""
    g = torch.Generator().manual_seed(seed)
    n_pages_each = [(n + page - 1) // page for n in lens]
    total = sum(n_pages_each) + n_extra_pages
    perm = torch.randperm(total, generator=g).tolist()
    W = max(n_pages_each)
    bt = torch.full((E, W), -1, dtype=torch.int32)
    k = 0
    for e in range(E):
        for i in range(n_pages_each[e]):
            bt[e, i] = perm[k]
            k += 1
    cache = torch.zeros(total, 2, nkv, page, hd, dtype=dtype)
    return bt, cache


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (5, 1, 48, 24), (6, 3, 32, 32), (3, 3, 80, 0)])
@pytest.mark.parametrize("many", [False, True])
@pytest.mark.parametrize("page", [16, 4, 32, 256])
def test_rope_store(cuda_device, dtype, nh, nkv, hd, rot, many, page):
    # a few tokens and many tokens go through two different kernels
    starts, qlens = ([0, 30, 15], [5, 1, 20]) if not many else ([0, 30, 15], [45, 1, 70])
    lens = [s + q for s, q in zip(starts, qlens)]
    bt, cache = _paged_setup(3, lens, nkv, hd, page, DT[dtype], 4)
    T = sum(qlens)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(DT[dtype])
    tok_pos = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, qlens)]).int()
    tok_entry = torch.cat([torch.full((q,), e) for e, q in enumerate(qlens)]).int()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(rot // 2, dtype=torch.float64) * 2 / max(rot, 1)))).float() if rot else None
    mscale = 1.1547
    d_qkv, d_cache = qkv.cuda(), cache.cuda()
    ops.rope_store(d_qkv, tok_pos.cuda(), tok_entry.cuda(), bt.cuda(), d_cache, page, nh, nkv, hd, rot,
                   inv_freq.cuda() if rot else None, mscale)
    x = qkv.float().view(T, nh + 2 * nkv, hd)
    ref = x.clone()
    if rot:
        ang = tok_pos.float()[:, None] * inv_freq[None]
        c, s = (torch.cos(ang) * mscale)[:, None], (torch.sin(ang) * mscale)[:, None]
        x1, x2 = x[:, :nh + nkv, :rot // 2], x[:, :nh + nkv, rot // 2:rot]
        ref[:, :nh + nkv, :rot // 2] = x1 * c - x2 * s
        ref[:, :nh + nkv, rot // 2:rot] = x2 * c + x1 * s
    close(d_qkv.cpu().view(T, -1, hd), ref, dtype)
    got = d_qkv.cpu().view(T, nh + 2 * nkv, hd)
    dc = d_cache.cpu()
    for t in range(T):
        e, p = int(tok_entry[t]), int(tok_pos[t])
        pg, off = int(bt[e, p // page]), p % page
        assert torch.equal(dc[pg, 0, :, off], got[t, nh:nh + nkv]) and torch.equal(dc[pg, 1, :, off], got[t, nh + nkv:])
    # nothing else was written
    written = torch.zeros_like(dc, dtype=torch.bool)
    for t in range(T):
        e, p = int(tok_entry[t]), int(tok_pos[t])
        written[int(bt[e, p // page]), :, :, p % page] = True
    assert float(dc[~written].abs().max()) == 0.0


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 3, 32, 32), (32, 2, 128, 128), (5, 1, 48, 16), (3, 3, 64, 32), (2, 2, 32, 0)])
@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
def test_gemm_skinny_rope(cuda_device, nh, nkv, hd, rot, M):
    """The q/k/v projection with rotation and cache write in its epilogue against the two kernels it stands for
    (projection, then rope_store): the same bits but for the last one of a rotated value, the same cache slots written,
    nothing else touched."""
    page, K = 16, 200
    N = (nh + 2 * nkv) * hd
    starts = [3 * i + (40 if i % 3 == 0 else 0) for i in range(M)]          # one token per request, at assorted positions
    bt, cache = _paged_setup(M, [s + 1 for s in starts], nkv, hd, page, torch.bfloat16, 21)
    g = torch.Generator().manual_seed(22)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.1).bfloat16().cuda()
    bias = torch.randn(N, generator=g).cuda() if (M % 2) else None
    tok_pos, tok_entry = torch.tensor(starts, dtype=torch.int32).cuda(), torch.arange(M, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(rot // 2, dtype=torch.float64) * 2 / max(rot, 1)))).float().cuda() if rot else None
    mscale, alpha = 1.0931, 0.75
    assert ops.skinny_rope_ok(M, K, hd, rot)
    # the two kernels
    ref_out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ref_cache = cache.clone().cuda()
    ops.gemm_skinny(x, w, ref_out, alpha, bias)
    ops.rope_store(ref_out, tok_pos, tok_entry, bt.cuda(), ref_cache, page, nh, nkv, hd, rot, inv_freq, mscale)
    # the fused one
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    d_cache = cache.clone().cuda()
    ops.gemm_skinny_rope(x, w, out, alpha, bias, tok_pos, tok_entry, bt.cuda(), d_cache, page, nh, nkv, hd, rot, inv_freq, mscale)
    close(out.cpu(), ref_out.cpu(), "float32", scale=ref_out.float().abs().max().cpu() * 400)   # 2e-5 * 400: one bfloat16 step
    close(d_cache.cpu(), ref_cache.cpu(), "float32", scale=ref_out.float().abs().max().cpu() * 400)
    assert torch.equal(d_cache == 0, ref_cache == 0)                       # the same slots, no other
    # and without a cache to write: the rows only
    out2 = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_skinny_rope(x, w, out2, alpha, bias, tok_pos, tok_entry, bt.cuda(), None, page, nh, nkv, hd, rot, inv_freq, mscale)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("H,K", [(64, 96), (200, 72), (1000, 264), (4096, 512)])
@pytest.mark.parametrize("M", [1, 7, 8, 12, 16])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
def test_gemm_skinny_resid_and_normed_consumers(cuda_device, H, K, M, wdtype):
    """The last product of a branch with the residual add in its epilogue, and the products that finish the norm:
    against plain float32 formulas, and against the kernels they stand for (product, add_rmsnorm, product)."""
    g = torch.Generator().manual_seed(31 + M)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(H, K, generator=g) * 0.1).bfloat16()
    bias = torch.randn(H, generator=g) if (M % 2) else None
    resid0 = torch.randn(M, H, generator=g) * 2.0
    nw = (1.0 + 0.3 * torch.randn(H, generator=g)).to(DT[wdtype])
    alpha, bscale, eps = 0.6, 0.35, 3e-5
    assert ops.skinny_resid_ok(M, K, H)
    # plain formulas
    y = (alpha * x.float() @ w.float().t() + (bias if bias is not None else 0.0)).bfloat16().float()
    h_ref = resid0 + bscale * y
    resid = resid0.clone().cuda()
    xw = torch.full((M, H), float("nan"), device="cuda", dtype=torch.bfloat16)
    nb = (H + 15) // 16
    sumsq = torch.full((M, nb), float("nan"), device="cuda")
    ni = ops.gemm_skinny_resid(x.cuda(), w.cuda(), alpha, bias.cuda() if bias is not None else None, resid, bscale, nw.cuda(), eps,
                               xw, sumsq)
    close(resid.cpu(), h_ref, "bfloat16", scale=y.abs().max() * bscale)   # one bfloat16 step of the branch at most
    h = resid.cpu()
    close(xw.float().cpu(), h * nw.float(), "bfloat16")
    pad = torch.zeros(M, nb * 16)
    pad[:, :H] = h * h
    close(sumsq.cpu(), pad.view(M, nb, 16).sum(-1), "float32")
    # against the kernels it stands for: the same residual bit for bit
    branch = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    ops.gemm_skinny(x.cuda(), w.cuda(), branch, alpha, bias.cuda() if bias is not None else None)
    resid2 = resid0.clone().cuda()
    normed = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    ops.add_rmsnorm(resid2, branch, bscale, nw.cuda(), eps, normed)
    assert torch.equal(resid2, resid)
    rstd = torch.rsqrt((h.double() ** 2).mean(-1, keepdim=True) + eps).float()
    # consumer 1: gate and up with SiLU(gate) * up
    N2 = 56
    wgu = (torch.randn(2 * N2, H, generator=g) * (2.0 / H ** 0.5)).bfloat16()
    act = torch.full((M, N2), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_skinny(ni.xw, wgu.cuda(), act, 1.0, None, glu=True, norm_in=ni)
    gu = rstd * (xw.float().cpu() @ wgu.float().t())
    close(act.float().cpu(), torch.nn.functional.silu(gu[:, :N2]) * gu[:, N2:], "bfloat16")
    act2 = torch.empty_like(act)
    ops.gemm_skinny(normed, wgu.cuda(), act2, 1.0, None, glu=True)
    close(act.float().cpu(), act2.float().cpu(), "bfloat16")              # the norm rounded at another place
    # consumer 2: q/k/v with rotation
    nh, nkv, hd, page = 3, 1, 32, 16
    Nq = (nh + 2 * nkv) * hd
    wq = (torch.randn(Nq, H, generator=g) * (1.0 / H ** 0.5)).bfloat16()
    starts = [5 * i + 1 for i in range(M)]
    bt, cache = _paged_setup(M, [s + 1 for s in starts], nkv, hd, page, torch.bfloat16, 33)
    tok_pos, tok_entry = torch.tensor(starts, dtype=torch.int32).cuda(), torch.arange(M, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))).float().cuda()
    outs = []
    for src, nin in ((ni.xw, ni), (normed, None)):
        o = torch.full((M, Nq), float("nan"), device="cuda", dtype=torch.bfloat16)
        c = cache.clone().cuda()
        ops.gemm_skinny_rope(src, wq.cuda(), o, 0.9, None, tok_pos, tok_entry, bt.cuda(), c, page, nh, nkv, hd, hd, inv_freq, 1.0,
                             norm_in=nin)
        outs.append((o.float().cpu(), c.float().cpu()))
    close(outs[0][0], outs[1][0], "bfloat16")
    close(outs[0][1], outs[1][1], "bfloat16")
    assert torch.equal(outs[0][1] == 0, outs[1][1] == 0)
    pre = 0.9 * rstd * (xw.float().cpu() @ wq.float().t())                 # before rotation: v is not rotated
    close(outs[0][0][:, (nh + nkv) * hd:], pre[:, (nh + nkv) * hd:], "bfloat16")


# -- attention -------------------------------------------------------------------------------------
def _attn_reference(q, kc, bt, entry_of_tok, pos_of_tok, nh, nkv, hd, page, window):
    """q [T, nh, hd] f32; kc cache f32; returns [T, nh*hd]."""
    T = q.shape[0]
    out = torch.zeros(T, nh, hd)
    G = nh // nkv
    for t in range(T):
        e, p = int(entry_of_tok[t]), int(pos_of_tok[t])
        lo = max(0, p - window + 1) if window else 0
        idx = torch.arange(lo, p + 1)
        pages = bt[e, idx // page].long()
        K = kc[pages, 0, :, idx % page]            # [n, nkv, hd]
        V = kc[pages, 1, :, idx % page]
        for j in range(nh):
            s = (K[:, j // G] @ q[t, j]) / math.sqrt(hd)
            out[t, j] = torch.softmax(s, 0) @ V[:, j // G]
    return out.view(T, nh * hd)


def _attn_case(dtype, nh, nkv, hd, starts, qlens, window, seed, dominate=False, page=16):
    E = len(starts)
    lens = [s + q for s, q in zip(starts, qlens)]
    bt, cache = _paged_setup(E, lens, nkv, hd, page, DT[dtype], seed)
    g = torch.Generator().manual_seed(seed + 1)
    cache.copy_(torch.randn(cache.shape, generator=g).to(DT[dtype]))       # stale pages hold data too
    T = sum(qlens)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(DT[dtype])
    tok_pos = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, qlens)]).int()
    tok_entry = torch.cat([torch.full((q,), e) for e, q in enumerate(qlens)]).int()
    if dominate:
        # one far key of each request gets a large score for one head: a kernel that skips or
        # misplaces it gives a visibly different output
        for e in range(E):
            far = 1 if lens[e] > 1 else 0
            pg, off = int(bt[e, far // page]), far % page
            t_last = sum(qlens[:e + 1]) - 1
            qv = qkv[t_last].view(-1, hd)[0].float()
            cache[pg, 0, 0, off] = (qv / qv.norm() * 30).to(DT[dtype])
    qstart = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    kvlen = torch.tensor(lens, dtype=torch.int32)
    ref = _attn_reference(qkv.float().view(T, -1, hd)[:, :nh], cache.float(), bt, tok_entry, tok_pos, nh, nkv, hd, page, window)
    return dict(page=page, bt=bt.cuda(), cache=cache.cuda(), qkv=qkv.cuda(), tok_pos=tok_pos.cuda(), tok_entry=tok_entry.cuda(),
                qstart=qstart.cuda(), kvlen=kvlen.cuda(), ref=ref, T=T, E=E, lens=lens, qlens=qlens)


SHAPES = [(4, 2, 16), (6, 3, 32), (5, 1, 48), (32, 2, 128), (3, 3, 64), (40, 2, 80), (8, 8, 256)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd", SHAPES)
@pytest.mark.parametrize("window", [None, 21])
@pytest.mark.parametrize("page", [16, 8, 32, 256])
def test_attention_plain(cuda_device, dtype, nh, nkv, hd, window, page):
    if page != 16 and (nh, nkv, hd) not in SHAPES[:3]:
        pytest.skip("other page sizes at three geometries")
    c = _attn_case(dtype, nh, nkv, hd, [0, 47, 16, 3], [33, 1, 17, 2], window, 10, dominate=True, page=page)
    out = torch.empty(c["T"], nh * hd, device="cuda", dtype=DT[dtype])
    ops.attention_plain(c["qkv"], out, c["cache"], c["bt"], c["tok_pos"], c["tok_entry"], c["page"], nh, nkv, hd,
                        1 / math.sqrt(hd), window)
    close(out.cpu(), c["ref"], dtype)


@pytest.mark.parametrize("nh,nkv,hd", SHAPES)
@pytest.mark.parametrize("window", [None, 21])
def test_attention_prefill_bf16(cuda_device, nh, nkv, hd, window):
    for starts, qlens in [([0, 47, 16, 3], [33, 2, 17, 2]), ([0], [130]), ([100, 0], [70, 65])]:
        c = _attn_case("bfloat16", nh, nkv, hd, starts, qlens, window, 11, dominate=True)
        out = torch.full((c["T"], nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
        tpt = max(1, 64 // (nh // nkv))
        n_tiles = sum((q + tpt - 1) // tpt for q in qlens)
        ops.attention_prefill(c["qkv"], out, c["cache"], c["bt"], c["qstart"], c["kvlen"], 0, c["E"], n_tiles, c["page"],
                              nh, nkv, hd, 1 / math.sqrt(hd), window)
        close(out.cpu(), c["ref"], "bfloat16")


@pytest.mark.parametrize("nh,nkv,hd", [(32, 2, 128), (3, 3, 64), (8, 2, 64), (6, 2, 128), (7, 1, 128), (40, 2, 64)])
@pytest.mark.parametrize("window", [None, 21, 100])
def test_attention_prefill_tc5(cuda_device, nh, nkv, hd, window):
    """The tcgen05 / tensor-memory prefill kernel: several entries with offsets, one whole prompt over many key tiles
    (the running maximum is raised late by the dominating far key), groups that do not divide 128."""
    G = nh // nkv
    assert ops.prefill_tc5_ok(hd, G, 16)
    for starts, qlens in [([0, 47, 16, 3], [33, 2, 17, 2]), ([0], [130]), ([100, 0], [70, 65]), ([5], [420])]:
        c = _attn_case("bfloat16", nh, nkv, hd, starts, qlens, window, 11, dominate=True)
        out = torch.full((c["T"], nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
        tpt = max(1, ops.prefill_tc5_rows(hd) // G)
        n_tiles = sum((q + tpt - 1) // tpt for q in qlens)
        kv_map = ops.kv_tensor_map(c["cache"])
        assert kv_map is not None
        ops.attention_prefill_tc5(c["qkv"], out, kv_map, c["bt"], c["qstart"], c["kvlen"], 0, c["E"], n_tiles, c["page"],
                                  nh, nkv, hd, 1 / math.sqrt(hd), window)
        torch.cuda.synchronize()
        ops.check_status("cuda:0")
        close(out.cpu(), c["ref"], "bfloat16")


def test_attention_prefill_tc5_late_maximum(cuda_device):
    """Scores that grow along the keys: every tile raises the running maximum by more than the threshold, so the
    accumulator in tensor memory is rescaled tile after tile; and scores that shrink, where it never is."""
    nh, nkv, hd, T = 4, 2, 64, 384
    for sign in (1.0, -1.0):
        bt, cache = _paged_setup(1, [T], nkv, hd, 16, torch.bfloat16, 3)
        g = torch.Generator().manual_seed(9)
        cache.copy_((torch.randn(cache.shape, generator=g) * 0.3).bfloat16())
        qkv = (torch.randn(T, (nh + 2 * nkv) * hd, generator=g) * 0.3).bfloat16()
        qkv.view(T, -1, hd)[:, :nh, 0] = 4.0                              # every query looks along dimension 0 ...
        for t in range(T):                                                # ... where the keys make the score rise (or fall) by 1/8 a key
            cache[int(bt[0, t // 16]), 0, :, t % 16, 0] = sign * 0.125 * t * math.sqrt(hd) / 4.0
        tok_pos, tok_entry = torch.arange(T).int(), torch.zeros(T).int()
        ref = _attn_reference(qkv.float().view(T, -1, hd)[:, :nh], cache.float(), bt, tok_entry, tok_pos, nh, nkv, hd, 16, None)
        out = torch.full((T, nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
        d_cache = cache.cuda()
        tpt = ops.prefill_tc5_rows(hd) // (nh // nkv)
        ops.attention_prefill_tc5(qkv.cuda(), out, ops.kv_tensor_map(d_cache), bt.cuda(), torch.tensor([0, T], dtype=torch.int32).cuda(),
                                  torch.tensor([T], dtype=torch.int32).cuda(), 0, 1, (T + tpt - 1) // tpt, 16, nh, nkv, hd,
                                  1 / math.sqrt(hd), None)
        torch.cuda.synchronize()
        ops.check_status("cuda:0")
        close(out.cpu(), ref, "bfloat16")


@pytest.mark.parametrize("nh,nkv,hd", SHAPES)
@pytest.mark.parametrize("window", [None, 40])
@pytest.mark.parametrize("splits", [1, 3, 7, 13])
def test_attention_decode_bf16(cuda_device, nh, nkv, hd, window, splits):
    starts = [0, 15, 16, 200, 63, 64]
    c = _attn_case("bfloat16", nh, nkv, hd, starts, [1] * len(starts), window, 12, dominate=True)
    E = c["E"]
    max_pages = (max(c["lens"]) + 15) // 16
    pps = (max_pages + splits - 1) // splits
    n_splits = (max_pages + pps - 1) // pps
    out = torch.full((E, nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    o_part = torch.full((E * nh * n_splits * hd,), float("nan"), device="cuda")
    ml_part = torch.full((E * nh * n_splits * 2,), float("nan"), device="cuda")
    ops.attention_decode(c["qkv"], out, c["cache"], c["bt"], c["kvlen"], E, c["page"], nh, nkv, hd, 1 / math.sqrt(hd),
                         window, pps, n_splits, o_part, ml_part)
    close(out.cpu(), c["ref"], "bfloat16")
    # the same through TMA tensor copies of the pages, where the head size has that path
    kv_map = ops.kv_tensor_map(c["cache"])
    assert (kv_map is not None) == (hd % 64 == 0)
    if kv_map is not None:
        assert bool(kv_map[128:].any()), "the driver refused the page view of the cache: pages would go in 2 KB boxes"
        out.fill_(float("nan"))
        ops.attention_decode(c["qkv"], out, c["cache"], c["bt"], c["kvlen"], E, c["page"], nh, nkv, hd, 1 / math.sqrt(hd),
                             window, pps, n_splits, o_part, ml_part, kv_map=kv_map)
        torch.cuda.synchronize()
        assert int(ops.stream_status("cuda:0").item()) == 0
        close(out.cpu(), c["ref"], "bfloat16")
    # pages_per_split 0: every request divides its own pages evenly over the splits
    out.fill_(float("nan"))
    o_part = torch.full((E * nh * splits * hd,), float("nan"), device="cuda")
    ml_part = torch.full((E * nh * splits * 2,), float("nan"), device="cuda")
    ops.attention_decode(c["qkv"], out, c["cache"], c["bt"], c["kvlen"], E, c["page"], nh, nkv, hd, 1 / math.sqrt(hd),
                         window, 0, splits, o_part, ml_part)
    close(out.cpu(), c["ref"], "bfloat16")


@pytest.mark.parametrize("nh,nkv,hd", [(32, 2, 128), (16, 2, 64), (5, 1, 48), (4, 2, 256)])
@pytest.mark.parametrize("splits", [9, 33, 70, 128])
def test_attention_decode_many_splits(cuda_device, nh, nkv, hd, splits):
    """Many splits (few requests, long contexts): the merge then runs four warps a row, each over every fourth split,
    in rounds of sixteen. Rows of 1,200, 700 and 16 keys, so that some splits of a row are empty."""
    starts = [1199, 699, 15]
    c = _attn_case("bfloat16", nh, nkv, hd, starts, [1] * len(starts), None, 21, dominate=True)
    E = c["E"]
    out = torch.full((E, nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    o_part = torch.full((E * nh * splits * hd,), float("nan"), device="cuda")
    ml_part = torch.full((E * nh * splits * 2,), float("nan"), device="cuda")
    for pps in (0, (75 + splits - 1) // splits):
        out.fill_(float("nan"))
        ops.attention_decode(c["qkv"], out, c["cache"], c["bt"], c["kvlen"], E, c["page"], nh, nkv, hd, 1 / math.sqrt(hd),
                             None, pps, splits, o_part, ml_part, kv_map=ops.kv_tensor_map(c["cache"]))
        torch.cuda.synchronize()
        assert int(ops.stream_status("cuda:0").item()) == 0
        close(out.cpu(), c["ref"], "bfloat16")


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (32, 2, 128), (6, 3, 64)])
def test_attention_decode_empty_rows_and_missing_pages(cuda_device, nh, nkv, hd):
    """Rows of length 0 (no keys) give zeros, and a block-table entry below 0 is never followed: its keys count as
    masked. Rows of 1, 16 and 17 keys beside them are as ever."""
    starts = [0, 15, 16, 40, 99]
    c = _attn_case("bfloat16", nh, nkv, hd, starts, [1] * len(starts), None, 14, dominate=False)
    E = c["E"]
    kvlen = c["kvlen"].clone()
    kvlen[3] = 0                                                            # a request with nothing in the cache
    bt = c["bt"].clone()
    bt[3, :] = -1
    bt[4, 2] = -1                                                           # keys 32..47 of the last request are gone
    T = c["T"]
    ref = c["ref"].clone().view(T, nh, hd)
    ref[3] = 0
    q = c["qkv"].float().cpu().view(T, -1, hd)[:, :nh]
    kc, page = c["cache"].float().cpu(), 16
    idx = torch.tensor([i for i in range(100) if not 32 <= i < 48])
    pages = c["bt"].cpu()[4, idx // page].long()
    K, V = kc[pages, 0, :, idx % page], kc[pages, 1, :, idx % page]
    for j in range(nh):
        sc = (K[:, j // (nh // nkv)] @ q[4, j]) / math.sqrt(hd)
        ref[4, j] = torch.softmax(sc, 0) @ V[:, j // (nh // nkv)]
    kv_map = ops.kv_tensor_map(c["cache"])
    for m in ([None] if kv_map is None else [None, kv_map]):
        for splits in (1, 3):
            out = torch.full((E, nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
            o_part = torch.full((E * nh * splits * hd,), float("nan"), device="cuda")
            ml_part = torch.full((E * nh * splits * 2,), float("nan"), device="cuda")
            ops.attention_decode(c["qkv"], out, c["cache"], bt, kvlen, E, 16, nh, nkv, hd, 1 / math.sqrt(hd), None, 0, splits,
                                 o_part, ml_part, kv_map=m)
            torch.cuda.synchronize()
            ops.check_status("cuda:0")
            close(out.cpu(), ref.view(T, nh * hd), "bfloat16")
            assert float(out[3].abs().max()) == 0.0


# -- sampling --------------------------------------------------------------------------------------
def test_argmax_lowest_index_wins(cuda_device):
    g = torch.Generator(device="cuda").manual_seed(6)
    logits = torch.randn(9, 73448, device="cuda", generator=g)
    logits[3, 500] = logits[3, 70000] = 50.0
    logits[4, 0] = 60.0
    logits[5, 73447] = 60.0
    out = torch.empty(9, dtype=torch.int32, device="cuda")
    ops.sample(logits, None, None, None, None, out, greedy=True)
    ref = torch.argmax(logits, -1)
    ref[3] = 500
    assert out.tolist() == ref.tolist()


def test_sampling_matches_plain(cuda_device):
    import plain_model
    g = torch.Generator().manual_seed(7)
    V = 331
    R = 24
    logits = (torch.randn(R, V, generator=g) * 3)
    temps = [0.7, 1.0, 1.3, 0.0] * 6
    ks = [0, 5, 1, 50, 331, 400] * 4
    ps = [1.0, 0.8, 0.5, 0.95] * 6
    us = [float(x) for x in torch.rand(R, generator=g)]
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), torch.tensor(temps).cuda(), torch.tensor(ks, dtype=torch.int32).cuda(),
               torch.tensor(ps).cuda(), torch.tensor(us).cuda(), out)
    ref = [plain_model.sample_plain(logits[i], temps[i], ks[i], ps[i], us[i]) for i in range(R)]
    assert out.tolist() == ref


def test_sampling_distribution(cuda_device):
    """Many draws follow softmax(logits / T) restricted to the kept set."""
    V = 50
    logits = torch.linspace(-2, 2, V)
    R = 4000
    g = torch.Generator().manual_seed(8)
    us = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits.repeat(R, 1).cuda(), torch.full((R,), 0.8).cuda(), torch.full((R,), 10, dtype=torch.int32).cuda(),
               torch.full((R,), 1.0).cuda(), us.cuda(), out)
    counts = torch.bincount(out.cpu().long(), minlength=V).float() / R
    p = torch.softmax(logits / 0.8, 0)
    p[:V - 10] = 0
    p /= p.sum()
    assert counts[:V - 10].sum() == 0
    assert float((counts - p).abs().max()) < 0.03


@pytest.mark.parametrize("M,N,K", [(1, 97, 64), (8, 331, 200), (3, 4096, 4096), (9, 300, 264), (16, 129, 1000), (5, 16, 8), (12, 5000, 320)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_skinny(cuda_device, M, N, K, out_dtype):
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    ops.gemm_skinny(x, w, out, 0.7, b)
    ref = 0.7 * (x.double() @ w.double().t()) + b.double()
    close(out, ref.float(), "float32" if out_dtype == "float32" else "bfloat16")
    # a row's bits do not depend on the rows beside it
    out1 = torch.empty(1, N, device="cuda", dtype=DT[out_dtype])
    ops.gemm_skinny(x[M - 1:M].contiguous(), w, out1, 0.7, b)
    assert torch.equal(out1[0], out[M - 1])


@pytest.mark.parametrize("M,I,K", [(1, 160, 64), (8, 264, 200), (13, 320, 192), (4, 16384, 4096)])
def test_gemm_skinny_swiglu(cuda_device, M, I, K):
    g = torch.Generator(device="cuda").manual_seed(10)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * 2 / math.sqrt(K)).bfloat16()
    b = torch.randn(2 * I, device="cuda", generator=g) * 0.1
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_skinny(x, w, out, 1.0, b, glu=True)
    y = x.double() @ w.double().t() + b.double()
    close(out, (torch.nn.functional.silu(y[:, :I]) * y[:, I:]).float(), "bfloat16")
    ops.gemm_skinny(x, w, out, 1.0, None, glu=True)
    y = x.double() @ w.double().t()
    close(out, (torch.nn.functional.silu(y[:, :I]) * y[:, I:]).float(), "bfloat16")


@pytest.mark.parametrize("M,N,K", [(17, 97, 64), (32, 128, 64), (64, 331, 200), (200, 513, 1000), (64, 4096, 4096), (256, 300, 264),
                                   (33, 73448, 256)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_tc5(cuda_device, M, N, K, out_dtype):
    """The tcgen05/TMA product (accumulators in tensor memory) against a float64 reference; its bounded waits never ran out."""
    g = torch.Generator(device="cuda").manual_seed(12)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    scratch = torch.empty(max(ops.gemm_tc5_scratch_bytes(M, N, K) // 4, 1), device="cuda")
    ops.gemm_tc5(x, w, out, 0.7, b, scratch)
    torch.cuda.synchronize()
    assert int(ops.stream_status("cuda:0").item()) == 0
    ref = 0.7 * (x.double() @ w.double().t()) + b.double()
    close(out, ref.float(), "float32" if out_dtype == "float32" else "bfloat16")
    ops.gemm_tc5(x, w, out, 1.0, None, scratch)
    close(out, (x.double() @ w.double().t()).float(), "float32" if out_dtype == "float32" else "bfloat16")


@pytest.mark.parametrize("M,N,K", [(17, 97, 64), (32, 128, 72), (64, 331, 200), (128, 513, 1000), (64, 4608, 4096), (33, 300, 264),
                                   (40, 4096, 16384)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("bm,nb", [(0, 0), (64, 16), (128, 32)])
def test_gemm_mid(cuda_device, M, N, K, out_dtype, bm, nb):
    """The tcgen05 product of 17..128 rows (tiles of 64 or 128 weight rows by blocks of activation rows, all of K in one
    unit, two issuing threads with an accumulator each) against a float64 reference, row by row."""
    g = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).bfloat16()
    b = torch.randn(N, device="cuda", generator=g)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    ops.gemm_mid(x, w, out, 0.7, b, nb=nb, bm=bm)
    torch.cuda.synchronize()
    assert int(ops.stream_status("cuda:0").item()) == 0
    ref = 0.7 * (x.double() @ w.double().t()) + b.double()
    close(out, ref.float(), "float32" if out_dtype == "float32" else "bfloat16")
    ops.gemm_mid(x, w, out, 1.0, None, nb=nb, bm=bm)
    close(out, (x.double() @ w.double().t()).float(), "float32" if out_dtype == "float32" else "bfloat16")


@pytest.mark.parametrize("M,I,K", [(20, 160, 72), (64, 264, 200), (48, 1000, 520), (128, 320, 192), (64, 16384, 4096)])
@pytest.mark.parametrize("bm,nb", [(0, 0), (64, 32), (128, 16)])
def test_gemm_mid_swiglu(cuda_device, M, I, K, bm, nb):
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * 2 / math.sqrt(K)).bfloat16()
    b = torch.randn(2 * I, device="cuda", generator=g) * 0.1
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_mid(x, w, out, 1.0, b, glu=True, nb=nb, bm=bm)
    torch.cuda.synchronize()
    assert int(ops.stream_status("cuda:0").item()) == 0
    y = x.double() @ w.double().t() + b.double()
    close(out, (torch.nn.functional.silu(y[:, :I]) * y[:, I:]).float(), "bfloat16")
    ops.gemm_mid(x, w, out, 1.0, None, glu=True, nb=nb, bm=bm)
    y = x.double() @ w.double().t()
    close(out, (torch.nn.functional.silu(y[:, :I]) * y[:, I:]).float(), "bfloat16")
    # against the library product and the SwiGLU kernel it replaces on 17..128 rows (which round gate and up to bfloat16 first)
    gu = torch.empty(M, 2 * I, device="cuda", dtype=torch.bfloat16)
    torch.mm(x, w.t(), out=gu)
    act = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
    ops.swiglu(gu, act)
    close(out, act.float(), "bfloat16")
