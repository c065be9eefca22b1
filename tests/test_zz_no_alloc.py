"""il_attn_decode_noalloc, the decode attention entry point for callers that cannot allocate
device memory (a host that forbids cudaMalloc after start-up, a thread that must not enter the
allocator): called here through its exported C symbol with ctypes, twice in a row with different
inputs, and compared with the regular entry point, which takes its scratch from the caller.
The two run the same kernels, so the outputs must agree bit for bit; the tolerance of the kernel
tests is the bound asserted. A call that needs more scratch than the built-in array holds is
refused without a launch.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from infinilm_b200 import ops  # noqa: E402
from infinilm_b200.csrc import build  # noqa: E402

HD = 64
TOL = 2e-2          # the bfloat16 tolerance of tests/test_kernels_gpu.py


def _lib():
    lib = ctypes.CDLL(build.compile_source("attn_decode_noalloc", {"HEAD_DIM": HD}))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.il_attn_decode_noalloc.argtypes = [vp, ci, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, ctypes.c_float, ci, ci, ci, vp]
    lib.il_attn_decode_noalloc.restype = ci
    lib.il_attn_decode_noalloc_strerror.argtypes = [ci]
    lib.il_attn_decode_noalloc_strerror.restype = ctypes.c_char_p
    lib.il_attn_decode_noalloc_max_rows.restype = ci
    lib.il_attn_decode_noalloc_scratch_bytes.restype = ctypes.c_longlong
    return lib


def _case(seed, nh, nkv, lens):
    page = 16
    g = torch.Generator().manual_seed(seed)
    E = len(lens)
    n_pages = [(n + page - 1) // page for n in lens]
    perm = torch.randperm(sum(n_pages) + 2, generator=g).tolist()
    bt = torch.full((E, max(n_pages)), -1, dtype=torch.int32)
    k = 0
    for e in range(E):
        for i in range(n_pages[e]):
            bt[e, i] = perm[k]
            k += 1
    cache = torch.randn(sum(n_pages) + 2, 2, nkv, page, HD, generator=g).bfloat16().cuda()
    qkv = torch.randn(E, (nh + 2 * nkv) * HD, generator=g).bfloat16().cuda()
    return qkv, cache, bt.cuda(), torch.tensor(lens, dtype=torch.int32).cuda()


def _both(lib, seed, nh, nkv, lens, n_splits_wanted):
    qkv, cache, bt, kvlen = _case(seed, nh, nkv, lens)
    E = len(lens)
    max_pages = (max(lens) + 15) // 16
    pps = (max_pages + n_splits_wanted - 1) // n_splits_wanted
    n_splits = (max_pages + pps - 1) // pps
    scale = 1 / math.sqrt(HD)
    ref = torch.empty(E, nh * HD, dtype=torch.bfloat16, device="cuda")
    rows = E * nh * n_splits
    ops.attention_decode(qkv, ref, cache, bt, kvlen, E, 16, nh, nkv, HD, scale, None, pps, n_splits,
                         torch.empty(rows * HD, device="cuda"), torch.empty(rows * 2, device="cuda"))
    out = torch.full((E, nh * HD), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.il_attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), cache.data_ptr(), bt.data_ptr(),
                                    bt.shape[1], kvlen.data_ptr(), 16, E, nh, nkv, HD, scale, 0, pps, n_splits, stream)
    assert rc == 0, lib.il_attn_decode_noalloc_strerror(rc).decode()
    torch.cuda.synchronize()
    return out.float().cpu(), ref.float().cpu()


def test_no_alloc_entry_point_matches_the_regular_one(cuda_device):
    lib = _lib()
    assert lib.il_attn_decode_noalloc_max_rows() == 8192
    assert lib.il_attn_decode_noalloc_scratch_bytes() == 4 * 8192 * (HD + 2)
    # two calls in a row; the second has other shapes and finds the first one's partials in the array
    for seed, nh, nkv, lens, splits in [(1, 8, 2, [300, 17, 64, 1, 129], 5), (2, 6, 3, [40, 200], 2)]:
        out, ref = _both(lib, seed, nh, nkv, lens, splits)
        assert torch.isfinite(out).all()
        err = float((out - ref).abs().max() / ref.abs().max())
        assert err <= TOL, f"rel err {err:.3e}"
        assert torch.equal(out, ref)             # the same kernels: identical bits


def test_no_alloc_entry_point_refuses_what_does_not_fit(cuda_device):
    lib = _lib()
    qkv, cache, bt, kvlen = _case(3, 8, 2, [32] * 4)
    out = torch.zeros(4, 8 * HD, dtype=torch.bfloat16, device="cuda")
    # 4 entries * 8 heads * 300 splits = 9600 rows > 8192
    rc = lib.il_attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), cache.data_ptr(), bt.data_ptr(),
                                    bt.shape[1], kvlen.data_ptr(), 16, 4, 8, 2, HD, 0.125, 0, 1, 300,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert b"exceeds" in lib.il_attn_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0          # nothing ran
    # a head size the library was not compiled for
    rc = lib.il_attn_decode_noalloc(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), cache.data_ptr(), bt.data_ptr(),
                                    bt.shape[1], kvlen.data_ptr(), 16, 4, 8, 2, 128, 0.125, 0, 1, 1,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -2
