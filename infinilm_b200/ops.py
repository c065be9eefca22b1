"""Python face of the hand-written sm_100a kernels.

Each function checks its arguments on the host (shapes, dtypes, contiguity, device), then calls
the `extern "C"` entry point of the kernel's shared object with raw device pointers and the
current CUDA stream. There is no CPU implementation and no library stand-in here: a tensor that
is not on a CUDA device, or a kernel library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def kind_of(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    return _c_void_p(t.data_ptr())


_raw_stream = torch._C._cuda_getCurrentRawStream
_cur_device = torch._C._cuda_getDevice


def _stream() -> _c_void_p:
    """The current device's current stream (asked of the runtime directly: this runs once per launch)."""
    return _c_void_p(_raw_stream(_cur_device()))


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("infinilm_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device} (there is no CPU path)")


def _contig(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (replayed graph nodes included)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    if code >= 1000:
        raise KernelError(f"{what}: CUDA launch failed (cudaError {code - 1000})")
    raise KernelError(f"{what}: error {code}")


_fns = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=None):
    """The entry point `fn_name` of the library built from `lib_name` with `defines`; looked up once."""
    key = (lib_name, fn_name, next(iter(defines.values())) if defines else None)
    f = _fns.get(key)
    if f is None:
        if defines and len(defines) != 1:
            raise KernelError("a kernel library is keyed by one definition")
        f = getattr(build.load(lib_name, defines), fn_name)
        f.argtypes = argtypes
        f.restype = _c_int
        _fns[key] = f
    return f


# ----------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor, round_bf16: bool) -> None:
    """out[t,:] (f32) = table[ids[t],:] * scale; rounded through bfloat16 when `round_bf16`."""
    _need_cuda(ids, table, out)
    T, (V, H) = ids.numel(), table.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or out.shape != (T, H):
        raise KernelError("embed: ids int32 [T], out float32 [T,H]")
    _contig("table", table), _contig("out", out)
    f = _fn("embedding", "il_embed", [_c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int,
                                      _c_int, _c_int, _c_void_p])
    _check(f(_ptr(ids), _ptr(table), kind_of(table.dtype), scale, _ptr(out), T, H, V, int(round_bf16),
             _stream()), "embed")


def patch_tokens(token_ids: torch.Tensor, rows: torch.Tensor, src_idx: torch.Tensor, src: torch.Tensor) -> None:
    """token_ids[rows[i]] = src[src_idx[i]], all int32 on the device."""
    _need_cuda(token_ids, rows, src_idx, src)
    for t in (token_ids, rows, src_idx, src):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("patch_tokens: contiguous int32 tensors")
    f = _fn("embedding", "il_patch_tokens", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(token_ids), _ptr(rows), _ptr(src_idx), _ptr(src), rows.numel(), _stream()), "patch_tokens")


def add_rmsnorm(resid: torch.Tensor, branch: Optional[torch.Tensor], branch_scale: float, weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """resid += branch_scale * branch (f32, in place); out = RMSNorm(resid) * weight.

    With `rows` (int32 indices) only those rows are normalised, into out[0..len(rows)), and
    `resid` is left as it was."""
    _need_cuda(resid, branch, weight, out, rows)
    T, H = resid.shape
    n = T if rows is None else rows.numel()
    if resid.dtype != torch.float32 or weight.numel() != H or out.shape[-1] != H or out.shape[0] < n:
        raise KernelError("add_rmsnorm: resid float32 [T,H], weight [H], out [n,H]")
    if branch is not None and (branch.shape != resid.shape or branch.dtype != out.dtype):
        raise KernelError("add_rmsnorm: branch must match resid's shape and out's dtype")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_rmsnorm: rows must be int32")
    _contig("resid", resid), _contig("out", out)
    if branch is not None:
        _contig("branch", branch)
    f = _fn("rmsnorm", "il_add_rmsnorm", [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_float, _c_void_p,
                                          _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(resid), _ptr(branch), branch_scale, _ptr(weight), kind_of(weight.dtype), eps, _ptr(out),
             kind_of(out.dtype), _ptr(rows), n, H, _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t,i] = silu(gate_up[t,i]) * gate_up[t,I+i]."""
    _need_cuda(gate_up, out)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: gate_up [T,2I], out [T,I] of the same dtype")
    _contig("gate_up", gate_up), _contig("out", out)
    f = _fn("swiglu", "il_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), kind_of(out.dtype), T, I2 // 2, _stream()), "swiglu")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    _need_cuda(y, bias)
    T, N = y.shape
    if bias.numel() != N:
        raise KernelError("add_bias: bias [N]")
    _contig("y", y)
    f = _fn("swiglu", "il_add_bias", [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(y), kind_of(y.dtype), _ptr(bias), kind_of(bias.dtype), T, N, _stream()), "add_bias")


def rope_store(qkv: torch.Tensor, tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor,
               cache: Optional[torch.Tensor], page_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
               rot_dim: int, inv_freq: Optional[torch.Tensor], mscale: float) -> None:
    """Rotates q and k of `qkv` in place and writes k and v to their cache slots (if `cache`)."""
    _need_cuda(qkv, tok_pos, tok_entry, block_table, cache, inv_freq)
    T = qkv.shape[0]
    _contig("qkv", qkv), _contig("block_table", block_table)
    if tok_pos.dtype != torch.int32 or tok_entry.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise KernelError("rope_store: descriptors must be int32")
    if rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_store: inv_freq float32 [rot_dim/2]")
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != qkv.dtype or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("rope_store: cache [pages,2,kv_heads,page,head_dim] of qkv's dtype")
    f = _fn("rope_cache", "il_rope_store", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                            _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                            _c_float, _c_void_p])
    _check(f(_ptr(qkv), kind_of(qkv.dtype), qkv.shape[1], _ptr(tok_pos), _ptr(tok_entry), _ptr(block_table),
             block_table.shape[1], _ptr(cache), page_size, T, n_heads, n_kv_heads, head_dim, rot_dim,
             _ptr(inv_freq), mscale, _stream()), "rope_store")


def attention_plain(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                    tok_pos: torch.Tensor, tok_entry: torch.Tensor, page_size: int, n_heads: int,
                    n_kv_heads: int, head_dim: int, scale: float, window: Optional[int] = None) -> None:
    """Causal attention of every token of `qkv` over its request's cache pages (plain kernel)."""
    _need_cuda(qkv, out, cache, block_table, tok_pos, tok_entry)
    T = qkv.shape[0]
    if out.shape != (T, n_heads * head_dim) or out.dtype != qkv.dtype or cache.dtype != qkv.dtype:
        raise KernelError("attention_plain: out [T, heads*head_dim], same dtype as qkv and cache")
    if head_dim > 256:
        raise KernelError(f"attention_plain: head_dim {head_dim} > 256 is not supported")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_plain", "il_attn_plain", [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                            _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                            _c_int, _c_void_p])
    _check(f(_ptr(qkv), kind_of(qkv.dtype), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table),
             block_table.shape[1], _ptr(tok_pos), _ptr(tok_entry), page_size, T, n_heads, n_kv_heads, head_dim,
             scale, int(window or 0), _stream()), "attention_plain")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0,
             bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = alpha * a[M,K] @ w[N,K]^T (+ bias), all float32, FP32 pipes only."""
    _need_cuda(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.float32 or w.dtype != torch.float32 or out.dtype != torch.float32:
        raise KernelError("gemm_f32: float32 tensors")
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_f32: bias float32 [N]")
    f = _fn("gemm_f32", "il_gemm_f32", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _ptr(bias), alpha, M, N, K,
             _stream()), "gemm_f32")


_ones_k = {}


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], uniform: Optional[torch.Tensor], out: torch.Tensor, greedy: bool = False) -> None:
    """One token per row of float32 logits [R,V]; per-row temperature, top_k, top_p, uniform number.
    `greedy`: argmax of every row (no parameters needed)."""
    _need_cuda(logits, temperature, top_k, top_p, uniform, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.numel() < R:
        raise KernelError("sample: logits float32 [R,V] with contiguous rows, out int32 [R]")
    if greedy:
        key = (logits.device, R)
        if key not in _ones_k:
            _ones_k[key] = torch.ones(max(R, 64), dtype=torch.int32, device=logits.device)
        top_k, temperature, top_p, uniform = _ones_k[key], None, None, None
    else:
        for nm, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                          ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32)):
            if t is None or t.dtype != dt or t.numel() < R or not t.is_contiguous():
                raise KernelError(f"sample: {nm} must be a contiguous {dt} tensor of R entries")
    f = _fn("sampling", "il_sample", [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                      _c_void_p, _c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
             _ptr(out), _stream()), "sample")


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     entry_kvlen: torch.Tensor, n_decode: int, page_size: int, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: Optional[int], pages_per_split: int, n_splits: int,
                     o_part: torch.Tensor, ml_part: torch.Tensor, kv_map: Optional[torch.Tensor] = None) -> None:
    """bfloat16 split-KV attention of token rows [0, n_decode) (entry i = row i, one token each), then the merge of
    the splits (a second launch; with n_splits = 1 there is none and the attention kernel writes `out` itself). A row whose length is 0 gets zeros; a block-table entry below 0 is never followed.
    pages_per_split 0: each request's pages are divided evenly over the n_splits splits.
    kv_map: the cache's tensor map from `kv_tensor_map` (pages then come in by TMA tensor copies).
    Scratch: o_part float32 [n_decode*heads*n_splits*head_dim], ml_part float32 [n_decode*heads*n_splits*2]."""
    _need_cuda(qkv, out, cache, block_table, entry_kvlen, o_part, ml_part)
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 tensors")
    if o_part is None or ml_part is None or o_part.dtype != torch.float32 or ml_part.dtype != torch.float32:
        raise KernelError("attention_decode: scratch must be float32")
    need = n_decode * n_heads * n_splits
    if o_part.numel() < need * head_dim or ml_part.numel() < need * 2:
        raise KernelError("attention_decode: scratch too small")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_decode or qkv.shape[0] < n_decode:
        raise KernelError("attention_decode: out [rows, heads*head_dim]")
    if block_table.dtype != torch.int32 or entry_kvlen.dtype != torch.int32 or block_table.shape[0] < n_decode or entry_kvlen.numel() < n_decode:
        raise KernelError("attention_decode: block_table int32 [entries, width], entry_kvlen int32 [entries]")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_decode", "il_attn_decode", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                                              _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void_p,
                                              _c_void_p, _c_void_p, _c_void_p, _c_void_p], defines={"HEAD_DIM": head_dim})
    if kv_map is not None and (kv_map.is_cuda or kv_map.dtype != torch.uint8 or kv_map.numel() != KV_MAP_BYTES):
        raise KernelError("attention_decode: kv_map must be the host tensor kv_tensor_map returned")
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(entry_kvlen),
             page_size, n_decode, n_heads, n_kv_heads, head_dim, scale, int(window or 0), pages_per_split, n_splits,
             _ptr(o_part), _ptr(ml_part), _ptr(kv_map), _ptr(stream_status(qkv.device)) if kv_map is not None else _c_void_p(0),
             _stream()), "attention_decode")
    if n_splits > 1:
        count_launches(1)                         # the merge kernel (a single split needs none: the attention kernel finishes the rows)


_resident = {}


def attention_decode_resident_blocks(head_dim: int) -> int:
    """Blocks of the decode attention kernel that the current device runs at once at this head size (occupancy x SMs)."""
    key = (torch.cuda.current_device(), head_dim)
    if key not in _resident:
        lib = build.load("attn_decode", {"HEAD_DIM": head_dim})
        fn = lib.il_attn_decode_resident_blocks
        fn.argtypes, fn.restype = [], _c_int
        n = int(fn())
        if n <= 0:
            raise KernelError("attention_decode: the occupancy query failed")
        _resident[key] = n
    return _resident[key]


KV_MAP_BYTES = 384


def kv_tensor_map(cache: torch.Tensor) -> Optional[torch.Tensor]:
    """The TMA tensor maps (3 x 128 bytes, on the host) of one layer's bfloat16 cache [pages,2,kv_heads,16,head_dim]: one
    for boxes of [16 keys x 64 columns], one whose box is a whole page of a kv head, one whose box is the K or V of a page
    as tensor-core tiles (the last two all zero if the driver refuses them).
    None when the attention kernels have no tensor-copy path for this geometry (head_dim not a multiple of 64)."""
    if not cache.is_cuda or cache.dtype != torch.bfloat16 or cache.dim() != 5 or cache.shape[3] != 16 or cache.shape[4] % 64:
        return None
    hd = cache.shape[4]
    lib = build.load("attn_decode", {"HEAD_DIM": hd})
    fn = lib.il_attn_decode_kv_map
    fn.argtypes, fn.restype = [_c_void_p, _c_void_p, ctypes.c_longlong, _c_int, _c_int], _c_int
    m = torch.zeros(KV_MAP_BYTES, dtype=torch.uint8)
    rc = fn(_c_void_p(m.data_ptr()), _ptr(cache), cache.numel() // hd, hd, cache.shape[2])
    return m if rc == 0 else None


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      entry_qstart: torch.Tensor, entry_kvlen: torch.Tensor, first_entry: int, n_entries: int,
                      n_tiles_total: int, page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                      window: Optional[int]) -> None:
    """bfloat16 causal attention of the tokens of entries [first_entry, n_entries) over their cache pages.
    n_tiles_total = sum over those entries of ceil(q_len / (64 // (heads/kv_heads)))."""
    _need_cuda(qkv, out, cache, block_table, entry_qstart, entry_kvlen)
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 tensors")
    if out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention_prefill: out [T, heads*head_dim]")
    _contig("qkv", qkv), _contig("out", out), _contig("cache", cache), _contig("block_table", block_table)
    f = _fn("attn_prefill", "il_attn_prefill", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                                                _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                                _c_int, _c_void_p], defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(entry_qstart),
             _ptr(entry_kvlen), page_size, first_entry, n_entries, n_tiles_total, n_heads, n_kv_heads, head_dim, scale,
             int(window or 0), _stream()), "attention_prefill")


_tc5_prefill_rows = {}


def prefill_tc5_rows(head_dim: int) -> int:
    """Rows (tokens x heads of a kv head) a block of the tensor-memory prefill kernel owns."""
    if head_dim not in _tc5_prefill_rows:
        lib = build.load("attn_prefill_tc5", {"HEAD_DIM": head_dim})
        fn = lib.il_attn_prefill_tc5_rows
        fn.argtypes, fn.restype = [], _c_int
        _tc5_prefill_rows[head_dim] = int(fn())
    return _tc5_prefill_rows[head_dim]


def prefill_tc5_ok(head_dim: int, group: int, page_size: int, kv_map: Optional[torch.Tensor] = None) -> bool:
    """Whether the tensor-memory prefill kernel takes this geometry and, if given, this tensor map of the cache (it
    needs the third map of `kv_tensor_map`, a page's K or V as tensor-core tiles)."""
    if not (head_dim in (64, 128) and 0 < group <= 128 and page_size == 16):
        return False
    return kv_map is None or _has_third_map(kv_map)


def _has_third_map(kv_map: torch.Tensor) -> bool:
    """Whether this host tensor is a `kv_tensor_map` result with its third map filled; looked at once per tensor
    object (the answer is kept on the object, so another tensor at the same address is looked at again)."""
    ok = getattr(kv_map, "_il_third_map", None)
    if ok is None:
        ok = (not kv_map.is_cuda and kv_map.dtype == torch.uint8 and kv_map.numel() == KV_MAP_BYTES
              and bool(kv_map[256:].any()))
        kv_map._il_third_map = ok
    return ok


def attention_prefill_tc5(qkv: torch.Tensor, out: torch.Tensor, kv_map: torch.Tensor, block_table: torch.Tensor,
                          entry_qstart: torch.Tensor, entry_kvlen: torch.Tensor, first_entry: int, n_entries: int,
                          n_tiles_total: int, page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                          window: Optional[int]) -> None:
    """The same attention as `attention_prefill`, on tcgen05 tensor cores with tensor memory; `kv_map` is the cache's
    tensor map (`kv_tensor_map`). n_tiles_total = sum over the entries of ceil(q_len / (prefill_tc5_rows(head_dim) // (heads/kv_heads)))."""
    _need_cuda(qkv, out, block_table, entry_qstart, entry_kvlen)
    if qkv.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc5: bfloat16 tensors")
    if not _has_third_map(kv_map):
        raise KernelError("attention_prefill_tc5: kv_map must be the host tensor kv_tensor_map returned, with its third map")
    if out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention_prefill_tc5: out [T, heads*head_dim]")
    _contig("qkv", qkv), _contig("out", out), _contig("block_table", block_table)
    f = _fn("attn_prefill_tc5", "il_attn_prefill_tc5",
            [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p, _c_void_p], defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(qkv), qkv.shape[1], _ptr(out), _c_void_p(kv_map.data_ptr() + 256), _ptr(block_table), block_table.shape[1],
             _ptr(entry_qstart), _ptr(entry_kvlen), page_size, first_entry, n_entries, n_tiles_total, n_heads, n_kv_heads,
             head_dim, scale, int(window or 0), _ptr(stream_status(qkv.device)), _stream()), "attention_prefill_tc5")


SKINNY_MAX_ROWS = 16


class NormedInput:
    """Activations whose RMSNorm is not finished: `xw` = residual * norm weight (bfloat16 [T,H]) and `sumsq`, the sums of
    the residual's squares per row and block of 16 columns (float32 [T, n_blocks]); the product that reads them divides
    by the rms. Made by `gemm_skinny_resid`, read by `gemm_skinny(glu=True)` and `gemm_skinny_rope`."""
    __slots__ = ("xw", "sumsq", "width", "eps")

    def __init__(self, xw: torch.Tensor, sumsq: torch.Tensor, width: int, eps: float):
        self.xw, self.sumsq, self.width, self.eps = xw, sumsq, int(width), float(eps)

    @property
    def shape(self):
        return self.xw.shape


NORM_MAX_BLOCKS = 256                             # blocks of 16 columns the fused norm handles: residual width <= 4096


def _norm_args(norm_in: Optional[NormedInput], M: int):
    if norm_in is None:
        return _c_void_p(0), 0, 0, 0.0
    sq = norm_in.sumsq
    if sq.dtype != torch.float32 or not sq.is_contiguous() or sq.shape[0] < M or sq.shape[1] > NORM_MAX_BLOCKS:
        raise KernelError("norm_in: sumsq float32 [rows, blocks <= 256], contiguous")
    return _ptr(sq), sq.shape[1], norm_in.width, norm_in.eps


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0,
                bias: Optional[torch.Tensor] = None, glu: bool = False, norm_in: Optional[NormedInput] = None) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) for M <= 16 bfloat16 rows; out bfloat16 or float32.
    glu: w is [2N,K] (gate rows, then up rows) and out[M,N] = silu(gate) * up.
    norm_in (glu only): x is `norm_in.xw`, and the results are divided by the rms that its sums give."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0] // 2 if glu else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_skinny: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_skinny: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.shape[0]):
        raise KernelError("gemm_skinny: bias float32, one per weight row")
    if norm_in is not None and not glu:
        raise KernelError("gemm_skinny: norm_in goes with glu=True (or gemm_skinny_rope)")
    f = _fn("gemm_skinny", "il_gemm_skinny", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p,
                                              _c_float, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_float,
                                              _c_void_p])
    np_, nb, nw, ne = _norm_args(norm_in, M)
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, int(glu), np_, nb, nw, ne, _stream()), "gemm_skinny")


def skinny_resid_ok(M: int, K: int, width: int) -> bool:
    """Whether `gemm_skinny_resid` takes this shape."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and (width + 15) // 16 <= NORM_MAX_BLOCKS


def gemm_skinny_resid(x: torch.Tensor, w: torch.Tensor, alpha: float, bias: Optional[torch.Tensor], resid: torch.Tensor,
                      branch_scale: float, norm_weight: torch.Tensor, eps: float, xw: torch.Tensor,
                      sumsq: torch.Tensor) -> NormedInput:
    """The last product of a branch (up to 16 bfloat16 rows) with the residual add and the next RMSNorm's inputs in its
    epilogue: resid (float32 [M,H], in place) += branch_scale * bf16(alpha * x @ w^T + bias); xw = resid * norm_weight;
    sumsq[m][b] = sum of resid[m]^2 over columns 16b..16b+15. Returns what the next product needs to finish the norm."""
    _need_cuda(x, w, bias, resid, norm_weight, xw, sumsq)
    M, K = x.shape
    H = w.shape[0]
    nb = (H + 15) // 16
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_skinny_resid: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)}")
    if resid.dtype != torch.float32 or tuple(resid.shape) != (M, H) or xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, H):
        raise KernelError("gemm_skinny_resid: resid float32 [M,H], xw bfloat16 [M,H]")
    if sumsq.dtype != torch.float32 or tuple(sumsq.shape) != (M, nb) or norm_weight.numel() != H:
        raise KernelError("gemm_skinny_resid: sumsq float32 [M, ceil(H/16)], norm_weight [H]")
    if x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_skinny_resid: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != H):
        raise KernelError("gemm_skinny_resid: bias float32 [H]")
    _contig("resid", resid), _contig("xw", xw), _contig("sumsq", sumsq), _contig("norm_weight", norm_weight)
    f = _fn("gemm_skinny", "il_gemm_skinny_resid", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float, _c_int, _c_int, _c_int,
                                                    _c_void_p, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), alpha, M, H, K, _ptr(resid), branch_scale, _ptr(norm_weight),
             kind_of(norm_weight.dtype), _ptr(xw), _ptr(sumsq), _stream()), "gemm_skinny_resid")
    return NormedInput(xw, sumsq, H, eps)


def skinny_rope_ok(M: int, K: int, head_dim: int, rot_dim: int) -> bool:
    """Whether `gemm_skinny_rope` takes this shape: a few rows, rotary and head sizes in steps of 16."""
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0 and head_dim % 16 == 0 and rot_dim % 16 == 0 and 0 <= rot_dim <= head_dim


def gemm_skinny_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float, bias: Optional[torch.Tensor],
                     tok_pos: torch.Tensor, tok_entry: torch.Tensor, block_table: torch.Tensor, cache: Optional[torch.Tensor],
                     page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, rot_dim: int,
                     inv_freq: Optional[torch.Tensor], mscale: float, norm_in: Optional[NormedInput] = None) -> None:
    """The q/k/v projection of up to 16 bfloat16 rows with what `rope_store` does in its epilogue: out[M, (heads + 2
    kv_heads) * head_dim] = alpha * x @ w^T (+ bias), q and k rotated, k and v written to their cache slots (if `cache`)."""
    _need_cuda(x, w, out, bias, tok_pos, tok_entry, block_table, cache, inv_freq)
    M, K = x.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or tuple(w.shape) != (N, K) or out.shape != (M, N):
        raise KernelError(f"gemm_skinny_rope: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_skinny_rope: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_skinny_rope: bias float32, one per weight row")
    if tok_pos.dtype != torch.int32 or tok_entry.dtype != torch.int32 or block_table.dtype != torch.int32 or tok_pos.numel() < M:
        raise KernelError("gemm_skinny_rope: descriptors must be int32, one position and entry per row")
    if rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("gemm_skinny_rope: inv_freq float32 [rot_dim/2]")
    _contig("block_table", block_table)
    if cache is not None:
        _contig("cache", cache)
        if cache.dtype != torch.bfloat16 or tuple(cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError("gemm_skinny_rope: cache bfloat16 [pages,2,kv_heads,page,head_dim]")
    f = _fn("gemm_skinny", "il_gemm_skinny_rope",
            [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_float, _c_int, _c_int, _c_void_p, _c_void_p,
             _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_int, _c_int,
             _c_float, _c_void_p])
    np_, nb, nw, ne = _norm_args(norm_in, M)
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _ptr(bias), alpha, M, K, _ptr(tok_pos),
             _ptr(tok_entry), _ptr(block_table), block_table.shape[1], _ptr(cache), page_size, n_heads, n_kv_heads, head_dim,
             rot_dim, _ptr(inv_freq), mscale, np_, nb, nw, ne, _stream()), "gemm_skinny_rope")


def skinny_ok(M: int, K: int) -> bool:
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0


_stream_status = {}


def stream_status(device) -> torch.Tensor:
    """The status word of the bulk-copy kernels on `device`: 0, or non-zero after a bounded wait ran out."""
    key = torch.device(device).index or 0
    if key not in _stream_status:
        _stream_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _stream_status[key]


def check_status(device) -> None:
    """Raises if a kernel with bounded waits (mbarriers of the TMA / tcgen05 kernels) gave up since the last check: its
    output is then not to be trusted. Reads one word from the device, so it synchronises; call it where the host
    waits anyway."""
    key = torch.device(device).index or 0
    t = _stream_status.get(key)
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(f"a kernel's bounded wait ran out (code {code}: 11-14 gemm_tc5, 21 attn_decode, 30-39 attn_prefill_tc5, 51-54 gemm_mid); the step's results are invalid")


TC5_MAX_ROWS = 256


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None,
             scratch: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulators in TMEM),
    M <= 256, bfloat16 inputs, out bfloat16 or float32. `scratch`: float32 buffer of `gemm_tc5_scratch_bytes` bytes
    (needed when the kernel slices K to fill the SMs)."""
    _need_cuda(x, w, out, bias, scratch)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_tc5: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_tc5: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tc5: bias float32 [N]")
    need = gemm_tc5_scratch_bytes(M, N, K)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() * 4 < need):
        raise KernelError(f"gemm_tc5: needs {need} bytes of float32 scratch")
    f = _fn("gemm_tc5", "il_gemm_tc5", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, _ptr(scratch), _ptr(stream_status(x.device)), _stream()), "gemm_tc5")


def gemm_tc5_scratch_bytes(M: int, N: int, K: int) -> int:
    lib = build.load("gemm_tc5")
    fn = lib.il_gemm_tc5_scratch_bytes
    fn.argtypes, fn.restype = [_c_int, _c_int, _c_int], ctypes.c_longlong
    return int(fn(M, N, K))


def tc5_ok(M: int, K: int) -> bool:
    return SKINNY_MAX_ROWS < M <= TC5_MAX_ROWS and K % 8 == 0



MID_MAX_ROWS = 128


def mid_ok(M: int, K: int) -> bool:
    return SKINNY_MAX_ROWS < M <= MID_MAX_ROWS and K % 8 == 0


def gemm_mid(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None,
             glu: bool = False, nb: int = 0, bm: int = 0) -> None:
    """out[M,N] = alpha * x[M,K] @ w[N,K]^T (+ bias) for 17..128 bfloat16 rows on the tcgen05 tensor cores: tiles of 64
    or 128 weight rows (`bm`; the A operand) by blocks of `nb` activation rows (0: chosen by the kernel) over all of K; out bfloat16
    or float32. glu: w is [2N,K] (gate rows, then up rows) and out[M,N] = silu(gate) * up (bfloat16)."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0] // 2 if glu else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_mid: bfloat16 x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_mid: innermost dimension must be contiguous")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.shape[0]):
        raise KernelError("gemm_mid: bias float32, one per weight row")
    f = _fn("gemm_mid", "il_gemm_mid", [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_float,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), kind_of(out.dtype), out.stride(0), _ptr(bias), alpha,
             M, N, K, int(glu), nb, bm, _ptr(stream_status(x.device)), _stream()), "gemm_mid")


# ----------------------------------------------------------------------------------------------
def _np_ptr(a) -> _c_void_p:
    return _c_void_p(a.ctypes.data)


def step_fill(out, out_cap: int, E: int, Ep: int, Tp: int, order, n_tok, start, slot, fresh, tokens, tok_off, widths, tbl_ptr,
              tbl_len, scratch_page, scratch_slot: int, want, want_off, pad_at: int, n_want_fixed: int, n_patch_cap: int, offsets,
              outs) -> int:
    """Native host code (csrc/step_fill.cpp): fills a step's descriptors into the int32 host array `out` from columns
    given as numpy arrays (int32 unless said: `fresh` uint8, `tokens` int64, `tbl_ptr` uint64 addresses of the block
    tables' arrays). The Ep - E padding entries of a step that is replayed as a graph run behind the first `pad_at`
    entries; `n_want_fixed` is such a step's number of wanted rows (-1: as many as are asked for). `offsets` (int32 [12]) receives where each part starts, `outs` (int32 [3]) the number of device
    tokens, of wanted rows, and the entry at fault. Returns 0 or the negative code of the fault."""
    for name, a, dt in (("order", order, "int32"), ("n_tok", n_tok, "int32"), ("start", start, "int32"), ("slot", slot, "int32"),
                        ("fresh", fresh, "uint8"), ("tokens", tokens, "int64"), ("tok_off", tok_off, "int32"),
                        ("widths", widths, "int32"), ("tbl_ptr", tbl_ptr, "uint64"), ("tbl_len", tbl_len, "int32"),
                        ("scratch_page", scratch_page, "int32"), ("want", want, "int32"), ("want_off", want_off, "int32"),
                        ("offsets", offsets, "int32"), ("outs", outs, "int32"), ("out", out, "int32")):
        if a.dtype.name != dt or not a.flags["C_CONTIGUOUS"]:
            raise KernelError(f"step_fill: {name} must be a contiguous {dt} array")
    if (len(order) != E or len(n_tok) != E or len(start) != E or len(slot) != E or len(fresh) != E or len(tok_off) != E + 1
            or len(want_off) != E + 1 or tbl_ptr.size != widths.size * E or tbl_len.size != widths.size * E
            or scratch_page.size != widths.size or offsets.size < 12 or outs.size < 3 or out.size < out_cap):
        raise KernelError("step_fill: array sizes do not match the number of entries and groups")
    lib = build.load("step_fill")
    f = lib.il_step_fill
    if not getattr(f, "_sig", False):
        f.argtypes = ([_c_void_p, ctypes.c_longlong, _c_int, _c_int, _c_int] + [_c_void_p] * 7 + [_c_int] + [_c_void_p] * 4 + [_c_int]
                      + [_c_void_p] * 2 + [_c_int, _c_int, _c_int] + [_c_void_p] * 4)
        f.restype = _c_int
        f._sig = True
    return int(f(_np_ptr(out), out_cap, E, Ep, Tp, _np_ptr(order), _np_ptr(n_tok), _np_ptr(start), _np_ptr(slot), _np_ptr(fresh),
                 _np_ptr(tokens), _np_ptr(tok_off), int(widths.size), _np_ptr(widths), _np_ptr(tbl_ptr), _np_ptr(tbl_len),
                 _np_ptr(scratch_page), scratch_slot, _np_ptr(want), _np_ptr(want_off), int(pad_at), int(n_want_fixed), n_patch_cap,
                 _c_void_p(offsets.ctypes.data), _c_void_p(outs.ctypes.data), _c_void_p(outs.ctypes.data + 4),
                 _c_void_p(outs.ctypes.data + 8)))
