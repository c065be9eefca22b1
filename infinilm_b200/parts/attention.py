"""Grouped-query attention over the paged cache.

Parity with InfiniLM: `csrc/layers/attention/attention.cpp:7-46` (fused QKV projection, o_proj,
scale 1/sqrt(head_dim)), `:96-137` (project, view as heads, rotate q and k in place, attend,
project out), `csrc/layers/attention/backends/paged_attn.cpp:20-84` (write k/v to their slots,
then attend over the pages), `csrc/layers/linear/fused_linear.cpp:57-71,102-110` (q, k, v are row
ranges of one weight).
"""
from __future__ import annotations

import math
import os
import warnings
from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Mixer, build_part, register_part
from .linear import Linear
from .spec import CacheNeed, PartSpec, WeightSpec


class Attention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, qkv_bias, out_bias, out_scale,
    window (None = all keys), position (PartSpec of a position encoding)."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.nkv, self.hd = int(p["hidden"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"attention: head_dim {self.hd} is not supported (multiples of 16 from 16 to 256)")
        self.qkv_bias, self.out_bias = bool(p.get("qkv_bias", False)), bool(p.get("out_bias", False))
        self.window: Optional[int] = p.get("window")
        self.force_plain = bool(p.get("plain_kernel", False))
        self.prefill_kernel = str(p.get("prefill_kernel", os.environ.get("INFINILM_B200_PREFILL_ATTN", "auto")))   # "mma": never tcgen05
        self.fuse_rope = os.environ.get("INFINILM_B200_FUSE_ROPE", "1") != "0"
        self.scale = 1.0 / math.sqrt(self.hd)
        self.n_qkv = (self.nh + 2 * self.nkv) * self.hd
        self.qkv = Linear(self.hidden, self.n_qkv, dtype)
        self.o_proj = Linear(self.nh * self.hd, self.hidden, dtype, alpha=float(p.get("out_scale", 1.0)))
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = build_part("position", pos, dtype)
        if self.position.rot_dim > self.hd:
            raise ValueError("attention: rotary dim exceeds head_dim")
        if self.position.has_transform and self.position.rot_dim:
            raise ValueError("attention: a position encoding is a rotary table or a transform, not both")

    def weight_specs(self) -> List[WeightSpec]:
        hd, H = self.hd, self.hidden
        specs = [WeightSpec("q_proj.weight", (self.nh * hd, H)), WeightSpec("k_proj.weight", (self.nkv * hd, H)),
                 WeightSpec("v_proj.weight", (self.nkv * hd, H)), WeightSpec("o_proj.weight", (H, self.nh * hd))]
        if self.qkv_bias:
            specs += [WeightSpec("q_proj.bias", (self.nh * hd,), "vector"), WeightSpec("k_proj.bias", (self.nkv * hd,), "vector"),
                      WeightSpec("v_proj.bias", (self.nkv * hd,), "vector")]
        if self.out_bias:
            specs.append(WeightSpec("o_proj.bias", (H,), "vector"))
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        w = torch.cat([t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([t["q_proj.bias"].float(), t["k_proj.bias"].float(), t["v_proj.bias"].float()])
        self.qkv.set(w, b)
        self.o_proj.set(t["o_proj.weight"], t.get("o_proj.bias"))
        self.position.to_device(w.device)

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("paged_kv", n_kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    @property
    def graph_safe(self):
        return self.position.graph_safe or not self.position.has_transform

    def accepts_normed(self, T):
        return (self.dtype == torch.bfloat16 and self.fuse_rope and not self.position.has_transform
                and ops.skinny_rope_ok(T, self.hidden, self.hd, self.position.rot_dim))

    def fuses_tail(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_resid_ok(T, self.nh * self.hd, self.hidden)

    def forward(self, x, ctx, cache, tail=None):
        T = x.shape[0]
        pos = self.position
        qkv = ctx.ws.rows("qkv", T, self.n_qkv, self.dtype)
        store = cache.storage if cache.writable else None
        if (self.dtype == torch.bfloat16 and self.fuse_rope and not pos.has_transform
                and ops.skinny_rope_ok(T, self.hidden, self.hd, pos.rot_dim)):
            # a few rows (decode): the projection rotates q and k and writes k, v to the cache in its epilogue
            normed = isinstance(x, ops.NormedInput)
            ops.gemm_skinny_rope(x.xw if normed else x, self.qkv.weight, qkv, self.qkv.alpha, self.qkv.bias, ctx.tok_pos,
                                 ctx.tok_entry, cache.block_table, store, cache.page_size, self.nh, self.nkv, self.hd,
                                 pos.rot_dim, pos.inv_freq, pos.mscale, norm_in=x if normed else None)
        else:
            self.qkv(x, qkv)
            if pos.has_transform:                 # an encoding that is no rotary table changes q and k itself
                pos.transform(qkv, ctx, self.nh, self.nkv, self.hd)
            ops.rope_store(qkv, ctx.tok_pos, ctx.tok_entry, cache.block_table, store, cache.page_size,
                           self.nh, self.nkv, self.hd, pos.rot_dim, pos.inv_freq, pos.mscale)
        out = ctx.ws.rows("attn_out", T, self.nh * self.hd, self.dtype)
        self.attend(qkv, out, ctx, cache)
        if tail is not None:                      # o_proj adds into the residual and prepares the next norm itself
            return ops.gemm_skinny_resid(out, self.o_proj.weight, self.o_proj.alpha, self.o_proj.bias, tail.resid, tail.scale,
                                         tail.norm.weight, tail.norm.eps, ctx.ws.rows("xw_mixer", T, self.hidden, self.dtype),
                                         ctx.ws.rows("sumsq_mixer", T, (self.hidden + 15) // 16, torch.float32))
        return self.o_proj(out, ctx.ws.rows("branch", T, self.hidden, self.dtype))

    # The fast bfloat16 kernels take kernel pages of 16 keys (the cache manager lays larger pages out as runs of them)
    # and at most 64 query heads per kv head; anything else, and the whole float32 path, runs the plain kernel.
    FAST_PAGE = 16
    FAST_MAX_GROUP = 64
    _warned_plain = False

    WAVE_FILL = 2.0 / 3.0                         # share of the blocks the device holds at once that the splits aim at

    def decode_splits(self, base: int, max_pages: int, resident: int) -> int:
        """Splits of the keys for `base` blocks per split: as many as fill the wanted share of one wave of blocks
        (`resident`: what the device runs at once, from the occupancy query), never more - a second, part-filled wave
        costs more in partials than it gains - and at least four pages a split."""
        target = max(1, int(resident * self.WAVE_FILL))
        return max(1, min(target // base, (max_pages + 3) // 4, 128))

    def attend(self, qkv, out, ctx, cache) -> None:
        G = self.nh // self.nkv
        if (self.dtype != torch.bfloat16 or cache.page_size != self.FAST_PAGE or G > self.FAST_MAX_GROUP
                or self.force_plain):
            if self.dtype == torch.bfloat16 and not self.force_plain and not Attention._warned_plain:
                Attention._warned_plain = True
                warnings.warn(f"attention: pages of {cache.page_size} keys / {G} query heads per kv head are outside the fast "
                              f"bfloat16 kernels (pages of 16 or a multiple, at most {self.FAST_MAX_GROUP} heads per kv head): "
                              "the plain kernel runs, at a fraction of their speed", RuntimeWarning, stacklevel=2)
            ops.attention_plain(qkv, out, cache.storage, cache.block_table, ctx.tok_pos, ctx.tok_entry,
                                cache.page_size, self.nh, self.nkv, self.hd, self.scale, self.window)
            return
        n_dec, E = ctx.n_decode, ctx.n_entries
        if n_dec > 0:
            max_len = max(ctx.h_kvlen[:n_dec])
            if self.window is not None:
                max_len = min(max_len, self.window + self.FAST_PAGE)
            max_pages = (max_len + self.FAST_PAGE - 1) // self.FAST_PAGE + (1 if self.window is not None else 0)
            base = n_dec * self.nkv * ((G + 15) // 16)
            n_splits = self.decode_splits(base, max_pages, ops.attention_decode_resident_blocks(self.hd))
            rows = n_dec * self.nh * n_splits
            ops.attention_decode(qkv, out, cache.storage, cache.block_table, ctx.entry_kvlen, n_dec, cache.page_size,
                                 self.nh, self.nkv, self.hd, self.scale, self.window, 0, n_splits,
                                 ctx.ws.flat("attn_o_part", rows * self.hd, torch.float32),
                                 ctx.ws.flat("attn_ml_part", rows * 2, torch.float32), kv_map=cache.tma_map)
        if E > n_dec:
            # prompt portions: on tcgen05 with tensor memory where the head size has that kernel (64, 128) and the cache
            # its tensor map; else the mma.sync kernel. The tile is 128 (64) rows = tokens x heads of a kv head.
            tc5 = (self.prefill_kernel != "mma" and cache.tma_map is not None
                   and ops.prefill_tc5_ok(self.hd, G, cache.page_size, cache.tma_map))
            tpt = max(1, (ops.prefill_tc5_rows(self.hd) if tc5 else 64) // G)
            n_tiles = ctx.prompt_tiles(tpt)
            if tc5:
                ops.attention_prefill_tc5(qkv, out, cache.tma_map, cache.block_table, ctx.entry_qstart, ctx.entry_kvlen,
                                          n_dec, E, n_tiles, cache.page_size, self.nh, self.nkv, self.hd, self.scale,
                                          self.window)
            else:
                ops.attention_prefill(qkv, out, cache.storage, cache.block_table, ctx.entry_qstart, ctx.entry_kvlen,
                                      n_dec, E, n_tiles, cache.page_size, self.nh, self.nkv, self.hd, self.scale,
                                      self.window)


register_part("mixer", "attention", Attention)
