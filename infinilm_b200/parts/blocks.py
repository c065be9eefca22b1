"""Arrangements: how a layer's parts sit around the residual stream.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:49-57` (fused-residual
form: each norm first adds the previous branch to the residual, then normalises it) and `:59-71`
(the same as h += s*Attn(norm(h)); h += s*MLP(norm(h))). The branch scale s is a parameter of the
arrangement; InfiniLM passes it as the `alpha` of o_proj and down_proj (`:27,33`), here it
multiplies the branch in f32 inside the fused add, where the residual sum is kept in f32.
"""
from __future__ import annotations

import os

from .. import ops
from .base import Arrangement, ResidualTail, register_part


class PreNormResidual(Arrangement):
    """params: residual_scale (default 1)."""

    # On a decode step of a few rows an add+norm kernel between two weight-streaming products costs about as much as
    # its boundary to them; where the parts on both sides can, the product before does the add and the product after
    # the division by the rms (ResidualTail / NormedInput). INFINILM_B200_FUSE_NORM=0: always the kernel.
    FUSE_NORM = os.environ.get("INFINILM_B200_FUSE_NORM", "1") != "0"

    takes_next_norm = True

    def accepts_normed_input(self, T):
        return self.FUSE_NORM and self.mixer_norm.fusable_rms and self.mixer.accepts_normed(T)

    def run(self, resid, pending, ctx, cache, next_norm=None):
        s = float(self.params.get("residual_scale", 1.0))
        T, H = resid.shape
        fuse = self.FUSE_NORM and ctx.tap is None
        if isinstance(pending, ops.NormedInput):
            normed = pending
        else:
            branch, bscale = pending if pending is not None else (None, 1.0)
            normed = self.mixer_norm.add_norm(resid, branch, bscale, ctx.ws.rows("normed", T, H, ctx.dtype))
        if fuse and self.ffn_norm.fusable_rms and self.mixer.fuses_tail(T) and self.ffn.accepts_normed(T):
            normed = self.mixer.forward(normed, ctx, cache, tail=ResidualTail(resid, s, self.ffn_norm))
        else:
            branch = self.mixer.forward(normed, ctx, cache)
            normed = self.ffn_norm.add_norm(resid, branch, s, ctx.ws.rows("normed", T, H, ctx.dtype))
        if fuse and next_norm is not None and next_norm.fusable_rms and self.ffn.fuses_tail(T):
            return self.ffn.forward(normed, ctx, tail=ResidualTail(resid, s, next_norm))
        branch = self.ffn.forward(normed, ctx)
        return branch, s


register_part("arrangement", "prenorm_residual", PreNormResidual)
