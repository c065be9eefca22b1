"""Arrangements: how a layer's parts sit around the residual stream.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:49-57` (fused-residual
form: each norm first adds the previous branch to the residual, then normalises it) and `:59-71`
(the same as h += s*Attn(norm(h)); h += s*MLP(norm(h))). The branch scale s is a parameter of the
arrangement; InfiniLM passes it as the `alpha` of o_proj and down_proj (`:27,33`), here it
multiplies the branch in f32 inside the fused add, where the residual sum is kept in f32.
"""
from __future__ import annotations

from .base import Arrangement, register_part


class PreNormResidual(Arrangement):
    """params: residual_scale (default 1)."""

    def run(self, resid, pending, ctx, cache):
        s = float(self.params.get("residual_scale", 1.0))
        T, H = resid.shape
        branch, bscale = pending if pending is not None else (None, 1.0)
        normed = self.mixer_norm.add_norm(resid, branch, bscale, ctx.ws.rows("normed", T, H, ctx.dtype))
        branch = self.mixer.forward(normed, ctx, cache)
        normed = self.ffn_norm.add_norm(resid, branch, s, ctx.ws.rows("normed", T, H, ctx.dtype))
        branch = self.ffn.forward(normed, ctx)
        return branch, s


register_part("arrangement", "prenorm_residual", PreNormResidual)
