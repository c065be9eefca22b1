"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)).

Parity with InfiniLM: `csrc/layers/mlp/mlp.cpp:7-38` (gate and up as one product, `swiglu(up, gate)`,
then down), `csrc/layers/linear/fused_linear.cpp:152-158,177-185` (gate rows first, up rows second).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from .base import FeedForward, register_part
from .linear import Linear
from .spec import WeightSpec


class SwiGLU(FeedForward):
    """params: hidden, intermediate, bias, out_scale."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.hidden, self.inter = int(params["hidden"]), int(params["intermediate"])
        self.bias = bool(params.get("bias", False))
        self.gate_up = Linear(self.hidden, 2 * self.inter, dtype)
        self.down = Linear(self.inter, self.hidden, dtype, alpha=float(params.get("out_scale", 1.0)))

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec("gate_proj.weight", (self.inter, self.hidden)), WeightSpec("up_proj.weight", (self.inter, self.hidden)),
                 WeightSpec("down_proj.weight", (self.hidden, self.inter))]
        if self.bias:
            specs += [WeightSpec("gate_proj.bias", (self.inter,), "vector"), WeightSpec("up_proj.bias", (self.inter,), "vector"),
                      WeightSpec("down_proj.bias", (self.hidden,), "vector")]
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        w = torch.cat([t["gate_proj.weight"], t["up_proj.weight"]], dim=0)
        b = torch.cat([t["gate_proj.bias"].float(), t["up_proj.bias"].float()]) if self.bias else None
        self.gate_up.set(w, b)
        self.down.set(t["down_proj.weight"], t.get("down_proj.bias"))

    def accepts_normed(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden)

    def fuses_tail(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden) and ops.skinny_resid_ok(T, self.inter, self.hidden)

    def forward(self, x, ctx, tail=None):
        T = x.shape[0]
        if self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden):
            # decode: gate and up rows streamed together, SiLU(gate)*up in the epilogue
            act = ctx.ws.rows("ffn_act", T, self.inter, self.dtype)
            if isinstance(x, ops.NormedInput):
                ops.gemm_skinny(x.xw, self.gate_up.weight, act, 1.0, self.gate_up.bias, glu=True, norm_in=x)
            else:
                ops.gemm_skinny(x, self.gate_up.weight, act, 1.0, self.gate_up.bias, glu=True)
            if tail is not None:                  # down adds into the residual and prepares the next norm itself
                return ops.gemm_skinny_resid(act, self.down.weight, self.down.alpha, self.down.bias, tail.resid, tail.scale,
                                             tail.norm.weight, tail.norm.eps,
                                             ctx.ws.rows("xw_ffn", T, self.hidden, self.dtype),
                                             ctx.ws.rows("sumsq_ffn", T, (self.hidden + 15) // 16, torch.float32))
            return self.down(act, ctx.ws.rows("branch", T, self.hidden, self.dtype))
        act = ctx.ws.rows("ffn_act", T, self.inter, self.dtype)
        if self.dtype == torch.bfloat16 and ops.mid_ok(T, self.hidden):
            # 17..128 rows: gate and up on the tcgen05 tensor cores as two accumulators in the same lanes, SiLU(gate)*up in
            # the epilogue (measured against the library product followed by the SwiGLU kernel at 8B sizes: 44.6 against
            # 48.4 us at 32 rows, 47.6 against 49.9 at 64, 52.5 against 57.6 at 128)
            ops.gemm_mid(x, self.gate_up.weight, act, 1.0, self.gate_up.bias, glu=True)
            return self.down(act, ctx.ws.rows("branch", T, self.hidden, self.dtype))
        gu = self.gate_up(x, ctx.ws.rows("gate_up", T, 2 * self.inter, self.dtype))
        ops.swiglu(gu, act)
        return self.down(act, ctx.ws.rows("branch", T, self.hidden, self.dtype))


register_part("feed_forward", "swiglu", SwiGLU)
