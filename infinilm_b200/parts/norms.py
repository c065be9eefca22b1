"""RMSNorm, fused with the residual add that precedes it.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:43,45,52,54,86,99`
(`RMSNorm(hidden_size, rms_norm_eps)` used through `forward_inplace(hidden, residual)`):
y = x / sqrt(mean(x^2) + eps) * w, no bias.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Norm, register_part
from .spec import WeightSpec


class RMSNorm(Norm):
    """params: size, eps."""
    fusable_rms = True
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec("weight", (self.size,), role="vector", init=("ones_normal", 0.01))]

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors["weight"]
        if w.dtype not in (torch.float32, torch.bfloat16):
            w = w.to(torch.float32)
        if self.dtype == torch.float32:
            w = w.to(torch.float32)
        self.weight = w.contiguous()

    def add_norm(self, resid, branch, branch_scale, out, rows=None):
        ops.add_rmsnorm(resid, branch, branch_scale, self.weight, self.eps, out, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
