"""y = alpha * x W^T (+ b): the matrix product every projection is made of.

Parity with InfiniLM: `csrc/layers/linear/base_linear.cpp:35-44` and
`csrc/layers/quantization/none_quantization.cpp:26-46` (weight [out,in], optional bias, a scale
`alpha` passed into the product). The float32 path runs the FFMA kernel of this package. On the
bfloat16 path up to 16 rows (decode) run this package's weight-streaming kernel; more rows call
the library matrix product, as InfiniLM does for its linears.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class Linear:
    def __init__(self, in_features: int, out_features: int, dtype: torch.dtype, alpha: float = 1.0):
        self.in_features, self.out_features = in_features, out_features
        self.dtype, self.alpha = dtype, float(alpha)
        self.weight: Optional[torch.Tensor] = None      # [out, in], compute dtype
        self.bias: Optional[torch.Tensor] = None        # [out], float32 or compute dtype

    def set(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"linear weight {tuple(weight.shape)} != {(self.out_features, self.in_features)}")
        self.weight = weight.to(self.dtype).contiguous()
        if bias is not None:
            self.bias = bias.to(torch.float32).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
        """x [M,in] -> out [M,out]. `out_f32`: out is float32 even on the bfloat16 path."""
        if self.dtype == torch.float32:
            ops.gemm_f32(x, self.weight, out, self.alpha, self.bias)
            return out
        if ops.skinny_ok(x.shape[0], self.in_features):
            # a few rows (decode): the weight-streaming kernel of this package
            ops.gemm_skinny(x, self.weight, out, self.alpha, self.bias)
            return out
        # Library matrix product (cuBLAS through torch), f32 accumulation inside.
        if out_f32:
            torch.mm(x, self.weight.t(), out_dtype=torch.float32, out=out)
            if self.alpha != 1.0:
                out.mul_(self.alpha)
        elif self.alpha != 1.0:
            torch.addmm(out, x, self.weight.t(), beta=0.0, alpha=self.alpha, out=out)
        else:
            torch.mm(x, self.weight.t(), out=out)
        if self.bias is not None:
            ops.add_bias(out, self.bias)
        return out
