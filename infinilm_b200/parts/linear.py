"""y = alpha * x W^T (+ b): the matrix product every projection is made of.

Parity with InfiniLM: `csrc/layers/linear/base_linear.cpp:35-44` and
`csrc/layers/quantization/none_quantization.cpp:26-46` (weight [out,in], optional bias, a scale
`alpha` passed into the product). The float32 path runs the FFMA kernel of this package. On the
bfloat16 path up to 16 rows (decode) run this package's weight-streaming kernel, 17 to 256 rows run
its tcgen05/TMA kernels where that is enabled (the output head: `gemm_mid` up to 64 rows, `gemm_tc5`
beyond), and everything else calls the library matrix product, as InfiniLM does for its linears.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops


class Linear:
    MID_ROWS = 64                                 # up to here `gemm_mid` measured faster than `gemm_tc5` on the vocabulary-sized head

    def __init__(self, in_features: int, out_features: int, dtype: torch.dtype, alpha: float = 1.0, use_tc5: bool = False):
        self.in_features, self.out_features = in_features, out_features
        self.dtype, self.alpha = dtype, float(alpha)
        self.weight: Optional[torch.Tensor] = None      # [out, in], compute dtype
        self.bias: Optional[torch.Tensor] = None        # [out], float32 or compute dtype
        # 17..256 rows on the bfloat16 path: this package's tcgen05/TMA kernel where it is the faster one
        # (measured: the vocabulary-sized head), the library product elsewhere; INFINILM_B200_TC5=1 uses it everywhere, =0 nowhere.
        env = os.environ.get("INFINILM_B200_TC5")
        self.use_tc5 = (use_tc5 and env != "0") or env == "1"
        self._tc5_scratch: Optional[torch.Tensor] = None

    def set(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"linear weight {tuple(weight.shape)} != {(self.out_features, self.in_features)}")
        self.weight = weight.to(self.dtype).contiguous()
        self._weight_t = self.weight.t()          # the view the library product takes, made once
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
        if self.use_tc5 and x.shape[0] <= self.MID_ROWS and ops.mid_ok(x.shape[0], self.in_features):
            # 17..64 rows: tiles of weight rows by blocks of activation rows over all of K, nothing cut along K
            ops.gemm_mid(x, self.weight, out, self.alpha, self.bias)
            return out
        if self.use_tc5 and ops.tc5_ok(x.shape[0], self.in_features) and (out_f32 or out.dtype == torch.bfloat16):
            if self._tc5_scratch is None:
                need = max(ops.gemm_tc5_scratch_bytes(m, self.out_features, self.in_features) for m in (32, 64, 128, 256))
                self._tc5_scratch = torch.empty(max(need // 4, 1), dtype=torch.float32, device=x.device)
            ops.gemm_tc5(x, self.weight, out, self.alpha, self.bias, self._tc5_scratch)
            return out
        # Library matrix product (cuBLAS through torch), f32 accumulation inside.
        if out_f32:
            torch.mm(x, self._weight_t, out_dtype=torch.float32, out=out)
            if self.alpha != 1.0:
                out.mul_(self.alpha)
        elif self.alpha != 1.0:
            torch.addmm(out, x, self._weight_t, beta=0.0, alpha=self.alpha, out=out)
        else:
            torch.mm(x, self._weight_t, out=out)
        if self.bias is not None:
            ops.add_bias(out, self.bias)
        return out
