"""Rotary position encodings: plain RoPE and LongRoPE, as frequency tables a mixer applies.

Parity with InfiniLM: `csrc/layers/rotary_embedding/rotary_embedding.cpp:50-113` (one rotary
object from head_dim, rotary_dim, max positions, theta, scaling), `rope_scaling_creators.cpp:23-47`
(LongRoPE takes short_factor, long_factor, original_max_position_embeddings, factor),
`csrc/config/model_config.hpp:139` (rotate-half pairing). The table arithmetic itself is inside
InfiniCore; here it is
    inv_freq[i] = 1 / (f[i] * theta^(2i/rot_dim)),  angle = position * inv_freq[i]
with f = 1 for plain RoPE. For LongRoPE, f is `long_factor` when the model's
max_position_embeddings exceeds original_max_position_embeddings, else `short_factor`, and
cos/sin are multiplied by sqrt(1 + ln(s) / ln(original_max)) with s = max/original (or `factor`
when given and not 1) if s > 1. The choice depends on the configuration only, never on the
length of the sequence at hand, so a position's encoding is the same however the work is cut.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .base import PositionEncoding, register_part


def rotary_inv_freq(rot_dim: int, theta: float, factors: Optional[List[float]]) -> List[float]:
    half = rot_dim // 2
    out = []
    for i in range(half):
        f = 1.0 if factors is None else float(factors[i])
        out.append(1.0 / (f * (float(theta) ** (2.0 * i / rot_dim))))
    return out


def longrope_choice(short_factor, long_factor, original_max: int, max_pos: int, factor: Optional[float]):
    """(factors, mscale) of a LongRoPE configuration."""
    s = max_pos / float(original_max)
    if factor is not None and factor != 1.0:
        s = float(factor)
    factors = long_factor if max_pos > original_max else short_factor
    mscale = math.sqrt(1.0 + math.log(s) / math.log(original_max)) if s > 1.0 else 1.0
    return factors, mscale


class Rope(PositionEncoding):
    """params: rot_dim, theta."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.rot_dim = int(params["rot_dim"])
        self.theta = float(params["theta"])
        self.mscale = 1.0
        self._table = rotary_inv_freq(self.rot_dim, self.theta, None)
        self.inv_freq = None

    def to_device(self, device):
        self.inv_freq = torch.tensor(self._table, dtype=torch.float64).to(torch.float32).to(device)


class LongRope(Rope):
    """params: rot_dim, theta, short_factor, long_factor, original_max_position_embeddings,
    max_position_embeddings, factor (optional)."""

    def __init__(self, params, prefix, dtype):
        PositionEncoding.__init__(self, params, prefix, dtype)
        self.rot_dim = int(params["rot_dim"])
        self.theta = float(params["theta"])
        factors, self.mscale = longrope_choice(params["short_factor"], params["long_factor"],
                                               int(params["original_max_position_embeddings"]),
                                               int(params["max_position_embeddings"]), params.get("factor"))
        if len(factors) != self.rot_dim // 2:
            raise ValueError("longrope: factor list must have rot_dim/2 entries")
        self._table = rotary_inv_freq(self.rot_dim, self.theta, factors)
        self.inv_freq = None


class NoPosition(PositionEncoding):
    """No position encoding (rot_dim 0)."""

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.rot_dim, self.mscale, self.inv_freq = 0, 1.0, None


register_part("position", "rope", Rope)
register_part("position", "longrope", LongRope)
register_part("position", "none", NoPosition)
