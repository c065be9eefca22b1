"""Token embedding and output head.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:81,92` (embedding),
`python/infinilm/modeling_utils.py:15-23,258-263` (the table is multiplied by scale_emb when it
is loaded, in the model dtype) - here the table stays as stored and the gather multiplies in
f32, rounding through the model dtype once, which gives the value the pre-scaled table holds;
`minicpm4_for_causal_lm.cpp:117-125` (lm_head with alpha = dim_model_base / hidden),
`modeling_utils.py:342-351` (an absent lm_head.weight is taken from the unscaled embedding).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Part, register_part
from .linear import Linear
from .spec import WeightSpec


class TokenEmbedding(Part):
    """params: vocab, hidden, scale."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.vocab, self.hidden, self.scale = int(params["vocab"]), int(params["hidden"]), float(params.get("scale", 1.0))
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec("weight", (self.vocab, self.hidden))]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t["weight"].to(self.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
        ops.embed(token_ids, self.table, self.scale, resid, round_bf16=(self.dtype == torch.bfloat16))
        return resid


class OutputHead(Part):
    """params: vocab, hidden, scale, tied_to (full name of the embedding table or None).
    Logits are float32 on both paths."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.linear = Linear(self.hidden, self.vocab, dtype, alpha=float(params.get("scale", 1.0)), use_tc5=True)
        self.tied_to = params.get("tied_to")

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec("weight", (self.vocab, self.hidden), fallback=self.tied_to)]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.linear.set(t["weight"])

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        return self.linear(x, out, out_f32=True)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", OutputHead)
