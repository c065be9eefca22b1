"""Data that describes a model: which parts each layer is made of and the order layers run in.

An architecture's `describe(config)` returns a `ModelSpec`. Nothing in it is code: a part is
named by its kind (a key of the part registries) and carries its sizes and constants as
parameters, so two layers of one model may use different mixers or feed-forwards, and the run
order may name a layer twice or let a layer read another entry's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    kind: str                                   # registry key, e.g. "attention", "swiglu", "rmsnorm"
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""                            # checkpoint name prefix of this part's tensors


@dataclass
class LayerSpec:
    """One block: two norms, a mixer and a feed-forward, and how they are arranged."""
    arrangement: str                            # registry key of the block, e.g. "prenorm_residual"
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: PartSpec
    ffn: PartSpec
    params: Dict[str, Any] = field(default_factory=dict)   # e.g. {"residual_scale": s}


@dataclass
class RunStep:
    """One entry of the run order. `layer` indexes `ModelSpec.layers`.

    `cache_from` names an earlier entry of the order whose cache this entry reads instead of
    keeping its own (it then writes nothing)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[RunStep]
    final_norm: PartSpec
    head: PartSpec


@dataclass
class WeightSpec:
    """One checkpoint tensor a part wants.

    role: "matrix" (operand of a matrix product: held in the compute dtype), "vector" (norm
          weights, biases: a tensor stored in 32-bit stays 32-bit), "table" (integer table: int32).
    init: ("normal", std) | ("ones_normal", std) | ("zeros",) - used by the random-weights mode.
    fallback: another tensor's full name used when this one is absent (a tied head)."""
    name: str                                   # local name, e.g. "q_proj.weight"
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    fallback: Optional[str] = None


@dataclass
class CacheNeed:
    """What a mixer keeps between steps, per request.

    kind "paged_kv": keys and values in pages; `window` None keeps all keys, else only the last
    `window` positions are ever read, so pages behind the window are given back.
    kind "state": one fixed-size tensor of `shape` per request (slot 0 of the pool is the zero state)."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    dtype: str = "compute"                      # "compute" | "float32"

    def group_key(self) -> Tuple:
        return (self.kind, self.n_kv_heads, self.head_dim, self.window, tuple(self.shape), self.dtype)
