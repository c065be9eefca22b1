"""Typed model configuration read from an architecture's own config.json keys.

A configuration class declares its fields once (name, type, default or
"required") and `from_json` fills them, so no model size or constant that
config.json carries is ever written down in code.

Parity with InfiniLM: `csrc/config/model_config.hpp:29-68` (typed getters that
throw on a missing key or a wrong type), `csrc/config/model_config.cpp:28-57`
(dtype from `dtype` / `torch_dtype`, rotary dim from `partial_rotary_factor`).
An architecture's own configuration class lives beside its model description (`models/`).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: names the key and what is wrong."""


_DTYPE_NAMES = {
    "float32": "float32", "fp32": "float32", "torch.float32": "float32",
    "bfloat16": "bfloat16", "bf16": "bfloat16", "torch.bfloat16": "bfloat16",
    "float16": "float16", "fp16": "float16", "half": "float16", "torch.float16": "float16",
}


def parse_dtype_name(name: str) -> str:
    """Canonical dtype name; the strings InfiniLM accepts (`csrc/utils.hpp:150-167`)."""
    try:
        return _DTYPE_NAMES[str(name).lower()]
    except KeyError:
        raise ConfigError(f"unsupported dtype {name!r} (float32, float16, bfloat16)") from None


_REQUIRED = object()


def take(raw: Dict[str, Any], key: str, typ, default=_REQUIRED):
    """Read `key` with a type check; error text names the key."""
    if key not in raw or raw[key] is None:
        if default is _REQUIRED:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = raw[key]
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                return int(v)
            raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
        return int(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: key '{key}' must be true/false, got {v!r}")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: key '{key}' must be a string, got {v!r}")
        return v
    return v


@dataclass
class RopeScaling:
    """`rope_scaling` block. Only the kinds InfiniLM routes for this family:
    none/default and longrope (`rope_scaling_creators.cpp:12-47`)."""
    kind: str = "none"                        # "none" | "longrope"
    short_factor: Optional[List[float]] = None
    long_factor: Optional[List[float]] = None
    original_max_position_embeddings: Optional[int] = None
    factor: Optional[float] = None

    @staticmethod
    def from_json(raw: Optional[Dict[str, Any]], rotary_dim: int) -> "RopeScaling":
        if raw is None:
            return RopeScaling()
        if not isinstance(raw, dict):
            raise ConfigError("config.json: 'rope_scaling' must be an object")
        kind = raw.get("rope_type", raw.get("type", "default"))
        if kind in ("default", "none", "dynamic"):
            # InfiniLM maps these three to "no scaling" (rope_scaling_creators.cpp:106-115).
            return RopeScaling()
        if kind != "longrope":
            raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported "
                              "(none, default, longrope)")
        for k in ("short_factor", "long_factor", "original_max_position_embeddings"):
            if k not in raw:
                raise ConfigError("config.json: longrope needs 'short_factor', 'long_factor' "
                                  f"and 'original_max_position_embeddings' ('{k}' is missing)")
        sf = [float(x) for x in raw["short_factor"]]
        lf = [float(x) for x in raw["long_factor"]]
        half = rotary_dim // 2
        if len(sf) != half or len(lf) != half:
            raise ConfigError(f"config.json: longrope factors must have rotary_dim/2 = {half} "
                              f"entries (short has {len(sf)}, long has {len(lf)})")
        fac = raw.get("factor")
        return RopeScaling("longrope", sf, lf,
                           take(raw, "original_max_position_embeddings", int),
                           None if fac is None else float(fac))


@dataclass
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses add their fields and implement `from_json`. The fields here are
    those the engine itself needs regardless of the architecture."""
    architecture: str = ""
    model_type: str = ""
    vocab_size: int = 0
    hidden_size: int = 0
    max_position_embeddings: int = 0
    torch_dtype: str = "bfloat16"
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict, repr=False)

    def to_json(self) -> Dict[str, Any]:
        """The config.json content that reproduces this configuration."""
        return dict(self.raw)


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path, "r") as f:
        raw = json.load(f)
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen) and "eos_token_id" not in raw:
        # generation_config.json may carry the end-of-sequence ids (infer_engine.py:109-114).
        with open(gen, "r") as f:
            g = json.load(f)
        if g.get("eos_token_id") is not None:
            raw["eos_token_id"] = g["eos_token_id"]
    return raw


def config_fields(cfg: ModelConfig) -> Dict[str, Any]:
    """Flat dict of the typed fields (for logs and the benchmark record)."""
    out = {}
    for f in dataclasses.fields(cfg):
        if f.name == "raw":
            continue
        out[f.name] = getattr(cfg, f.name)
    return out
