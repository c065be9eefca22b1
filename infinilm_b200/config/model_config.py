"""Typed model configuration read from an architecture's own config.json keys.

A configuration class declares its fields once (name, type, default or
"required") and `from_json` fills them, so no model size or constant that
config.json carries is ever written down in code.

Parity with InfiniLM: `csrc/config/model_config.hpp:29-68` (typed getters that
throw on a missing key or a wrong type), `csrc/config/model_config.cpp:28-57`
(dtype from `dtype` / `torch_dtype`, rotary dim from `partial_rotary_factor`),
`csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:137-164` and
`python/infinilm/infer_engine.py:73-100` (defaults of the MiniCPM family).
"""
from __future__ import annotations

import dataclasses
import json
import math
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


def _take(raw: Dict[str, Any], key: str, typ, default=_REQUIRED):
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
                           _take(raw, "original_max_position_embeddings", int),
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


@dataclass
class MiniCPM4Config(ModelConfig):
    """MiniCPM4 (`MiniCPMForCausalLM`): GQA dense decoder, RMSNorm, SwiGLU,
    RoPE/LongRoPE and muP scale factors."""
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    scale_emb: float = 1.0
    scale_depth: float = 1.0
    dim_model_base: Optional[float] = None
    attention_bias: bool = False
    attention_output_bias: bool = False
    mlp_bias: bool = False
    tie_word_embeddings: bool = False

    # -- derived values ---------------------------------------------------------------
    @property
    def rotary_dim(self) -> int:
        """`csrc/config/model_config.cpp:41-57`."""
        f = self.partial_rotary_factor
        if f <= 0.0 or f >= 1.0:
            return self.head_dim
        r = int(round(self.head_dim * f))
        r = min(max(r, 2), self.head_dim)
        if r % 2:
            r -= 1
        return max(r, 2)

    @property
    def residual_scale(self) -> float:
        """scale_depth / sqrt(num_hidden_layers) (`minicpm4_for_causal_lm.cpp:12-20`)."""
        return self.scale_depth / math.sqrt(self.num_hidden_layers)

    @property
    def logit_scale(self) -> float:
        """dim_model_base / hidden_size, 1 when the key is absent (`:117-120`)."""
        if self.dim_model_base is None:
            return 1.0
        return self.dim_model_base / float(self.hidden_size)

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "MiniCPM4Config":
        raw = dict(raw)
        mt = _take(raw, "model_type", str)
        if mt not in ("minicpm", "minicpm4"):
            raise ConfigError(f"config.json: model_type {mt!r} is not a MiniCPM4 model")
        if raw.get("quantization_config") is not None:
            raise ConfigError("config.json: quantization_config is set; quantized weights are not supported")
        archs = raw.get("architectures") or ["MiniCPMForCausalLM"]
        hidden = _take(raw, "hidden_size", int)
        heads = _take(raw, "num_attention_heads", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: hidden_size and num_attention_heads must be positive")
        head_dim = _take(raw, "head_dim", int, hidden // heads)
        kv = _take(raw, "num_key_value_heads", int)
        if kv <= 0 or heads % kv != 0:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv})")
        # `bias` sets both attention_bias and mlp_bias (minicpm4_for_causal_lm.cpp:150-153).
        if "bias" in raw and raw["bias"] is not None:
            b = _take(raw, "bias", bool)
            raw["attention_bias"] = b
            raw["mlp_bias"] = b
        dt = raw.get("dtype", raw.get("torch_dtype"))
        if dt is None:
            raise ConfigError("config.json: neither 'dtype' nor 'torch_dtype' is given")
        eos = raw.get("eos_token_id", [])
        if eos is None:
            eos = []
        if isinstance(eos, int):
            eos = [eos]
        prf = _take(raw, "partial_rotary_factor", float, 1.0)
        cfg = cls(
            architecture=str(archs[0]), model_type="minicpm4",
            vocab_size=_take(raw, "vocab_size", int), hidden_size=hidden,
            max_position_embeddings=_take(raw, "max_position_embeddings", int),
            torch_dtype=parse_dtype_name(dt), eos_token_ids=[int(e) for e in eos], raw=raw,
            num_hidden_layers=_take(raw, "num_hidden_layers", int),
            num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim,
            intermediate_size=_take(raw, "intermediate_size", int),
            rms_norm_eps=_take(raw, "rms_norm_eps", float),
            rope_theta=_take(raw, "rope_theta", float, 10000.0),
            partial_rotary_factor=prf,
            scale_emb=_take(raw, "scale_emb", float, 1.0),
            scale_depth=_take(raw, "scale_depth", float, 1.0),
            dim_model_base=(None if raw.get("dim_model_base") is None
                            else _take(raw, "dim_model_base", float)),
            attention_bias=_take(raw, "attention_bias", bool, False),
            attention_output_bias=_take(raw, "attention_output_bias", bool, False),
            mlp_bias=_take(raw, "mlp_bias", bool, False),
            tie_word_embeddings=_take(raw, "tie_word_embeddings", bool, False),
        )
        cfg.rope_scaling = RopeScaling.from_json(raw.get("rope_scaling"), cfg.rotary_dim)
        if cfg.num_hidden_layers <= 0 or cfg.intermediate_size <= 0 or cfg.vocab_size <= 0:
            raise ConfigError("config.json: num_hidden_layers, intermediate_size and vocab_size must be positive")
        return cfg


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
