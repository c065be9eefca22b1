"""MiniCPM4 (`MiniCPMForCausalLM`) described as data: its parts layer by layer.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp` - `:12-20` residual
scale scale_depth/sqrt(layers), `:36-47` a layer is norm, attention, norm, MLP, `:73-87`
embedding, layers, final norm, `:107-121` head with alpha dim_model_base/hidden, `:137-164`
configuration defaults (also `python/infinilm/infer_engine.py:73-100`), `:168-173` registration under "minicpm4";
`python/infinilm/infer_engine.py:83-88` ("minicpm" is this architecture too). Tensor names are those of the checkpoint
(`minicpm4_for_causal_lm.hpp:50-53,66-68,83-84`, `csrc/layers/attention/attention.cpp:31-34`,
`csrc/layers/mlp/mlp.cpp:21-23`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

from ..config.model_config import ConfigError, ModelConfig, RopeScaling, parse_dtype_name, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


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
        mt = take(raw, "model_type", str)
        if mt not in ("minicpm", "minicpm4"):
            raise ConfigError(f"config.json: model_type {mt!r} is not a MiniCPM4 model")
        if raw.get("quantization_config") is not None:
            raise ConfigError("config.json: quantization_config is set; quantized weights are not supported")
        archs = raw.get("architectures") or ["MiniCPMForCausalLM"]
        hidden = take(raw, "hidden_size", int)
        heads = take(raw, "num_attention_heads", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: hidden_size and num_attention_heads must be positive")
        head_dim = take(raw, "head_dim", int, hidden // heads)
        kv = take(raw, "num_key_value_heads", int)
        if kv <= 0 or heads % kv != 0:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv})")
        # `bias` sets both attention_bias and mlp_bias (minicpm4_for_causal_lm.cpp:150-153).
        if "bias" in raw and raw["bias"] is not None:
            b = take(raw, "bias", bool)
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
        prf = take(raw, "partial_rotary_factor", float, 1.0)
        cfg = cls(
            architecture=str(archs[0]), model_type="minicpm4",
            vocab_size=take(raw, "vocab_size", int), hidden_size=hidden,
            max_position_embeddings=take(raw, "max_position_embeddings", int),
            torch_dtype=parse_dtype_name(dt), eos_token_ids=[int(e) for e in eos], raw=raw,
            num_hidden_layers=take(raw, "num_hidden_layers", int),
            num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim,
            intermediate_size=take(raw, "intermediate_size", int),
            rms_norm_eps=take(raw, "rms_norm_eps", float),
            rope_theta=take(raw, "rope_theta", float, 10000.0),
            partial_rotary_factor=prf,
            scale_emb=take(raw, "scale_emb", float, 1.0),
            scale_depth=take(raw, "scale_depth", float, 1.0),
            dim_model_base=(None if raw.get("dim_model_base") is None
                            else take(raw, "dim_model_base", float)),
            attention_bias=take(raw, "attention_bias", bool, False),
            attention_output_bias=take(raw, "attention_output_bias", bool, False),
            mlp_bias=take(raw, "mlp_bias", bool, False),
            tie_word_embeddings=take(raw, "tie_word_embeddings", bool, False),
        )
        cfg.rope_scaling = RopeScaling.from_json(raw.get("rope_scaling"), cfg.rotary_dim)
        if cfg.num_hidden_layers <= 0 or cfg.intermediate_size <= 0 or cfg.vocab_size <= 0:
            raise ConfigError("config.json: num_hidden_layers, intermediate_size and vocab_size must be positive")
        return cfg




def position_spec(cfg: MiniCPM4Config) -> PartSpec:
    rs = cfg.rope_scaling
    if rs.kind == "longrope":
        return PartSpec("longrope", {
            "rot_dim": cfg.rotary_dim, "theta": cfg.rope_theta,
            "short_factor": rs.short_factor, "long_factor": rs.long_factor,
            "original_max_position_embeddings": rs.original_max_position_embeddings,
            "max_position_embeddings": cfg.max_position_embeddings, "factor": rs.factor})
    return PartSpec("rope", {"rot_dim": cfg.rotary_dim, "theta": cfg.rope_theta})


def describe(cfg: MiniCPM4Config) -> ModelSpec:
    H = cfg.hidden_size
    pos = position_spec(cfg)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            arrangement="prenorm_residual",
            mixer_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, f"{p}.input_layernorm"),
            mixer=PartSpec("attention", {
                "hidden": H, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "qkv_bias": cfg.attention_bias, "out_bias": cfg.attention_output_bias,
                "window": None, "position": pos}, f"{p}.self_attn"),
            ffn_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, f"{p}.post_attention_layernorm"),
            ffn=PartSpec("swiglu", {"hidden": H, "intermediate": cfg.intermediate_size, "bias": cfg.mlp_bias}, f"{p}.mlp"),
            params={"residual_scale": cfg.residual_scale}))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": H, "scale": cfg.scale_emb},
                           "model.embed_tokens"),
        layers=layers,
        order=[RunStep(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, "model.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": H, "scale": cfg.logit_scale,
                                      "tied_to": head_fallback(cfg)}, "lm_head"))


def head_fallback(cfg: MiniCPM4Config) -> Optional[str]:
    """Where the head's matrix comes from when the checkpoint has no lm_head.weight. InfiniLM takes the (unscaled)
    embedding table whenever lm_head.weight is absent and never reads tie_word_embeddings on this path
    (`python/infinilm/modeling_utils.py:342-351`). The same here, with one exception: a config.json that SAYS
    "tie_word_embeddings": false asks for a head of its own, and a checkpoint without one is then reported as
    incomplete instead of being run with the wrong matrix."""
    if cfg.raw.get("tie_word_embeddings") is False:
        return None
    return "model.embed_tokens.weight"


register_architecture(["MiniCPMForCausalLM", "minicpm", "minicpm4"], MiniCPM4Config, describe)
