"""MiniCPM4 (`MiniCPMForCausalLM`) described as data: its parts layer by layer.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp` - `:12-20` residual
scale scale_depth/sqrt(layers), `:36-47` a layer is norm, attention, norm, MLP, `:73-87`
embedding, layers, final norm, `:107-121` head with alpha dim_model_base/hidden, `:137-164`
configuration defaults, `:168-173` registration under "minicpm4"; `python/infinilm/infer_engine.py:83-88`
("minicpm" is this architecture too). Tensor names are those of the checkpoint
(`minicpm4_for_causal_lm.hpp:50-53,66-68,83-84`, `csrc/layers/attention/attention.cpp:31-34`,
`csrc/layers/mlp/mlp.cpp:21-23`).
"""
from __future__ import annotations

from ..config.model_config import MiniCPM4Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


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
                                      "tied_to": "model.embed_tokens.weight"}, "lm_head"))


register_architecture(["MiniCPMForCausalLM", "minicpm", "minicpm4"], MiniCPM4Config, describe)
