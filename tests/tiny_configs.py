"""Two tiny MiniCPM4 configurations that differ in every size and option, plus helpers that
make random weights for them. Used by the CPU and the GPU tests."""
from __future__ import annotations

import random
from typing import Dict, List

import torch


def tiny_a() -> dict:
    # plain RoPE, tied head, 2 kv heads, head_dim 16
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 160, "vocab_size": 256,
        "rope_theta": 10000.0, "max_position_embeddings": 128,
        "scale_emb": 12, "dim_model_base": 32, "scale_depth": 1.4,
        "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "torch_dtype": "float32",
        "eos_token_id": 2,
    }


def tiny_b() -> dict:
    # LongRoPE crossing its original maximum, untied head, 3 kv heads, head_dim 32, hidden 192
    rng = random.Random(7)
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 3,
        "head_dim": 32, "intermediate_size": 320, "vocab_size": 512,
        "rope_theta": 1e6, "max_position_embeddings": 256,
        "rope_scaling": {"rope_type": "longrope",
                         "short_factor": [round(rng.uniform(1, 4), 4) for _ in range(16)],
                         "long_factor": [round(rng.uniform(1, 4), 4) for _ in range(16)],
                         "original_max_position_embeddings": 64},
        "scale_emb": 8, "dim_model_base": 64, "scale_depth": 1.0,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "torch_dtype": "float32",
        "eos_token_id": [1, 3],
    }


def tiny_c() -> dict:
    # odd sizes: hidden and vocabulary no power of two, head_dim 48 with heads*head_dim != hidden,
    # group of 5, partial rotary, biases, bfloat16 storage
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm4",
        "num_hidden_layers": 2, "hidden_size": 200, "num_attention_heads": 5, "num_key_value_heads": 1,
        "head_dim": 48, "intermediate_size": 264, "vocab_size": 331,
        "rope_theta": 50000.0, "max_position_embeddings": 512, "partial_rotary_factor": 0.5,
        "scale_emb": 3.5, "dim_model_base": 100, "scale_depth": 2.0,
        "rms_norm_eps": 1e-4, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
        "attention_bias": True, "mlp_bias": True, "attention_output_bias": True,
    }


def tiny_d() -> dict:
    # head_dim 64 (the size with TMA / tensor-memory attention kernels), groups of 4, heads*head_dim != hidden,
    # LongRoPE that stays below its original maximum (short factors), long enough for several key tiles
    rng = random.Random(11)
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm4",
        "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 8, "num_key_value_heads": 2,
        "head_dim": 64, "intermediate_size": 224, "vocab_size": 300,
        "rope_theta": 20000.0, "max_position_embeddings": 512,
        "rope_scaling": {"rope_type": "longrope",
                         "short_factor": [round(rng.uniform(1, 2), 4) for _ in range(32)],
                         "long_factor": [round(rng.uniform(2, 6), 4) for _ in range(32)],
                         "original_max_position_embeddings": 512},
        "scale_emb": 6, "dim_model_base": 80, "scale_depth": 1.2,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
        "eos_token_id": 0,
    }


TINY = {"a": tiny_a, "b": tiny_b, "c": tiny_c, "d": tiny_d}


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def make_weights(raw_cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random tensors by checkpoint name through the framework's random-weights mode (values
    are bfloat16-representable so both compute paths see identical weights)."""
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors
    return random_tensors(config_from_json(raw_cfg), seed, "cpu")
