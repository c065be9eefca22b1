"""Random-weights mode: tensors for a configuration from a seed, and a model folder written
from them (config.json, model.safetensors).

InfiniLM's counterpart is `--skip-load`, which leaves parameters as allocated
(`python/infinilm/llm/model_runner/model_runner.py:104-107`); here every tensor is drawn from a
generator keyed by (seed, tensor name), so a tensor's values do not depend on the order or the
device of generation of the others. Values are rounded to bfloat16 before they are stored, so
the float32 and the bfloat16 path of one folder compute with identical weights.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.registry import describe_model
from ..models.causal_lm import CausalLM
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(cfg: ModelConfig, seed: int, device: str = "cpu", dtype: Optional[torch.dtype] = None,
                   tie: Optional[bool] = None) -> Dict[str, torch.Tensor]:
    """name -> tensor for every tensor the model wants. `dtype` None: the config's torch_dtype.
    A tied head (`tie_word_embeddings`) gets no tensor of its own."""
    store = dtype or {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.bfloat16}[cfg.torch_dtype]
    if tie is None:
        tie = bool(getattr(cfg, "tie_word_embeddings", False))
    model = CausalLM(describe_model(cfg), torch.float32)
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for part, ws in model.weight_specs():
        full = part.full_name(ws.name)
        if ws.fallback is not None and tie:
            continue
        g = torch.Generator(device=dev)
        g.manual_seed(_seed_for(seed, full))
        kind = ws.init[0]
        if kind == "zeros":
            t = torch.zeros(ws.shape, dtype=torch.float32, device=dev)
        else:
            t = torch.randn(ws.shape, generator=g, dtype=torch.float32, device=dev) * float(ws.init[1])
            if kind == "ones_normal":
                t += 1.0
            elif kind != "normal":
                raise ValueError(f"unknown init {ws.init}")
        if ws.role == "table":
            out[full] = t.to(torch.int32)
        else:
            out[full] = t.to(torch.bfloat16).to(store)
    return out


def write_model_folder(cfg: ModelConfig, seed: int, out_dir: str) -> str:
    """Writes config.json and model.safetensors for `cfg` with weights drawn from `seed`."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg.to_json(), f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(cfg, seed, "cpu"))
    return out_dir
