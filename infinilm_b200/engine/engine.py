"""The engine: a model on one GPU with its cache and its step function.

    eng = Engine.from_folder(model_dir, dtype="bfloat16", max_tokens=4096)
    seq = eng.open("a"); logits = eng.step([StepEntry(seq, [5, 17, 3], want=[2])]); eng.close(seq)

Parity with InfiniLM: `python/infinilm/infer_engine.py:152-214` (read config.json, build the C++
engine with a cache configuration), `csrc/engine/infer_engine.cpp:51-108` (config -> model ->
cache), `python/infinilm/llm/model_runner/model_runner.py:45-153` (cache config from num_blocks
and block_size, then load the weights).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence

import torch

from .. import ops
from ..cache.manager import CacheManager, SequenceCache
from ..config.model_config import ModelConfig, parse_dtype_name
from ..config.registry import config_from_json, describe_model, load_config
from ..models.causal_lm import CausalLM
from ..weights.loader import DictSource, FolderSource, TensorSource, load_into
from .step import StepEntry, StepRunner

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class Engine:
    def __init__(self, config: ModelConfig, source: TensorSource, dtype: str = "bfloat16", device: str = "cuda:0",
                 page_size: int = 16, num_pages: Optional[int] = None, max_tokens: Optional[int] = None,
                 max_seqs: int = 64, max_batch_tokens: int = 8192, progress=None):
        """`num_pages` pages of `page_size` tokens per cache group, or enough for `max_tokens`
        cached tokens (each request's count rounded up to whole pages)."""
        if not torch.cuda.is_available():
            raise RuntimeError("infinilm_b200 runs on a CUDA device (sm_100a); none is visible and there is no CPU path")
        name = parse_dtype_name(dtype)
        if name not in _TORCH_DTYPES:
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype!r}")
        self.config, self.dtype_name, self.dtype = config, name, _TORCH_DTYPES[name]
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        # Library matrix products never use a reduced-precision mode on the float32 path.
        torch.backends.cuda.matmul.allow_tf32 = False
        self.model = CausalLM(describe_model(config), self.dtype)
        load_into(self.model, source, self.device, progress)
        if num_pages is None:
            if max_tokens is None:
                max_tokens = min(config.max_position_embeddings, 8192)
            num_pages = (int(max_tokens) + page_size - 1) // page_size + max_seqs
        self.page_size, self.num_pages = page_size, int(num_pages)
        self.cache = CacheManager(self.model.cache_needs(), page_size, self.num_pages, max_seqs,
                                  device=self.device, dtype=self.dtype)
        self.runner = StepRunner(self.model, self.cache, self.device, max_batch_tokens)
        self.runner.max_positions = config.max_position_embeddings
        self.vocab_size = self.model.vocab

    # -- construction ----------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, **kw) -> "Engine":
        """A folder with config.json and safetensors; the model class follows from config.json."""
        cfg = load_config(model_dir)
        src = FolderSource(model_dir)
        try:
            return cls(cfg, src, **kw)
        finally:
            src.close()

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: Mapping[str, torch.Tensor], **kw) -> "Engine":
        return cls(config, DictSource(tensors), **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int = 0, **kw) -> "Engine":
        """Random weights drawn on the device (no folder is written)."""
        from ..weights.random_init import random_tensors
        device = kw.get("device", "cuda:0")
        return cls(config, DictSource(random_tensors(config, seed, device)), **kw)

    # -- requests and steps ----------------------------------------------------------------
    def open(self, seq_id) -> SequenceCache:
        return self.cache.open(seq_id)

    def close(self, seq: SequenceCache) -> None:
        self.cache.close(seq)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.runner.step(entries, device_tokens)

    def enable_graphs(self) -> None:
        """Replay decode-only steps as CUDA graphs from now on."""
        self.runner.use_graphs = True

    def synchronize(self) -> None:
        """Waits for the device and raises if a kernel reported that one of its bounded waits ran out."""
        torch.cuda.current_stream(self.device).synchronize()
        ops.check_status(self.device)
