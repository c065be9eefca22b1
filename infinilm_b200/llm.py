"""The Python entry point: `LLM(model_path, ...).generate(...)`, in InfiniLM's manner.

Parity with InfiniLM: `python/infinilm/llm/llm.py:335-423` (`LLM.__init__` and its option names:
model_path, device, dtype, cache_type, max_batch_size, max_tokens, num_blocks, block_size,
temperature, top_p, top_k, enable_graph, attn_backend, skip_load, enable_prefix_caching),
`:428-535` (`generate(prompts | messages, sampling_params, use_tqdm)` returns `RequestOutput`s),
`:537-559` (`chat`), `:143-176` (`step` = schedule, run, update), `python/infinilm/llm/request.py:85-120`
(`RequestOutput`, `CompletionOutput`). Options that select other devices, parallelism, MoE,
drafts or a static cache are accepted where a script would pass them and must keep their
single-GPU, paged defaults. A prompt may also be given as token ids, since a folder of random
weights has no tokenizer.
"""
from __future__ import annotations

import os
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Union

import torch

from .config.model_config import ModelConfig
from .config.registry import load_config
from .engine.engine import Engine
from .engine.scheduler import FinishReason, Request, Scheduler, SchedulerOutput
from .engine.step import StepEntry
from .sampling.sampler import Sampler, SamplingParams, uniform01


@dataclass
class CompletionOutput:
    index: int = 0
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[FinishReason] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str] = None
    prompt_token_ids: Optional[List[int]] = None
    outputs: List[CompletionOutput] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[FinishReason] = None


class LLM:
    def __init__(self, model_path: Optional[str] = None, device: str = "cuda", dtype: Optional[str] = None,
                 tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1, cache_type: str = "paged",
                 max_batch_size: int = 16, max_tokens: int = 4096, num_blocks: int = 512, block_size: int = 256,
                 temperature: float = 1.0, top_p: float = 0.8, top_k: int = 1, enable_graph: bool = False,
                 attn_backend: str = "default", skip_load: bool = False, enable_prefix_caching: bool = False,
                 max_num_batched_tokens: Optional[int] = None, chunk_size: int = 2048, seed: int = 0,
                 admission: str = "worst_case", pipelined: bool = True, _config: Optional[ModelConfig] = None,
                 _tensors: Optional[Mapping[str, torch.Tensor]] = None):
        """`model_path`: folder with config.json and safetensors. `skip_load`: random weights
        (seeded) instead of the folder's. `num_blocks` pages of `block_size` tokens. `pipelined`: a
        step's tokens are read back while the next step runs (the next step gets them on the device)."""
        if tensor_parallel_size != 1 or pipeline_parallel_size != 1:
            raise ValueError("this engine runs on one GPU: tensor_parallel_size and pipeline_parallel_size must be 1")
        if cache_type != "paged":
            raise ValueError("only the paged cache exists here (cache_type='paged')")
        if attn_backend not in ("default", "paged-attn", "flash-attn"):
            raise ValueError(f"unknown attn_backend {attn_backend!r}")
        if enable_prefix_caching:
            raise ValueError("prefix caching is not built; pass enable_prefix_caching=False")
        if device not in ("cuda", "nvidia", "auto") and not str(device).startswith("cuda"):
            raise ValueError(f"device {device!r}: this engine runs on a CUDA device only")
        dev = device if str(device).startswith("cuda:") else "cuda:0"
        cfg = _config if _config is not None else load_config(model_path)
        self.model_config = cfg
        dtype = dtype or cfg.torch_dtype
        if dtype == "float16":
            dtype = "bfloat16"                    # 16-bit weights are kept as bfloat16
        mnbt = max_num_batched_tokens or int(os.environ.get("INFINILM_MAX_NUM_BATCHED_TOKENS", "0")) or 8192
        kw = dict(dtype=dtype, device=dev, page_size=block_size, num_pages=num_blocks, max_seqs=max_batch_size,
                  max_batch_tokens=mnbt)
        if _tensors is not None:
            self.engine = Engine.from_tensors(cfg, _tensors, **kw)
        elif skip_load:
            self.engine = Engine.from_random(cfg, seed, **kw)
        else:
            self.engine = Engine.from_folder(model_path, **kw)
        self.scheduler = Scheduler(self.engine.cache, max_batch_size=max_batch_size, max_num_batched_tokens=mnbt,
                                   chunk_size=chunk_size, admission=admission,
                                   max_model_len=cfg.max_position_embeddings)
        self.sampler = Sampler(self.engine.device, max_rows=max(max_batch_size, 8))
        self.default_params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, max_tokens=max_tokens)
        self.seed = seed
        self.enable_graph = enable_graph
        self.eos_token_ids = list(cfg.eos_token_ids)
        self.model_path = model_path
        self._tokenizer = None
        self._n_requests = 0
        nrow = max(max_batch_size, 8)
        self._ids_host = [torch.empty(nrow, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._ids_dev = [torch.zeros(nrow, dtype=torch.int32, device=self.engine.device) for _ in range(2)]
        self._parity = 0
        self._inflight = None                     # the step whose tokens the host has not read yet
        self.pipelined = pipelined
        if enable_graph:
            self.engine.enable_graphs()

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: Mapping[str, torch.Tensor], **kw) -> "LLM":
        return cls(None, _config=config, _tensors=tensors, **kw)

    # -- text ------------------------------------------------------------------------------
    @property
    def tokenizer(self):
        """The tokenizer of the model folder, if it has one (loaded on first use)."""
        if self._tokenizer is None:
            if self.model_path is None:
                raise RuntimeError("this LLM was built without a model folder, so it has no tokenizer; "
                                   "pass prompt_token_ids")
            from transformers import AutoTokenizer
            self._tokenizer = AutoTokenizer.from_pretrained(self.model_path, trust_remote_code=True)
        return self._tokenizer

    def tokenize(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text))

    def detokenize(self, ids: Sequence[int]) -> str:
        if self.model_path is None:
            return ""
        try:
            return self.tokenizer.decode(list(ids), skip_special_tokens=True)
        except Exception:
            return ""

    # -- requests ----------------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
                    prompt: Optional[str] = None, request_id: Optional[str] = None) -> Request:
        p = (sampling_params or self.default_params).clone()
        r = Request(request_id or f"cmpl-{uuid.uuid4().hex}", list(prompt_token_ids), p, tuple(self.eos_token_ids),
                    prompt=prompt, sample_stream=self._n_requests)
        self._n_requests += 1
        self.scheduler.add_request(r)
        return r

    def step(self) -> List[Request]:
        """One step: schedule, run, sample; then read back the tokens of the step BEFORE this one and
        apply the finish rules to them. The step just issued stays in flight: its tokens are fed to
        the next step on the device, so the host never waits for the GPU between two steps. Returns
        the requests that finished. When nothing is left to schedule, the step in flight is retired."""
        out = self.scheduler.schedule()
        if not out.entries:
            if self._inflight is not None:
                return self._retire()
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler has requests but could schedule none (pool too small?)")
            return []
        entries = []
        for e in out.entries:
            toks = e.tokens
            if toks[-1] < 0:                      # sampled by the step in flight: row of that step's sampler output
                toks = toks[:-1] + [-(1 + e.request.last_sample_row)]
            entries.append(StepEntry(e.request.seq, toks, [len(toks) - 1] if e.samples else []))
        prev_ids = self._ids_dev[self._parity ^ 1] if self._inflight is not None else None
        logits = self.engine.step(entries, prev_ids)
        rows = [e for e in out.entries if e.samples]
        ids_dev = self._ids_dev[self._parity]
        host = self._ids_host[self._parity]
        ev = None
        if rows:
            params = [e.request.params for e in rows]
            us = [0.0 if e.request.params.greedy else                       # a greedy row draws nothing
                  uniform01(e.request.params.seed if e.request.params.seed is not None else self.seed,
                            e.request.sample_stream, len(e.request.output_token_ids)) for e in rows]
            self.sampler.sample(logits, params, us, out=ids_dev)
            host[:len(rows)].copy_(ids_dev[:len(rows)], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self.scheduler.launched(out)
        finished = self._retire() if self._inflight is not None else []
        self._inflight = (out, len(rows), host, ev)
        self._parity ^= 1
        if not self.pipelined:
            finished += self._retire()
        return finished

    def _retire(self) -> List[Request]:
        """Waits for the tokens of the step in flight and hands them to the scheduler."""
        out, n, host, ev = self._inflight
        self._inflight = None
        if ev is not None:
            ev.synchronize()
        return self.scheduler.retire(out, host[:n].tolist())

    # -- batch generation --------------------------------------------------------------------
    def generate(self, prompts: Union[str, List[str], None] = None, messages=None,
                 sampling_params: Optional[SamplingParams] = None, use_tqdm: bool = False,
                 prompt_token_ids: Optional[List[List[int]]] = None) -> List[RequestOutput]:
        """InfiniLM's `LLM.generate` (`python/infinilm/llm/llm.py:428-501`): prompts or conversations in, one
        `RequestOutput` each out, in order. Beside it: `prompt_token_ids` (token ids instead of text), and
        `sampling_params` may be a list, one for each prompt."""
        if isinstance(prompts, str):
            prompts = [prompts]

        def sp_of(i: int):
            return sampling_params[i] if isinstance(sampling_params, (list, tuple)) else sampling_params
        reqs: List[Request] = []
        if prompt_token_ids is not None:
            for i, ids in enumerate(prompt_token_ids):
                reqs.append(self.add_request(ids, sp_of(i)))
        elif messages is not None:
            if messages and isinstance(messages[0], dict):
                messages = [messages]
            for i, conv in enumerate(messages):
                text = self.tokenizer.apply_chat_template(conv, add_generation_prompt=True, tokenize=False)
                reqs.append(self.add_request(self.tokenize(text), sp_of(i), prompt=text))
        elif prompts is not None:
            for i, text in enumerate(prompts):
                reqs.append(self.add_request(self.tokenize(text), sp_of(i), prompt=text))
        else:
            raise ValueError("generate needs prompts, messages or prompt_token_ids")
        pbar = None
        if use_tqdm:
            try:
                from tqdm import tqdm
                pbar = tqdm(total=len(reqs), desc="Generating")
            except ImportError:
                pbar = None
        done = 0
        while done < len(reqs):
            self.step()
            now = sum(1 for r in reqs if r.finished)
            if pbar is not None and now > done:
                pbar.update(now - done)
            done = now
        if pbar is not None:
            pbar.close()
        return [self._output_of(r) for r in reqs]

    def chat(self, messages, sampling_params: Optional[SamplingParams] = None, use_tqdm: bool = False):
        return self.generate(messages=messages, sampling_params=sampling_params, use_tqdm=use_tqdm)

    def _output_of(self, r: Request) -> RequestOutput:
        text = self.detokenize(r.output_token_ids) if self.model_path is not None and self._tokenizer is not None else ""
        return RequestOutput(r.request_id, r.prompt, list(r.prompt_token_ids),
                             [CompletionOutput(0, text, list(r.output_token_ids), r.finish_reason)],
                             r.finished, r.finish_reason)

    def stats(self) -> Dict[str, int]:
        s = self.scheduler.stats()
        s.update(steps=self.engine.runner.steps_run, tokens=self.engine.runner.tokens_run)
        return s

    def close(self) -> None:
        if self._inflight is not None:
            self._retire()
        self.engine.synchronize()
