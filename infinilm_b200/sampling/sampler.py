"""Greedy and temperature / top-k / top-p sampling over batches of float32 logits.

Parity with InfiniLM: `python/infinilm/llm/sampling_params.py:9-39` (`SamplingParams`: temperature
1.0, top_p 0.8, top_k 1, max_tokens 512, stop, stop_token_ids, ignore_eos; top_k = 1 means
greedy), `csrc/engine/rank_worker.cpp:467-513` (one `random_sample_(logits_row, random_val, top_p,
top_k, temperature)` per request, random_val uniform in [0,1) from an unseeded mt19937). Here one
kernel launch samples all rows, each row has its own parameters, and the uniform numbers come from
a counter-based generator keyed by (seed, request, token index), so a request's tokens do not
depend on what else is in the batch and a run can be repeated.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops


@dataclass
class SamplingParams:
    """Sampling parameters of one request (names and defaults as in InfiniLM)."""
    temperature: float = 1.0
    top_p: float = 0.8
    top_k: int = 1
    max_tokens: int = 512
    stop: Optional[List[str]] = None
    stop_token_ids: Optional[List[int]] = None
    ignore_eos: bool = False
    seed: Optional[int] = None                    # ours: None draws the seed from the engine's

    def __post_init__(self):
        if self.stop is None:
            self.stop = []
        if self.stop_token_ids is None:
            self.stop_token_ids = []
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")

    @property
    def greedy(self) -> bool:
        return self.top_k == 1 or self.temperature == 0.0

    def clone(self) -> "SamplingParams":
        return SamplingParams(self.temperature, self.top_p, self.top_k, self.max_tokens, list(self.stop),
                              list(self.stop_token_ids), self.ignore_eos, self.seed)


_MASK = (1 << 64) - 1


def uniform01(seed: int, stream: int, counter: int) -> float:
    """A number in [0,1) that depends only on (seed, stream, counter) (splitmix64 finaliser)."""
    x = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + counter * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _MASK
    for _ in range(2):
        x ^= x >> 30
        x = (x * 0xBF58476D1CE4E5B9) & _MASK
        x ^= x >> 27
        x = (x * 0x94D049BB133111EB) & _MASK
        x ^= x >> 31
    return (x >> 40) / float(1 << 24)


class Sampler:
    """Samples one token per row of logits on the device."""

    RING = 4

    def __init__(self, device, max_rows: int = 1024):
        self.device = torch.device(device)
        self.max_rows = max_rows
        # The parameters of a step go to the device by an asynchronous copy from pinned memory. The host may fill the
        # buffer of step k+1 before the GPU has run the copy of step k (pipelined stepping), so each step takes the
        # next pair of a small ring (host and device), and a pair is reused only after the event recorded behind its
        # last sampling kernel has passed.
        self._host = [torch.empty((4, max_rows), dtype=torch.float32, pin_memory=True) for _ in range(self.RING)]
        self._dev = [torch.empty((4, max_rows), dtype=torch.float32, device=self.device) for _ in range(self.RING)]
        self._events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self._turn = -1
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float],
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits float32 [R,V] on the device -> int32 [R] on the device (into `out` if given)."""
        R, V = logits.shape
        if out is None:
            out = self._out
        if R == 0:
            return out[:0]
        if R > self.max_rows or len(params) != R or len(uniforms) != R:
            raise ValueError("sampler: rows, params and uniforms must agree (and fit max_rows)")
        if all(p.greedy for p in params):
            return self.argmax(logits, out)
        self._turn = i = (self._turn + 1) % self.RING
        if self._events[i] is not None:
            self._events[i].synchronize()
        host, dev = self._host[i], self._dev[i]
        hn = host.numpy()
        hn[0, :R] = [0.0 if p.greedy else p.temperature for p in params]
        host.view(torch.int32).numpy()[1, :R] = [1 if p.greedy else int(p.top_k) for p in params]
        hn[2, :R] = [p.top_p for p in params]
        hn[3, :R] = list(uniforms)
        dev.copy_(host, non_blocking=True)        # whole buffers: contiguous, so a true asynchronous copy
        ops.sample(logits, dev[0, :R], dev[1, :R].view(torch.int32), dev[2, :R], dev[3, :R], out[:R])
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return out[:R]

    def argmax(self, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        R = logits.shape[0]
        if out is None:
            out = self._out
        if R > self.max_rows or R > out.numel():
            raise ValueError("sampler: too many rows")
        ops.sample(logits, None, None, None, None, out[:R], greedy=True)
        return out[:R]
