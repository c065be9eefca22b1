"""Helpers of the GPU tests: build an engine for a tiny configuration and replay requests
through its step function under different ways of cutting the work."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

import plain_model
from tiny_configs import make_weights

# Largest |engine - plain| allowed, as a fraction of the largest |plain logit| of the row.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def build_engine(raw_cfg: dict, weights: Dict[str, torch.Tensor], dtype: str, num_pages: int = 64,
                 page_size: int = 16, max_seqs: int = 8, max_batch_tokens: int = 512):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine
    return Engine.from_tensors(config_from_json(raw_cfg), weights, dtype=dtype, page_size=page_size,
                               num_pages=num_pages, max_seqs=max_seqs, max_batch_tokens=max_batch_tokens)


def plain_logits(raw_cfg: dict, weights, ids: List[int], dtype: str) -> torch.Tensor:
    return plain_model.forward(raw_cfg, weights, ids, round_embedding_bf16=(dtype == "bfloat16"))


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if not torch.isfinite(got).all():
        return float("inf")
    denom = ref.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6)
    return float(((got - ref).abs() / denom).max())


def first_bad_row(got: torch.Tensor, ref: torch.Tensor, tol: float) -> Optional[int]:
    got, ref = got.float().cpu(), ref.float().cpu()
    denom = ref.abs().amax(dim=-1, keepdim=True).clamp_min(1e-6)
    bad = (((got - ref).abs() / denom).amax(dim=-1) > tol) | ~torch.isfinite(got).all(dim=-1)
    idx = torch.nonzero(bad)
    return None if idx.numel() == 0 else int(idx[0])


def run_cut(eng, ids: List[int], cuts: Sequence[int], seq_id="r") -> torch.Tensor:
    """Feeds `ids` in portions of the given sizes (their sum is len(ids)); logits at every position."""
    from infinilm_b200.engine import StepEntry
    assert sum(cuts) == len(ids)
    seq = eng.open(seq_id)
    outs, a = [], 0
    for c in cuts:
        outs.append(eng.step([StepEntry(seq, ids[a:a + c], list(range(c)))]).clone())
        a += c
    eng.close(seq)
    return torch.cat(outs, 0)


def run_schedule(eng, requests: Dict[str, List[int]], schedule: List[List[Tuple[str, int]]],
                 check_invariants: bool = True) -> Dict[str, torch.Tensor]:
    """`schedule` is a list of steps; a step is a list of (request id, number of next tokens).
    A request is opened at its first portion and closed right after its last. Logits at every
    position of every request are returned."""
    from infinilm_b200.engine import StepEntry
    done = {k: 0 for k in requests}
    seqs, outs = {}, {k: [] for k in requests}
    for step in schedule:
        entries, who = [], []
        for rid, n in step:
            if rid not in seqs:
                seqs[rid] = eng.open(rid)
            a = done[rid]
            entries.append(StepEntry(seqs[rid], requests[rid][a:a + n], list(range(n))))
            who.append((rid, n))
            done[rid] = a + n
        logits = eng.step(entries).clone()
        r = 0
        for rid, n in who:
            outs[rid].append(logits[r:r + n])
            r += n
        for rid, _ in who:
            if done[rid] == len(requests[rid]) and rid in seqs:
                eng.close(seqs.pop(rid))
        if check_invariants:
            eng.cache.check_invariants()
    assert all(done[k] == len(requests[k]) for k in requests), "schedule does not cover the requests"
    return {k: torch.cat(v, 0) for k, v in outs.items()}


def check_greedy(raw_cfg: dict, weights, prompt: List[int], tokens: List[int], dtype: str) -> None:
    """`tokens` is a greedy continuation of `prompt` by the plain implementation: exactly in float32; in bfloat16
    wherever the plain top-2 margin is wide enough to survive rounding (a token inside the margin is followed)."""
    if dtype == "float32":
        assert tokens == plain_model.greedy_generate(raw_cfg, weights, prompt, len(tokens))
        return
    ids = list(prompt)
    for t in tokens:
        lg = plain_logits(raw_cfg, weights, ids, dtype)[-1]
        top2 = torch.topk(lg, 2).values
        if float(top2[0] - top2[1]) > 4 * TOL[dtype] * float(lg.abs().max()):
            assert t == int(torch.argmax(lg)), f"token {len(ids) - len(prompt)}: {t} != {int(torch.argmax(lg))}"
        ids.append(t)
