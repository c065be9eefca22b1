"""A causal language model built from a `ModelSpec`: embedding, blocks in their run order,
final norm, head. It holds no size of its own and knows no architecture.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:89-101` (embed, run the
layers carrying (hidden, residual), final norm) and `:123-127` (head), with one difference that
is ours: the head runs only on the rows whose logits are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import Part, build_part, part_class
from ..parts.spec import CacheNeed, ModelSpec, WeightSpec


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        self.spec, self.dtype = spec, dtype
        self.embedding = build_part("embedding", spec.embedding, dtype)
        self.blocks = []
        for ls in spec.layers:
            arr = part_class("arrangement", ls.arrangement)
            self.blocks.append(arr(build_part("norm", ls.mixer_norm, dtype), build_part("mixer", ls.mixer, dtype),
                                   build_part("norm", ls.ffn_norm, dtype), build_part("feed_forward", ls.ffn, dtype),
                                   ls.params))
        self.final_norm = build_part("norm", spec.final_norm, dtype)
        self.head = build_part("head", spec.head, dtype)
        self.order = list(spec.order)
        for i, st in enumerate(self.order):
            if not 0 <= st.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {st.layer}, which does not exist")
            if st.cache_from is not None and not (0 <= st.cache_from < i and self.order[st.cache_from].cache_from is None):
                raise ValueError(f"run order entry {i}: cache_from must name an earlier entry that owns its cache")
        self.hidden = self.embedding.hidden
        self.vocab = self.head.vocab
        # decode steps are replayed as CUDA graphs only if every part says it can be (`Part.graph_safe`)
        self.graph_safe = all(p.graph_safe for p in self.parts())

    # -- weights ---------------------------------------------------------------------------
    def parts(self) -> List[Part]:
        out: List[Part] = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out += [self.final_norm, self.head]
        return out

    def weight_specs(self) -> List[Tuple[Part, WeightSpec]]:
        return [(p, ws) for p in self.parts() for ws in p.weight_specs()]

    # -- cache -----------------------------------------------------------------------------
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per run-order entry: what it keeps (None: nothing, or it reads another's)."""
        needs = []
        for st in self.order:
            needs.append(None if st.cache_from is not None else self.blocks[st.layer].mixer.cache_need())
        return needs

    # -- forward ---------------------------------------------------------------------------
    def forward(self, ctx, caches) -> torch.Tensor:
        """Runs the tokens of `ctx` and returns float32 logits [len(ctx.want_rows), vocab].
        `caches[i]` is the cache view of run-order entry i."""
        T = ctx.T
        resid = ctx.ws.rows("resid", T, self.hidden, torch.float32)
        self.embedding.forward(ctx.token_ids, resid)
        pending = None
        for i, st in enumerate(self.order):
            # the block that runs next may take its first norm half done (its weights applied, the rms still to divide by)
            blk = self.blocks[st.layer]
            nxt = self.blocks[self.order[i + 1].layer] if i + 1 < len(self.order) else None
            if blk.takes_next_norm and nxt is not None and nxt.accepts_normed_input(T):
                pending = blk.run(resid, pending, ctx, caches[i], next_norm=nxt.mixer_norm)
            else:
                pending = blk.run(resid, pending, ctx, caches[i])
            if ctx.tap is not None:
                ctx.tap(f"layer{i}", resid, pending)
        n = ctx.n_want
        logits = ctx.ws.rows("logits", n, self.vocab, torch.float32)
        if n == 0:
            return logits
        branch, bscale = pending if pending is not None else (None, 1.0)
        normed = self.final_norm.add_norm(resid, branch, bscale, ctx.ws.rows("final_normed", n, self.hidden, self.dtype),
                                          rows=ctx.want_rows)
        return self.head.forward(normed, logits)
