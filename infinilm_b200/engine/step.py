"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere. It runs only
the tokens it is given, as one batch, reading earlier tokens from the cache, and returns the
float32 logits at the places asked for. The logits at a position do not depend on how the
tokens were cut into steps or on what else is in the batch, beyond rounding.

Parity with InfiniLM: `csrc/engine/infer_engine.hpp:53` / `csrc/models/infinilm_model.hpp:20-67`
(`forward(Input) -> Output`; Input carries input_ids, position_ids, past/total lengths,
input_offsets, block_tables, slot_mapping), `python/infinilm/processors/basic_llm_processor.py:161-263`
(how a batch is flattened). Here positions, lengths and slots are derived from three small
arrays per step (token ids, per-token position and entry, per-entry block-table rows) that go to
the device in one copy, and the head runs only on the wanted rows.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, OutOfPages, PagedKVView, SequenceCache, StateView
from ..models.causal_lm import CausalLM


class StepError(ValueError):
    """A batch that cannot be run: says which entry and why."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and the places among them (indices into
    `tokens`) whose logits are wanted."""
    seq: SequenceCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Workspace:
    """Device buffers that live as long as the engine; a buffer is named by its use and sized
    for the largest step, so no step allocates."""

    def __init__(self, device, max_tokens: int):
        self.device, self.max_tokens = device, int(max_tokens)
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}      # the first n rows of a buffer, made once per n (a step asks
        self.version = 0                          # bumped when a buffer is replaced (captured graphs go stale)

    def rows(self, tag: str, n: int, width: int, dtype: torch.dtype) -> torch.Tensor:
        vkey = (tag, n, width, dtype)             # for the same few dozen views layer after layer)
        view = self._views.get(vkey)
        if view is not None:
            return view
        key = (tag, width, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < n:
            if buf is None:
                # per-token buffers are made for the largest step; the logits (rows x vocabulary) for 256 rows
                cap = max(n, min(self.max_tokens, 256) if tag == "logits" else self.max_tokens)
            else:
                cap = max(n, buf.shape[0] * 2)
                self.version += 1
            buf = torch.empty((cap, width), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self._views = {k: v for k, v in self._views.items() if k[0] != tag}
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[vkey] = buf[:n]
        return view

    def flat(self, tag: str, n: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """`zero`: the buffer is zero when it is made (its users leave it zero)."""
        key = (tag, "flat", dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if buf is not None:
                self.version += 1
            buf = (torch.zeros if zero else torch.empty)(max(n, 1024), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n]


@dataclass
class StepContext:
    """What the parts see of a step. Device arrays are int32."""
    dtype: torch.dtype
    T: int
    n_entries: int
    n_decode: int                                 # the first n_decode entries bring one token each
    token_ids: torch.Tensor                       # [T]
    tok_pos: torch.Tensor                         # [T] absolute position of each token in its request
    tok_entry: torch.Tensor                       # [T] entry index of each token
    entry_qstart: torch.Tensor                    # [E+1] first token row of each entry
    entry_kvlen: torch.Tensor                     # [E] tokens in cache after this step (start + q_len)
    want_rows: torch.Tensor                       # [n_want] token rows whose logits are wanted
    n_want: int
    ws: Workspace
    h_qlen: List[int] = field(default_factory=list)     # host copies for launch planning
    h_kvlen: List[int] = field(default_factory=list)
    max_qlen: int = 0
    max_kvlen: int = 0
    tap: Optional[Callable] = None                # debug hook: tap(name, resid, pending)
    lengths_are_bounds: bool = False              # h_qlen / h_kvlen are upper bounds (a step replayed as a graph)

    def prompt_tiles(self, tokens_per_tile: int) -> int:
        """How many tiles of `tokens_per_tile` tokens the prompt portions (the entries behind the first n_decode) are cut
        into, each portion by itself: the exact number, or - when lengths are bounds - the most that any split of the
        portions' tokens can give, so that a kernel launched per tile gets the same grid whenever the step is replayed."""
        if not self.lengths_are_bounds:
            return sum((q + tokens_per_tile - 1) // tokens_per_tile for q in self.h_qlen[self.n_decode:])
        n_portions = self.n_entries - self.n_decode
        if n_portions <= 0:
            return 0
        return (self.T - self.n_decode + tokens_per_tile - 1) // tokens_per_tile + n_portions - 1


class StepRunner:
    """Owns the model, the cache manager and the device buffers, and runs steps."""
    GRAPH_AFTER = 2                               # a step with prompt portions is captured when its key comes a third time
    MAX_GRAPHS = 128                              # captured steps kept

    def __init__(self, model: CausalLM, cache: CacheManager, device, max_batch_tokens: int):
        self.model, self.cache, self.device = model, cache, torch.device(device)
        self.max_batch_tokens = int(max_batch_tokens)
        self.ws = Workspace(self.device, self.max_batch_tokens)
        self.dtype = model.dtype
        self._desc_dev: Optional[torch.Tensor] = None
        self.tap: Optional[Callable] = None
        self.use_graphs = False
        self._graphs: Dict[tuple, "_GraphSlot"] = {}
        self._graph_pool = None
        self.graph_prompts = True                 # steps with prompt portions are replayed too, once their key has come back
        self._shapes_seen: Dict[tuple, int] = {}
        self.h2d_bytes = 0
        self.steps_run = 0
        self.tokens_run = 0
        self.portion_replays = 0                  # steps with prompt portions that were replayed as graphs
        self._last_decode: Optional["_DecodeBatch"] = None    # the replayed decode step just run, if the next may follow it
        self.fast_steps = 0

    # -- descriptor buffers ----------------------------------------------------------------
    def _desc(self, n_ints: int):
        """A pinned host buffer (one of a small ring, so the copy of an earlier step is never
        overwritten while in flight) and the device buffer the kernels read."""
        if self._desc_dev is None or self._desc_dev.numel() < n_ints:
            cap = max(2 * n_ints, 1 << 16)          # grown with headroom: pinned allocations are slow
            if self._desc_dev is not None:
                torch.cuda.current_stream(self.device).synchronize()
            self._desc_ring = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._desc_events = [None] * 4
            self._desc_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self._desc_i = (getattr(self, "_desc_i", -1) + 1) % 4
        ev = self._desc_events[self._desc_i]
        if ev is not None:
            ev.synchronize()
        return self._desc_ring[self._desc_i], self._desc_dev

    # -- a decode step that follows the same decode step ----------------------------------------
    def _follow_decode(self, last: "_DecodeBatch", entries: Sequence[StepEntry], device_tokens) -> Optional[torch.Tensor]:
        """The step after a replayed decode-only step, if it is the same requests in the same order with one token each
        (what a serving run is mostly made of): nothing is built per request but its token; lengths and positions
        advance as columns, a block table row is rewritten only where a request begins a page, the same graph is
        replayed. Returns None when the step is anything else; the general path then runs (and reports what is wrong
        with a batch that is wrong). With hundreds of live requests the general path cost the host more per step than
        the GPU needed to run it."""
        E = last.E
        if len(entries) != E or self.tap is not None or not self.use_graphs:
            return None
        gs = last.gs
        if gs.graph is None or gs.ws_version != self.ws.version:
            return None
        seqs = last.seqs
        for e, s in zip(entries, seqs):
            if e.seq is not s or len(e.tokens) != 1 or len(e.want) != 1:
                return None
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=E)
        lens = last.lens
        neg = tokens < 0
        if int(tokens.max()) >= self.model.vocab or (neg.any() and (device_tokens is None or int(-1 - tokens.min()) >= device_tokens.numel())):
            return None
        max_pos = getattr(self, "max_positions", None)
        if max_pos is not None and int(lens.max()) + 1 > max_pos:
            return None
        cache, sub, ps = self.cache, self.cache.sub, self.cache.page_size
        starts = np.flatnonzero(lens % ps == 0)   # these requests' next token begins a page
        paged = list(last.widths)
        for i in starts:
            for g in paged:
                if (len(seqs[i].tables[g]) + 1) * sub > last.widths[g]:
                    return None                   # the table outgrows this graph's width: the general path picks the next
        if starts.size:
            if not cache.can_reserve([(seqs[i], int(lens[i]) + 1) for i in starts]):
                return None                       # (the general path raises OutOfPages)
            for i in starts:
                cache.reserve(seqs[i], int(lens[i]) + 1)
        m, sp = last.mirror, last.spans
        m[sp["tok"][0]: sp["tok"][0] + E] = np.maximum(tokens, 0)
        m[sp["pos"][0]: sp["pos"][0] + E] = lens
        m[sp["kv"][0]: sp["kv"][0] + E] = lens + 1
        m[sp["rs"][0]: sp["rs"][0] + E] = m[sp["wsl"][0]: sp["wsl"][0] + E]       # no request is at its first step any more
        for i in starts:
            for g in paged:
                tbl = seqs[i].tables[g]
                a = sp["bt"][g][0] + int(i) * last.widths[g]
                m[a: a + len(tbl) * sub] = tbl.array()
        rows = np.flatnonzero(neg)
        n_patch = int(rows.size)
        if n_patch:
            m[sp["prow"][0]: sp["prow"][0] + n_patch] = rows
            m[sp["psrc"][0]: sp["psrc"][0] + n_patch] = -1 - tokens[rows]
        n = last.n_ints
        host, _ = self._desc(n)
        host.numpy()[:n] = m
        dev = gs.desc
        dev[:n].copy_(host[:n], non_blocking=True)
        if n_patch:
            ops.patch_tokens(dev[sp["tok"][0]: sp["tok"][1]], dev[sp["prow"][0]: sp["prow"][0] + n_patch],
                             dev[sp["psrc"][0]: sp["psrc"][0] + n_patch], device_tokens)
        ev = torch.cuda.Event()
        ev.record()
        self._desc_events[self._desc_i] = ev
        self.h2d_bytes += 4 * n
        gs.graph.replay()
        ops.count_launches(gs.n_kernels)
        for s_ in seqs:                           # what CacheManager.commit does for a request without a window
            s_.length += 1
        last.lens = lens + 1
        self._last_decode = last
        self.steps_run += 1
        self.tokens_run += E
        self.fast_steps += 1
        return gs.logits[:E]

    # -- a step's entries as columns, checked --------------------------------------------------------
    def _columns(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor]) -> "_Columns":
        """The entries' numbers as arrays, one element an entry (or a token, or a wanted place), and every check that
        needs no page: made on whole columns; a fault is then looked up entry by entry, for the message."""
        vocab = self.model.vocab
        E = len(entries)
        seqs = [e.seq for e in entries]
        n_tok = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=E)
        start = np.fromiter((s_.length for s_ in seqs), dtype=np.int32, count=E)
        T = int(n_tok.sum())
        if int(n_tok.min()) < 1:
            i = int(np.argmin(n_tok))
            raise StepError(f"entry {i} ({seqs[i].seq_id!r}) brings no token")
        if len(set(map(id, seqs))) != E:
            seen = set()
            for s_ in seqs:
                if id(s_) in seen:
                    raise StepError(f"request {s_.seq_id!r} appears twice in one step")
                seen.add(id(s_))
        tokens = np.fromiter(itertools.chain.from_iterable(e.tokens for e in entries), dtype=np.int64, count=T)
        tok_off = np.zeros(E + 1, dtype=np.int32)
        np.cumsum(n_tok, out=tok_off[1:])
        lo, hi = int(tokens.min()), int(tokens.max())
        if hi >= vocab or (lo < 0 and device_tokens is None):
            t = int(np.argmax(tokens >= vocab)) if hi >= vocab else int(np.argmax(tokens < 0))
            i = int(np.searchsorted(tok_off, t, side="right")) - 1
            raise StepError(f"request {seqs[i].seq_id!r}: token id outside [0, {vocab})")
        if lo < 0 and -1 - lo >= device_tokens.numel():
            i = int(np.searchsorted(tok_off, int(np.argmin(tokens)), side="right")) - 1
            raise StepError(f"request {seqs[i].seq_id!r}: device token {-1 - lo} does not exist")
        max_pos = getattr(self, "max_positions", None)
        if max_pos is not None and int((start + n_tok).max()) > max_pos:
            i = int(np.argmax(start + n_tok))
            raise StepError(f"request {seqs[i].seq_id!r} would pass max_position_embeddings {max_pos}")
        if T > self.max_batch_tokens:
            raise StepError(f"step of {T} tokens exceeds max_batch_tokens {self.max_batch_tokens}")
        n_want_of = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=E)
        want_off = np.zeros(E + 1, dtype=np.int32)
        np.cumsum(n_want_of, out=want_off[1:])
        want = np.fromiter(itertools.chain.from_iterable(e.want for e in entries), dtype=np.int32, count=int(want_off[E]))
        if want.size:
            bad = (want < 0) | (want >= np.repeat(n_tok, n_want_of))
            if bad.any():
                j = int(np.argmax(bad))
                i = int(np.searchsorted(want_off, j, side="right")) - 1
                raise StepError(f"entry {i} ({seqs[i].seq_id!r}): wanted place {int(want[j])} is outside its {int(n_tok[i])} tokens")
        return _Columns(E, seqs, n_tok, start, T, tokens, tok_off, n_want_of, want_off, want)

    # -- whether a step is replayed as a graph -------------------------------------------------------
    def _replay_key(self, c: "_Columns", n_decode: int, widths: Dict[int, int]):
        """A step can be replayed as a CUDA graph when its launches and the addresses they read depend on nothing but a
        key. A decode-only step that wants every row: the batch is padded to a bucket of entries and of block-table
        width. A step with prompt portions, each entry wanting at most one row: the single tokens are padded to a
        bucket, the number of portions and of their tokens is part of the key (kernels that are launched per tile of
        a portion are given a bound on the tiles that the key fixes), and the key must have been seen before - a
        serving run that cuts long prompts into equal portions repeats it, arbitrary mixes do not.
        Returns (key or None, entries and tokens with the padding, block-table widths)."""
        E, T, n_want_of = c.E, c.T, c.n_want_of
        if not (self.use_graphs and self.tap is None and self.model.graph_safe):
            return None, E, T, widths
        if n_decode == E and int(n_want_of.min()) == 1 and int(n_want_of.max()) == 1:
            Ep = _bucket(E, _ENTRY_BUCKETS)
            widths = {g: _bucket_pow2(w, 16) for g, w in widths.items()}
            return (Ep, tuple(sorted(widths.items()))), Ep, Ep, widths
        single_want = n_want_of[c.n_tok == 1]
        if self.graph_prompts and int(n_want_of.max()) <= 1 and (single_want.size == 0 or int(single_want.min()) == 1):
            Dp = _bucket(n_decode, _ENTRY_BUCKETS) if n_decode else 0
            bw = {g: _bucket_pow2(w, 16) for g, w in widths.items()}
            key = ("portions", Dp, E - n_decode, T - n_decode, tuple(sorted(bw.items())))
            seen = self._shapes_seen.get(key, 0)
            if seen >= self.GRAPH_AFTER:
                return key, Dp + E - n_decode, Dp + T - n_decode, bw
            if len(self._shapes_seen) > 4096:
                self._shapes_seen.clear()
            self._shapes_seen[key] = seen + 1
        return None, E, T, widths

    # -- the step ----------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one batch; returns float32 logits [wanted, vocab] on the device, in the order of
        `entries` and of each entry's `want`.

        A token given as -(1 + i) is not known to the host yet: it is taken from `device_tokens[i]`
        (int32 on the device, e.g. what the sampler drew in the step before) when the step runs."""
        if not entries:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.device)
        last, self._last_decode = self._last_decode, None
        if last is not None:
            logits = self._follow_decode(last, entries, device_tokens)
            if logits is not None:
                return logits
        c = self._columns(entries, device_tokens)
        E, seqs, n_tok, start, T, tokens, tok_off = c.E, c.seqs, c.n_tok, c.start, c.T, c.tokens, c.tok_off
        n_want_of, want_off, want = c.n_want_of, c.want_off, c.want
        # Reserve pages for all entries, or for none.
        new_len = (start + n_tok).tolist()
        if not self.cache.can_reserve(list(zip(seqs, new_len))):
            raise OutOfPages("the step needs more pages than are free: "
                             + ", ".join(f"{e.seq.seq_id!r}+{len(e.tokens)}" for e in entries))
        for s_, n_ in zip(seqs, new_len):
            self.cache.reserve(s_, n_)

        # Single decoded tokens first, prompt portions after; the wanted rows keep the caller's order.
        order = np.argsort(n_tok != 1, kind="stable").astype(np.int32)
        n_decode = int((n_tok == 1).sum())
        groups = self.cache.groups
        paged = [g for g, grp in enumerate(groups) if grp.need.kind == "paged_kv"]
        sub, kpage = self.cache.sub, self.cache.kernel_page      # block tables name kernel pages: `sub` to a page
        tbl_len = np.array([[len(s_.tables[g]) * sub for s_ in seqs] for g in paged], dtype=np.int32).reshape(len(paged), E)
        tbl_ptr = np.array([[s_.tables[g].address() for s_ in seqs] for g in paged], dtype=np.uint64).reshape(len(paged), E)
        widths = {g: max(1, int(tbl_len[k].max())) for k, g in enumerate(paged)}

        graph_key, Ep, Tp, widths = self._replay_key(c, n_decode, widths)
        pad_at, n_want_fixed = (n_decode, Ep) if graph_key is not None else (E, -1)
        n_want = n_want_fixed if graph_key is not None else int(want_off[E])
        n_neg = int((tokens < 0).sum())
        n_patch = Tp if graph_key is not None else n_neg          # a replayed step's buffer is sized once, for any number
        n_ints = (3 * Tp + (Ep + 1) + Ep + max(n_want, 1) + 2 * Ep + sum(Ep * w for w in widths.values()) + 2 * n_patch)
        host, dev = self._desc(n_ints)
        if graph_key is not None:
            gs = self._graphs.get(graph_key)
            if gs is None:
                if len(self._graphs) >= self.MAX_GRAPHS:          # the key used longest ago makes room
                    torch.cuda.current_stream(self.device).synchronize()
                    del self._graphs[next(iter(self._graphs))]
                gs = _GraphSlot(torch.empty(n_ints, dtype=torch.int32, device=self.device))
            else:
                del self._graphs[graph_key]
            self._graphs[graph_key] = gs          # (a dict keeps the order of insertion: the last used key is last)
            dev = gs.desc
        h = host.numpy()
        # ---- the descriptors, filled by native code (csrc/step_fill.cpp) --------------------------------------------
        slots = np.fromiter((s_.state_slot for s_ in seqs), dtype=np.int32, count=E)
        fresh = np.fromiter((s_.fresh_state for s_ in seqs), dtype=np.uint8, count=E)
        w_arr = np.array([widths[g] for g in paged], dtype=np.int32)
        scratch = np.array([groups[g].pool.n_pages * sub for g in paged], dtype=np.int32)
        offs = np.zeros(12, dtype=np.int32)
        outs = np.zeros(3, dtype=np.int32)          # patches, wanted rows, entry at fault
        rc = ops.step_fill(h, host.numel(), E, Ep, Tp, order, n_tok, start, slots, fresh, tokens, tok_off, w_arr, tbl_ptr, tbl_len,
                           scratch, self.cache.slots.n_slots, want, want_off, pad_at, n_want_fixed, n_patch, offs, outs)
        if rc != 0:
            i = int(outs[2])
            who = f"entry {i} ({seqs[i].seq_id!r})" if i >= 0 else "the step"
            raise StepError({-11: f"{who}: a wanted place is outside its {int(n_tok[i]) if i >= 0 else 0} tokens",
                             -12: f"{who}: its block table is wider than the step's", -13: "the step's descriptors outgrew their buffer",
                             -14: f"{who}: more device tokens than the step has room for",
                             -15: "the step's counts do not fit together"}.get(rc, f"step_fill failed ({rc})"))
        n_patches = int(outs[0])
        o = offs.tolist()
        off = o[11]
        s_tok, s_pos, s_ent = (o[0], o[0] + Tp), (o[1], o[1] + Tp), (o[2], o[2] + Tp)
        s_qs, s_kv, s_want = (o[3], o[3] + Ep + 1), (o[4], o[4] + Ep), (o[5], o[5] + max(n_want, 1))
        s_rs, s_wsl = (o[6], o[6] + Ep), (o[7], o[7] + Ep)
        s_bt, a_ = {}, o[8]
        for g in paged:
            s_bt[g] = (a_, a_ + Ep * widths[g])
            a_ += Ep * widths[g]
        s_prow, s_psrc = (o[9], o[9] + n_patch), (o[10], o[10] + n_patch)
        n_pad = Ep - E
        h_qlen = n_tok[order].tolist()
        h_kvlen = (start + n_tok)[order].tolist()
        h_qlen[n_decode:n_decode] = [1] * n_pad
        h_kvlen[n_decode:n_decode] = [1] * n_pad
        dev[:off].copy_(host[:off], non_blocking=True)
        if n_patches:                             # tokens the host has not seen: copied in on the device
            ops.patch_tokens(dev[s_tok[0]: s_tok[1]], dev[s_prow[0]: s_prow[0] + n_patches],
                             dev[s_psrc[0]: s_psrc[0] + n_patches], device_tokens)
        ev = torch.cuda.Event()
        ev.record()
        self._desc_events[self._desc_i] = ev
        self.h2d_bytes += 4 * off

        def view(s):
            return dev[s[0]: s[1]]
        n_single = n_decode + n_pad
        if graph_key is not None:                 # launch plans must not depend on this step's lengths, only on the key
            bound = min(widths[g] for g in paged) * kpage if paged else 1
            h_kvlen = [bound] * Ep
            h_qlen = [1] * n_single + [Tp - n_single] * (Ep - n_single)
        ctx = StepContext(
            dtype=self.dtype, T=Tp, n_entries=Ep, n_decode=n_single,
            token_ids=view(s_tok), tok_pos=view(s_pos), tok_entry=view(s_ent), entry_qstart=view(s_qs),
            entry_kvlen=view(s_kv), want_rows=dev[s_want[0]: s_want[0] + n_want], n_want=n_want, ws=self.ws,
            h_qlen=h_qlen, h_kvlen=h_kvlen, max_qlen=max(h_qlen), max_kvlen=max(h_kvlen), tap=self.tap,
            lengths_are_bounds=graph_key is not None)

        caches = []
        for i, st in enumerate(self.model.order):
            owner = i if st.cache_from is None else st.cache_from
            g = self.cache.group_of_entry.get(owner)
            if g is None:
                caches.append(None)
                continue
            grp = groups[g]
            if grp.need.kind == "paged_kv":
                caches.append(PagedKVView(grp.storage[owner], view(s_bt[g]).view(Ep, widths[g]), kpage,
                                          writable=(owner == i), max_pages=widths[g], tma_map=grp.tma_maps.get(owner)))
            else:
                caches.append(StateView(grp.storage[owner], view(s_rs), view(s_wsl), writable=(owner == i)))

        if graph_key is None:
            logits = self.model.forward(ctx, caches)
        else:
            gs = self._graphs[graph_key]
            if gs.graph is not None and gs.ws_version != self.ws.version:
                gs.graph, gs.warm = None, 0       # a workspace buffer moved: capture again
            if gs.graph is None:
                if gs.warm < 1:                   # first time eagerly: buffers get allocated, libraries initialised
                    logits = self.model.forward(ctx, caches)
                    gs.warm += 1
                    gs.logits = logits
                else:
                    n0 = ops.launch_count()
                    g_ = torch.cuda.CUDAGraph()
                    if self._graph_pool is None:  # one pool for all graphs: they never run at the same time
                        self._graph_pool = torch.cuda.graph_pool_handle()
                    with torch.cuda.graph(g_, pool=self._graph_pool):
                        gs.logits = self.model.forward(ctx, caches)
                    gs.n_kernels = ops.launch_count() - n0
                    ops.count_launches(-gs.n_kernels)    # capturing launches nothing
                    gs.graph = g_
                    gs.ws_version = self.ws.version
            if gs.graph is not None:
                gs.graph.replay()
                ops.count_launches(gs.n_kernels)
                self.portion_replays += n_decode != E
                if n_decode == E and not any(grp.need.kind == "paged_kv" and grp.need.window is not None for grp in groups):
                    # the next step may be the same requests with one more token each: keep what it can start from
                    self._last_decode = _DecodeBatch(
                        seqs=seqs, gs=gs, E=E, Ep=Ep, widths=dict(widths), mirror=h[:off].copy(), lens=start + 1,
                        spans=dict(tok=s_tok, pos=s_pos, kv=s_kv, rs=s_rs, wsl=s_wsl, bt=dict(s_bt), prow=s_prow, psrc=s_psrc), n_ints=off)
            logits = gs.logits[:int(want_off[E])]         # the rows asked for come first, in the caller's order
        for s_, n_ in zip(seqs, new_len):
            self.cache.commit(s_, n_)
        self.steps_run += 1
        self.tokens_run += T
        return logits


@dataclass
class _Columns:
    """A step's entries as arrays (`StepRunner._columns`)."""
    E: int
    seqs: list
    n_tok: np.ndarray                             # tokens an entry brings
    start: np.ndarray                             # tokens it has in the cache
    T: int
    tokens: np.ndarray                            # all tokens, entry after entry (int64; below 0: still on the device)
    tok_off: np.ndarray                           # [E + 1] where an entry's tokens start
    n_want_of: np.ndarray
    want_off: np.ndarray                          # [E + 1] where an entry's wanted places start
    want: np.ndarray                              # all wanted places, entry after entry


@dataclass
class _DecodeBatch:
    """A replayed decode-only step, kept so that the step after it - the same requests in the same order, one more
    token each - is made from it: lengths go up by one, block tables change only where a request starts a page."""
    seqs: list
    gs: "_GraphSlot"
    E: int
    Ep: int
    widths: Dict[int, int]
    mirror: np.ndarray                            # the step's descriptors as they went to the device
    lens: np.ndarray                              # cached tokens per request after that step
    spans: dict
    n_ints: int


_ENTRY_BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512]


def _bucket(n: int, buckets) -> int:
    for b in buckets:
        if n <= b:
            return b
    return ((n + 127) // 128) * 128


def _bucket_pow2(n: int, lo: int) -> int:
    b = lo
    while b < n:
        b *= 2
    return b


class _GraphSlot:
    """One captured decode step: its descriptor buffer, its graph and where its logits land."""

    def __init__(self, desc: torch.Tensor):
        self.desc, self.graph, self.logits, self.warm, self.n_kernels, self.ws_version = desc, None, None, 0, 0, -1
