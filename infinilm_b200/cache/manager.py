"""The cache manager: pages of keys and values with a block table per request, groups of layers
with pages of their own, and slots for per-request state of fixed size.

Host-side bookkeeping is plain Python and runs without a GPU (device storage is only allocated
when a device is given), so every decision here is tested on the CPU.

Parity with InfiniLM: `python/infinilm/llm/cache_manager.py:71-364` (`BlockManager`: free list,
pages handed out at allocation, given back when a request ends, `allocate_slots` / `append_slot`
/ `free_blocks`), `:33-68` (`MambaCacheManager`: a pool of fixed-size state rows, row 0 kept as
the zero state), `csrc/cache/kv_cache.cpp:113-148` (one tensor of pages per layer). Ours differs
in that pages hold [K|V] of a page side by side, groups with a window give pages back as the
window passes them, and no slot mapping is kept: a token's slot follows from block table and position.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..parts.spec import CacheNeed


class OutOfPages(RuntimeError):
    """A reservation needs more free pages (or state slots) than there are."""


class CacheStateError(RuntimeError):
    """A page or slot was freed twice, or a request was used after it was closed."""


class PagePool:
    """Page ids 0..n-1; first-in first-out reuse, so a page just freed is not the next one out."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free: Deque[int] = deque(range(self.n_pages))
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.popleft()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not (0 <= page < self.n_pages) or not self._held[page]:
            raise CacheStateError(f"page {page} freed while not held")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


class StateSlots:
    """Fixed-size per-request state: slot 0 is reserved as the zero state, 1..n-1 are handed out."""

    def __init__(self, n_slots: int):
        self.n_slots = int(n_slots)
        self._free: Deque[int] = deque(range(1, self.n_slots))
        self._held = [False] * self.n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        s = self._free.popleft()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not (1 <= slot < self.n_slots) or not self._held[slot]:
            raise CacheStateError(f"state slot {slot} freed while not held")
        self._held[slot] = False
        self._free.append(slot)


@dataclass
class CacheGroup:
    """Run-order entries whose caches have the same geometry and policy share page ids:
    one block table per (request, group), one storage tensor per entry."""
    need: CacheNeed
    entries: List[int]                            # run-order indices that own a cache in this group
    pool: Optional[PagePool] = None               # paged_kv groups
    storage: Dict[int, object] = field(default_factory=dict)   # run-order index -> device tensor
    tma_maps: Dict[int, object] = field(default_factory=dict)  # run-order index -> tensor map of its storage (or absent)


class PageTable(list):
    """A request's page ids of one group (a list: -1 where a page was given back) with an int32 array kept beside it, so
    that a step can copy the table into its descriptors without walking it: with hundreds of live requests, lists turned
    into arrays every step were most of a decode step's host time. The array is what the kernels read: a page of the
    manager is `sub` kernel pages that lie one behind the other, so page p stands there as p*sub .. p*sub+sub-1.
    `append`, `tbl[i] = p` and `clear` keep the array in step; any other change marks it stale and `array()` rebuilds it."""

    def __init__(self, *a, sub: int = 1):
        super().__init__(*a)
        self.sub = int(sub)
        self._arr = np.empty(max(16, 2 * len(self)) * self.sub, dtype=np.int32)
        self._stale = len(self) > 0
        self._steps = np.arange(self.sub, dtype=np.int32)
        self._addr_of, self._addr = None, 0       # the array whose address `_addr` is

    def _put(self, i: int, p: int) -> None:
        sub = self.sub
        if sub == 1:
            self._arr[i] = p
        elif p < 0:
            self._arr[i * sub: (i + 1) * sub] = -1
        else:
            self._arr[i * sub: (i + 1) * sub] = p * sub + self._steps

    def append(self, p) -> None:
        n = len(self)
        super().append(p)
        if (n + 1) * self.sub > self._arr.shape[0]:
            grown = np.empty(2 * self._arr.shape[0], dtype=np.int32)
            grown[:n * self.sub] = self._arr[:n * self.sub]
            self._arr = grown
        self._put(n, p)

    def __setitem__(self, i, p) -> None:
        super().__setitem__(i, p)
        if isinstance(i, int):
            self._put(i if i >= 0 else len(self) + i, p)
        else:
            self._stale = True

    def clear(self) -> None:
        super().clear()
        self._stale = False

    def _touched(name):                           # noqa: N805 (a helper of the class body, deleted below)
        def f(self, *a, **k):
            self._stale = True
            return getattr(list, name)(self, *a, **k)
        return f
    extend, insert, pop, remove = _touched("extend"), _touched("insert"), _touched("pop"), _touched("remove")
    reverse, sort = _touched("reverse"), _touched("sort")
    __delitem__, __iadd__, __imul__ = _touched("__delitem__"), _touched("__iadd__"), _touched("__imul__")
    del _touched

    @property
    def n_kernel_pages(self) -> int:
        return len(self) * self.sub

    def address(self) -> int:
        """Host address of the kernel page ids (int32, `n_kernel_pages` of them), for native code; valid until the table changes."""
        if self._stale:
            self.array()
        if self._addr_of is not self._arr:        # (taking .ctypes.data costs a microsecond: once per array)
            self._addr_of, self._addr = self._arr, self._arr.ctypes.data
        return self._addr

    def array(self) -> np.ndarray:
        """The kernel page ids as int32 [len * sub]; a view, valid until the table changes."""
        n = len(self)
        if self._stale:
            if n * self.sub > self._arr.shape[0]:
                self._arr = np.empty(2 * n * self.sub, dtype=np.int32)
            for i, p in enumerate(self):
                self._put(i, p)
            self._stale = False
        return self._arr[:n * self.sub]


@dataclass(eq=False)                              # a request's cache is itself: compared by identity
class SequenceCache:
    """What the cache holds for one request."""
    seq_id: object
    length: int = 0                               # tokens whose keys/values (or state) are in the cache
    tables: Dict[int, List[int]] = field(default_factory=dict)   # group -> page id per page index (-1: given back)
    state_slot: int = 0
    fresh_state: bool = True                      # no step has run yet: state groups start from the zero state
    open: bool = True


class CacheManager:
    KERNEL_PAGE = 16

    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_size: int, num_pages: int, max_seqs: int,
                 device=None, dtype=None, pages_per_group: Optional[Dict[int, int]] = None):
        """`needs[i]` is what run-order entry i keeps (None: nothing). `num_pages` pages are made
        for every paged group (or `pages_per_group[g]`); `max_seqs` bounds live requests."""
        self.page_size, self.max_seqs = int(page_size), int(max_seqs)
        if self.page_size <= 0 or (self.page_size & (self.page_size - 1)):
            raise ValueError("page_size must be a power of two")
        # What the kernels call a page is `KERNEL_PAGE` tokens (the tile of the attention kernels). A larger page of the
        # manager is `sub` of them one behind the other in memory: requests get and give back whole pages, block tables
        # name kernel pages. A smaller page is a kernel page of its own size (plain kernels only).
        self.kernel_page = min(self.page_size, self.KERNEL_PAGE)
        self.sub = self.page_size // self.kernel_page
        self.groups: List[CacheGroup] = []
        self.group_of_entry: Dict[int, int] = {}
        by_key: Dict[Tuple, int] = {}
        for i, need in enumerate(needs):
            if need is None:
                continue
            k = need.group_key()
            if k not in by_key:
                by_key[k] = len(self.groups)
                self.groups.append(CacheGroup(need, []))
            g = by_key[k]
            self.groups[g].entries.append(i)
            self.group_of_entry[i] = g
        for g, grp in enumerate(self.groups):
            if grp.need.kind == "paged_kv":
                grp.pool = PagePool((pages_per_group or {}).get(g, num_pages))
            elif grp.need.kind != "state":
                raise ValueError(f"unknown cache kind {grp.need.kind!r}")
        self.has_state = any(g.need.kind == "state" for g in self.groups)
        self.slots = StateSlots(self.max_seqs + 1)
        self.live: Dict[object, SequenceCache] = {}
        self.device, self.dtype = device, dtype
        if device is not None:
            self._allocate_storage()

    # -- device storage --------------------------------------------------------------------
    def _allocate_storage(self) -> None:
        import torch
        for grp in self.groups:
            n = grp.need
            for i in grp.entries:
                if n.kind == "paged_kv":
                    # one page more than the pool hands out: padding rows of a replayed step write there
                    shape = ((grp.pool.n_pages + 1) * self.sub, 2, n.n_kv_heads, self.kernel_page, n.head_dim)
                    dt = self.dtype
                else:
                    # one slot more than are handed out: padding rows of a replayed step write there
                    shape = (self.slots.n_slots + 1,) + tuple(n.shape)
                    dt = torch.float32 if n.dtype == "float32" else self.dtype
                grp.storage[i] = torch.zeros(shape, dtype=dt, device=self.device)
                if n.kind == "paged_kv" and dt == torch.bfloat16 and self.kernel_page == 16:
                    from .. import ops
                    m = ops.kv_tensor_map(grp.storage[i])
                    if m is not None:
                        grp.tma_maps[i] = m

    def bytes_per_token(self, elem_size: int) -> int:
        b = 0
        for grp in self.groups:
            if grp.need.kind == "paged_kv":
                b += len(grp.entries) * 2 * grp.need.n_kv_heads * grp.need.head_dim * elem_size
        return b

    # -- requests --------------------------------------------------------------------------
    def open(self, seq_id) -> SequenceCache:
        if seq_id in self.live:
            raise CacheStateError(f"request {seq_id!r} is already open")
        if len(self.live) >= self.max_seqs:
            raise OutOfPages(f"{self.max_seqs} requests are live already")
        seq = SequenceCache(seq_id, state_slot=self.slots.alloc())
        for g, grp in enumerate(self.groups):
            if grp.need.kind == "paged_kv":
                seq.tables[g] = PageTable(sub=self.sub)
        self.live[seq_id] = seq
        return seq

    def _first_needed_page(self, grp: CacheGroup, first_query_pos: int) -> int:
        """Index of the first page a query at `first_query_pos` (or later) can still read."""
        w = grp.need.window
        if w is None:
            return 0
        return max(0, first_query_pos - w + 1) // self.page_size

    def pages_needed(self, seq: SequenceCache, new_len: int) -> Dict[int, int]:
        """How many new pages each paged group needs so that positions < new_len are covered."""
        out = {}
        n_idx = (new_len + self.page_size - 1) // self.page_size
        for g, tbl in seq.tables.items():
            out[g] = max(0, n_idx - len(tbl))
        return out

    def can_reserve(self, wants: Sequence[Tuple[SequenceCache, int]]) -> bool:
        """Whether all of `wants` (request, new length) can be reserved together now."""
        total: Dict[int, int] = {}
        ps = self.page_size
        for seq, new_len in wants:
            n_idx = (new_len + ps - 1) // ps
            for g, tbl in seq.tables.items():
                if n_idx > len(tbl):              # most decode steps need no page: nothing is built for them
                    total[g] = total.get(g, 0) + n_idx - len(tbl)
        return all(self.groups[g].pool.n_free >= n for g, n in total.items())

    def reserve(self, seq: SequenceCache, new_len: int) -> None:
        """Grows the block tables so that positions < new_len have pages. All or nothing."""
        self._check_open(seq)
        if new_len < seq.length:
            raise CacheStateError("a reservation cannot shrink a request")
        n_idx = (new_len + self.page_size - 1) // self.page_size
        if all(n_idx <= len(tbl) for tbl in seq.tables.values()):
            return
        need = self.pages_needed(seq, new_len)
        for g, n in need.items():
            if self.groups[g].pool.n_free < n:
                raise OutOfPages(f"request {seq.seq_id!r} needs {n} more page(s) in cache group {g}, "
                                 f"{self.groups[g].pool.n_free} are free")
        for g, n in need.items():
            for _ in range(n):
                seq.tables[g].append(self.groups[g].pool.alloc())

    def commit(self, seq: SequenceCache, new_len: int) -> None:
        """The step that wrote positions < new_len has been issued: advance the length and give
        back pages that a window has passed (no later query can read them)."""
        self._check_open(seq)
        seq.length = new_len
        seq.fresh_state = False
        for g, tbl in seq.tables.items():
            grp = self.groups[g]
            if grp.need.window is None:
                continue
            first = self._first_needed_page(grp, new_len)
            for idx in range(min(first, len(tbl))):
                if tbl[idx] >= 0:
                    grp.pool.free(tbl[idx])
                    tbl[idx] = -1

    def close(self, seq: SequenceCache) -> None:
        """The request is finished: all it holds is given back."""
        self._check_open(seq)
        for g, tbl in seq.tables.items():
            for p in tbl:
                if p >= 0:
                    self.groups[g].pool.free(p)
            tbl.clear()
        self.slots.free(seq.state_slot)
        seq.open = False
        del self.live[seq.seq_id]

    def _check_open(self, seq: SequenceCache) -> None:
        if not seq.open or self.live.get(seq.seq_id) is not seq:
            raise CacheStateError(f"request {seq.seq_id!r} is not open")

    # -- views -----------------------------------------------------------------------------
    def free_pages(self) -> Dict[int, int]:
        return {g: grp.pool.n_free for g, grp in enumerate(self.groups) if grp.pool is not None}

    def check_invariants(self) -> None:
        """No page lost, none held twice: used by tests and debug runs."""
        for g, grp in enumerate(self.groups):
            if grp.pool is None:
                continue
            held = []
            for seq in self.live.values():
                held += [p for p in seq.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheStateError(f"group {g}: a page is held twice")
            if sorted(held) != grp.pool.held():
                raise CacheStateError(f"group {g}: pages held by requests differ from the pool's record")
            if len(held) + grp.pool.n_free != grp.pool.n_pages:
                raise CacheStateError(f"group {g}: a page is lost")


@dataclass
class PagedKVView:
    """What a mixer sees of a paged cache in one step."""
    storage: object                               # [kernel pages, 2, kv_heads, page_size, head_dim]
    block_table: object                           # int32 [entries, width] on the device: kernel page ids
    page_size: int                                # tokens of a kernel page
    writable: bool = True
    max_pages: int = 0                            # width in use this step
    tma_map: object = None                        # tensor map of `storage` for kernels that copy pages by TMA


@dataclass
class StateView:
    """What a mixer sees of a state group in one step: read from `read_slots` (slot 0, the zero
    state, for a request's first step), write to `write_slots`."""
    storage: object                               # [slots + 1, *shape]; the last one is scratch for padding rows
    read_slots: object                            # int32 [entries]
    write_slots: object                           # int32 [entries]
    writable: bool = True
