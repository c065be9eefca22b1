"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees. Pure host code; it decides, the step function runs.

Each step holds, in this order: one token for every running request that is decoding; the next
portion (at most `chunk_size` tokens) of every running request whose prompt is not yet in the
cache, oldest first; then newly admitted requests, while the token budget, the number of live
requests and the pages allow. Decoding requests are never held up by a long prompt.

When pages run out:
  admission "worst_case" (default, InfiniLM's rule): a request is admitted only if the pages that
    all running requests can still need (prompt + max_tokens) plus its own fit; it waits otherwise,
    and a decode step can then never lack a page.
  admission "optimistic": a request is admitted if its next portion fits. If a later step lacks
    pages, the youngest running request is preempted: its pages are given back and it returns to
    the head of the waiting queue with the tokens it has produced appended to its prompt, to be
    recomputed; the request keeps its output.
A request that could never fit (prompt + max_tokens beyond the whole pool or the model's maximum
length) is refused when it is added.

Parity with InfiniLM: `python/infinilm/llm/scheduler.py:55-127` (queues, token budget),
`:129-306` (prefill branch: budget, `can_accept_request`, allocate), `:308-366` (decode branch),
`:404-451` (`complete_requests` frees the pages of finished requests), `:453-501` (worst-case page
check); `python/infinilm/llm/llm.py:279-303` (finish reasons: length, eos_token, stop);
`python/infinilm/llm/request.py:49-83` (request status). InfiniLM never cuts a prompt and never
mixes prefill with decode; both are ours.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager, OutOfPages, SequenceCache
from ..sampling.sampler import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(enum.Enum):
    LENGTH = "length"
    EOS_TOKEN = "eos_token"
    STOP = "stop"
    ABORTED = "aborted"


@dataclass(eq=False)                              # a request is itself: compared and hashed by identity
class Request:
    request_id: str
    prompt_token_ids: List[int]
    params: SamplingParams
    eos_token_ids: Sequence[int] = ()
    prompt: Optional[str] = None
    output_token_ids: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: Optional[FinishReason] = None
    seq: Optional[SequenceCache] = None
    arrival: int = 0
    n_preempted: int = 0
    sample_stream: int = 0                        # which stream of uniform numbers this request draws from
    last_sample_row: int = -1                     # row of this request in the sampler output of the step that last sampled for it
    closing: bool = False                         # its last token is on its way (max_tokens reached): schedule it no more

    @property
    def all_token_ids(self) -> List[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def n_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def tokens_from(self, start: int, n: int) -> List[int]:
        """Tokens start .. start+n of prompt followed by output, without joining the two lists."""
        np_ = len(self.prompt_token_ids)
        if start + n <= np_:
            return self.prompt_token_ids[start: start + n]
        if start >= np_:
            return self.output_token_ids[start - np_: start - np_ + n]
        return self.prompt_token_ids[start:] + self.output_token_ids[: start + n - np_]

    @property
    def n_cached(self) -> int:
        return 0 if self.seq is None else self.seq.length

    @property
    def finished(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.ABORTED)


PENDING = -1     # placeholder in output_token_ids for a token that was sampled on the device and not read back yet


@dataclass
class ScheduledEntry:
    request: Request
    tokens: List[int]                             # PENDING stands for the token the previous step sampled for this request
    samples: bool                                 # the logits of the last token are wanted (and sampled from)
    out_index: int = -1                           # where in output_token_ids the sampled token goes


@dataclass
class SchedulerOutput:
    entries: List[ScheduledEntry]
    preempted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int = 8, max_num_batched_tokens: int = 8192,
                 chunk_size: int = 2048, admission: str = "worst_case", max_model_len: Optional[int] = None):
        if admission not in ("worst_case", "optimistic"):
            raise ValueError("admission must be 'worst_case' or 'optimistic'")
        if max_num_batched_tokens < 1 or chunk_size < 1 or max_batch_size < 1:
            raise ValueError("budgets must be positive")
        self.cache = cache
        self.max_batch_size = min(int(max_batch_size), cache.max_seqs)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.chunk_size = int(chunk_size)
        self.admission = admission
        self.max_model_len = max_model_len
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0
        self.n_preemptions = 0

    # -- sizes -----------------------------------------------------------------------------
    def _pages(self, n_tokens: int) -> int:
        return (n_tokens + self.cache.page_size - 1) // self.cache.page_size

    def _pool_pages(self) -> int:
        pools = [g.pool.n_pages for g in self.cache.groups if g.pool is not None]
        return min(pools) if pools else 1 << 60

    def _free_pages(self) -> int:
        pools = [g.pool.n_free for g in self.cache.groups if g.pool is not None]
        return min(pools) if pools else 1 << 60

    def _held_pages(self, r: Request) -> int:
        if r.seq is None or not r.seq.tables:
            return 0
        return max(len(t) for t in r.seq.tables.values())

    def _worst_case_left(self, r: Request) -> int:
        """Pages `r` can still ask for until it has produced max_tokens."""
        total = len(r.prompt_token_ids) + r.params.max_tokens
        return max(0, self._pages(total) - self._held_pages(r))

    # -- requests ----------------------------------------------------------------------------
    def add_request(self, r: Request) -> None:
        if not r.prompt_token_ids:
            raise ValueError(f"request {r.request_id}: empty prompt")
        total = len(r.prompt_token_ids) + r.params.max_tokens
        if self.max_model_len is not None and len(r.prompt_token_ids) + 1 > self.max_model_len:
            raise ValueError(f"request {r.request_id}: prompt of {len(r.prompt_token_ids)} tokens leaves no room "
                             f"under the model's maximum length {self.max_model_len}")
        if self.max_model_len is not None and total > self.max_model_len:
            r.params = r.params.clone()
            r.params.max_tokens = self.max_model_len - len(r.prompt_token_ids)
            total = self.max_model_len
        if self._pages(total) > self._pool_pages():
            raise ValueError(f"request {r.request_id}: prompt + max_tokens = {total} tokens need "
                             f"{self._pages(total)} pages, the pool has {self._pool_pages()}")
        r.status = RequestStatus.WAITING
        r.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(r)

    def abort(self, request_id: str) -> bool:
        for r in list(self.running):
            if r.request_id == request_id:
                self._finish(r, FinishReason.ABORTED)
                return True
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                r.status, r.finish_reason = RequestStatus.ABORTED, FinishReason.ABORTED
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step's decisions ----------------------------------------------------------------
    def _next_tokens(self, r: Request, budget: int) -> List[int]:
        """The tokens `r` would run next: one if it is decoding, else a portion of what is not
        yet in the cache (prompt, and after a preemption also the tokens already produced)."""
        left = r.n_tokens - r.n_cached
        n = min(left, self.chunk_size, budget)
        return r.tokens_from(r.n_cached, n)

    def _preempt_youngest(self, out: SchedulerOutput, keep: Request) -> bool:
        """Gives back the pages of the youngest running request other than `keep` that is not
        already in this step. Returns False if there is none."""
        in_step = {id(e.request) for e in out.entries}
        # a request whose last token is on its way (`closing`) gives its pages back at the next retire anyway; taken
        # out now it would be admitted and run a second time
        cands = [r for r in self.running if r is not keep and id(r) not in in_step and not r.closing]
        if not cands:
            return False
        victim = max(cands, key=lambda r: r.arrival)
        self.running.remove(victim)
        self.cache.close(victim.seq)
        victim.seq = None
        victim.status = RequestStatus.WAITING
        victim.n_preempted += 1
        self.n_preemptions += 1
        self.waiting.appendleft(victim)
        out.preempted.append(victim)
        return True

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput([])
        budget = self.max_num_batched_tokens
        free = self._free_pages()                 # pages not yet promised to an entry of this step

        def fits(r: Request, n: int) -> int:
            """Pages the next n tokens of r need beyond what it holds, or -1 if they are not free."""
            need = max(0, self._pages(r.n_cached + n) - self._held_pages(r))
            return need if need <= free else -1

        # 1. running requests, decoding ones first (one token each), then unfinished prompts, oldest first
        # (lengths are taken once per request: with hundreds of live requests this pass is the scheduler's cost)
        decoding, filling = [], []
        for r in self.running:
            if r.closing:
                continue
            left = len(r.prompt_token_ids) + len(r.output_token_ids) - r.seq.length
            (decoding if left == 1 else filling).append(r)
        decoding.sort(key=lambda r: r.arrival)
        filling.sort(key=lambda r: r.arrival)
        ps = self.cache.page_size
        for r in decoding + filling:
            if out.preempted and any(r is v for v in out.preempted):      # preempted a moment ago
                continue
            if budget <= 0:
                break
            if r.output_token_ids and len(r.prompt_token_ids) + len(r.output_token_ids) - r.seq.length == 1:
                toks = r.output_token_ids[-1:]    # decoding: its last token, and a page only at a page's edge
                # (the tables of all paged groups grow together; a model without paged groups needs none)
                need = fits(r, 1) if r.seq.tables and r.seq.length % ps == 0 else 0
            else:
                toks = self._next_tokens(r, budget)
                need = fits(r, len(toks))
            while need < 0:
                if self.admission == "optimistic" and self._preempt_youngest(out, r):
                    free = self._free_pages() - sum(
                        max(0, self._pages(e.request.n_cached + len(e.tokens)) - self._held_pages(e.request))
                        for e in out.entries)
                    need = fits(r, len(toks))
                    continue
                break
            if need < 0:
                continue                           # waits for pages; an older request will free some
            free -= need
            budget -= len(toks)
            out.entries.append(ScheduledEntry(r, toks, samples=(r.seq.length + len(toks) == len(r.prompt_token_ids) + len(r.output_token_ids))))

        # 2. admissions, in arrival order; the first that does not fit stops the scan
        promised = None                           # pages the running requests may still ask for (worst case), summed once
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_size:
            r = self.waiting[0]
            if r.finished:                        # ended (or was aborted) while it waited
                self.waiting.popleft()
                continue
            toks = self._next_tokens(r, budget)
            need = self._pages(len(toks))
            if self.admission == "worst_case":
                if promised is None:
                    promised = sum(self._worst_case_left(x) for x in self.running)
                if promised + self._worst_case_left(r) > self._free_pages():
                    break
            if need > free:
                break
            try:
                r.seq = self.cache.open(r.request_id)
            except OutOfPages:
                break
            self.waiting.popleft()
            r.status = RequestStatus.RUNNING
            self.running.append(r)
            if promised is not None:
                promised += self._worst_case_left(r)
            free -= need
            budget -= len(toks)
            out.entries.append(ScheduledEntry(r, toks, samples=(len(toks) == r.n_tokens)))
        return out

    # -- after the step ----------------------------------------------------------------------
    def _finish(self, r: Request, reason: FinishReason) -> None:
        r.status = RequestStatus.ABORTED if reason is FinishReason.ABORTED else RequestStatus.FINISHED
        r.finish_reason = reason
        if r in self.running:
            self.running.remove(r)
        if r in self.waiting:                     # preempted while its last token was on its way: nothing to recompute
            self.waiting.remove(r)
        if r.seq is not None:
            self.cache.close(r.seq)
            r.seq = None

    def launched(self, out: SchedulerOutput) -> None:
        """The step has been issued: every entry that samples gets a PENDING place in its request's
        output (the token is on the device); a request whose output is now max_tokens long is not
        scheduled again (`closing`), so no step runs past a length limit."""
        row = 0
        for e in out.entries:
            if not e.samples:
                continue
            r = e.request
            e.out_index = len(r.output_token_ids)
            r.output_token_ids.append(PENDING)
            r.last_sample_row = row
            row += 1
            if len(r.output_token_ids) >= r.params.max_tokens or (
                    self.max_model_len is not None and r.n_tokens >= self.max_model_len):
                r.closing = True

    def retire(self, out: SchedulerOutput, sampled: Sequence[int]) -> List[Request]:
        """The tokens of a step have been read back (`sampled[i]` for its i-th sampling entry): they
        take their places, the finish rules apply, finished requests give back what they hold. A
        request that ended on an earlier token (end of sequence) while this step already ran ahead
        for it simply drops the token. Returns the requests that finished."""
        finished = []
        row = -1
        for e in out.entries:
            if not e.samples:
                continue
            row += 1
            r = e.request
            if r.finished:
                continue
            tok = int(sampled[row])
            r.output_token_ids[e.out_index] = tok
            p = r.params
            if not p.ignore_eos and tok in r.eos_token_ids:
                reason = FinishReason.EOS_TOKEN
            elif tok in p.stop_token_ids:
                reason = FinishReason.STOP
            elif e.out_index + 1 >= p.max_tokens:
                reason = FinishReason.LENGTH
            elif self.max_model_len is not None and len(r.prompt_token_ids) + e.out_index + 1 >= self.max_model_len:
                reason = FinishReason.LENGTH
            else:
                continue
            del r.output_token_ids[e.out_index + 1:]      # a token a later step ran ahead for is dropped
            self._finish(r, reason)
            finished.append(r)
        return finished

    def update(self, out: SchedulerOutput, sampled: Dict[str, int]) -> List[Request]:
        """Launch and retire in one call, for a caller that reads every step's tokens before the next
        step: `sampled[request_id]` is the token drawn for each entry that sampled."""
        self.launched(out)
        return self.retire(out, [sampled[e.request.request_id] for e in out.entries if e.samples])

    def stats(self) -> Dict[str, int]:
        return {"waiting": len(self.waiting), "running": len(self.running), "free_pages": self._free_pages(),
                "pool_pages": self._pool_pages(), "preemptions": self.n_preemptions}
