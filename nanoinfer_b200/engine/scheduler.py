"""First-come-first-served scheduler with continuous batching and chunked prefill.

Every step is ONE batch: each running request contributes its next tokens - one token if it
is decoding, otherwise a portion of at most ``prefill_chunk_size`` - and waiting requests are
admitted in arrival order while the token budget, the batch size, the request slots and the
pages allow.  Pages are taken portion by portion.

The reference admits by batch size and sequence count only, reserves the pages of a whole
prompt when a request is added, runs every prefill portion as a forward pass of its own
(src/engine/scheduler.cpp:51-91, src/engine/engine.cpp:142-173,215-250) and stops the whole
engine when a decode step finds no free page (src/engine/engine.cpp:403-404,194-198).

When pages run out here: the most recently admitted running request is preempted - its pages
and slot are given back, it returns to the FRONT of the waiting queue and is recomputed
later from its prompt plus the tokens it had generated.  If the request that needs the page
is the only one running, the pool is simply too small for it: it fails with reason
"out_of_pages" and the engine goes on.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..cache import CacheManager
from .request import InferenceRequest, RequestState


@dataclass
class ScheduledBatch:
    """(request, number of tokens) pairs of one step, plus what the decision displaced."""
    entries: List[Tuple[InferenceRequest, int]] = field(default_factory=list)
    preempted: List[InferenceRequest] = field(default_factory=list)
    failed: List[InferenceRequest] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(n for _, n in self.entries)


@dataclass
class SchedulerStats:
    num_running: int
    num_waiting: int
    num_finished: int
    total_requests: int
    num_preemptions: int


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int = 32, max_sequences: int = 128,
                 prefill_chunk_size: int = 512, max_num_batched_tokens: int = 2048) -> None:
        if min(max_batch_size, max_sequences, prefill_chunk_size, max_num_batched_tokens) <= 0:
            raise ValueError("scheduler limits must be positive")
        self.cache = cache
        self.max_batch_size = max_batch_size
        self.max_sequences = min(max_sequences, cache.max_requests)
        self.prefill_chunk_size = prefill_chunk_size
        self.max_num_batched_tokens = max_num_batched_tokens
        self.waiting: Deque[InferenceRequest] = deque()
        self.running: List[InferenceRequest] = []   # in order of admission
        self.requests: Dict[int, InferenceRequest] = {}
        self.num_finished = 0
        self.num_preemptions = 0

    def add_request(self, req: InferenceRequest) -> None:
        self.requests[req.request_id] = req
        req.state = RequestState.WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one scheduling decision ----------------------------------------------------------
    def schedule(self) -> ScheduledBatch:
        cache = self.cache
        batch = ScheduledBatch()
        n_groups = len(cache.groups)
        reserved = [0] * n_groups            # pages this step's entries will take
        budget = self.max_num_batched_tokens
        # decoding requests need one token each: set that aside before portions are cut
        decoding = sum(1 for r in self.running if r.num_remaining == 1)
        portion_budget = max(0, budget - decoding)

        one_page, no_page = [1] * n_groups, [0] * n_groups

        def fits(need) -> bool:
            if need is no_page:
                return True
            return all(reserved[g] + need[g] <= cache.num_free_pages(g) for g in range(n_groups))

        i = 0
        while i < len(self.running):
            req = self.running[i]
            if len(batch.entries) >= self.max_batch_size:
                break
            remaining = req.num_remaining
            if remaining == 1:
                n = 1 if budget > 0 else 0
            else:
                n = min(remaining, self.prefill_chunk_size, portion_budget)
            if n <= 0:
                i += 1
                continue
            if n == 1 and cache.has(req.request_id):
                need = one_page if cache.needs_page_for_one(req.request_id) else no_page
            else:
                need = cache.pages_needed(req.request_id, n)
            while not fits(need):
                victim = self.running[-1]
                if victim is req:
                    if len(self.running) == 1:
                        # alone and still no room: the pool cannot hold this request
                        self._drop(req)
                        req.fail("out_of_pages")
                        self.num_finished += 1
                        batch.failed.append(req)
                    else:
                        self._preempt(req)
                        batch.preempted.append(req)
                    req = None
                    break
                self._preempt(victim)
                batch.preempted.append(victim)
            if req is None:
                continue                      # running[i] is now the next request (or the end)
            batch.entries.append((req, n))
            if need is not no_page:
                reserved = [a + b for a, b in zip(reserved, need)]
            budget -= n
            if remaining > 1:
                portion_budget -= n
            i += 1

        # admit waiting requests in arrival order; stop at the first that does not fit
        slots_left = cache.num_free_slots
        while (self.waiting and not batch.preempted and len(self.running) < self.max_sequences
               and len(batch.entries) < self.max_batch_size and slots_left > 0):
            req = self.waiting[0]
            n = min(req.num_remaining, self.prefill_chunk_size, portion_budget)
            if n <= 0:
                break
            need = cache.pages_for_new_request(n)
            if not fits(need):
                if not self.running and not batch.entries:
                    # nothing is running and the first portion still does not fit
                    self.waiting.popleft()
                    req.fail("out_of_pages")
                    self.num_finished += 1
                    batch.failed.append(req)
                    continue
                break
            self.waiting.popleft()
            req.state = RequestState.RUNNING
            self.running.append(req)
            batch.entries.append((req, n))
            reserved = [a + b for a, b in zip(reserved, need)]
            budget -= n
            portion_budget -= n
            slots_left -= 1
        return batch

    def _drop(self, req: InferenceRequest) -> None:
        self.running.remove(req)
        if self.cache.has(req.request_id):
            self.cache.free(req.request_id)

    def _preempt(self, req: InferenceRequest) -> None:
        self._drop(req)
        req.num_computed_tokens = 0
        req.state = RequestState.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    # ---- after the forward pass -----------------------------------------------------------
    def advance(self, batch: ScheduledBatch, emitting) -> None:
        """The batch has been launched: its tokens count as computed, and every request in
        ``emitting`` has one sampled token on the way (known to the host at ``commit``)."""
        for req, n in batch.entries:
            req.num_computed_tokens += n
        for req in emitting:
            req.num_pending += 1

    def commit(self, sampled: Dict[int, int]) -> List[InferenceRequest]:
        """``sampled[request_id]`` is the token drawn for a request whose token was on the way.
        A request that finished or was dropped meanwhile ignores it.  Returns the requests that
        finished; their pages and slots are given back."""
        finished = []
        for rid, tok in sampled.items():
            req = self.requests[rid]
            if req.is_finished() or req.num_pending == 0:
                continue
            if not req.add_token(tok):
                finished.append(req)
        for req in finished:
            if req in self.running:
                self._drop(req)
            else:
                self.waiting.remove(req)      # finished while preempted
            self.num_finished += 1
        return finished

    def update_after_step(self, batch: ScheduledBatch, sampled: Dict[int, int]) -> List[InferenceRequest]:
        """advance + commit in one call, for a step whose tokens are read at once."""
        self.advance(batch, [req for req, _ in batch.entries if req.request_id in sampled])
        return self.commit(sampled)

    def can_continue_decoding(self, previous: ScheduledBatch) -> bool:
        """True if the next decision is known without the tokens of ``previous``, the batch
        still in flight: it held every running request, all of them get their token from it
        and go on decoding, nobody waits for admission, and every page they need is free - so
        the next batch is the same requests in the same order, one token each."""
        if self.waiting or len(previous.entries) != len(self.running):
            return False
        need = 0
        for (req, _), running in zip(previous.entries, self.running):
            if req is not running or req.num_pending != 1 or req.num_remaining != 1 or req.pending_reaches_limit():
                return False
            need += self.cache.needs_page_for_one(req.request_id)
        return (len(self.running) <= min(self.max_batch_size, self.max_num_batched_tokens)
                and all(need <= self.cache.num_free_pages(g) for g in range(len(self.cache.groups))))

    def stats(self) -> SchedulerStats:
        return SchedulerStats(len(self.running), len(self.waiting), self.num_finished,
                              len(self.requests), self.num_preemptions)
