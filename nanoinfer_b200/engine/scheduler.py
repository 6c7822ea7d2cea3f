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

The decisions are made by compiled code (csrc/host_runtime.cpp, as the reference's scheduler is
C++); it knows requests by id and by counts.  This class keeps the request objects, translates
a decision into (request, number of tokens) pairs and reports sampled tokens back.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

from ..cache import CacheManager, native
from .request import InferenceRequest


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


def _ids(values) -> "ctypes.Array":
    return (ctypes.c_longlong * max(len(values), 1))(*values)


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
        self.requests: Dict[int, InferenceRequest] = {}
        self._lib = native.lib()
        self._h = self._lib.ni_sched_create(cache._h, max_batch_size, max_sequences, prefill_chunk_size,
                                            max_num_batched_tokens)
        if not self._h:
            raise ValueError("the scheduler could not be created from these limits")
        self._buf = (ctypes.c_longlong * max(max_batch_size, cache.max_requests, 1))()

    def __del__(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ni_sched_destroy(self._h)
            self._h = None

    def request_field(self, request_id: int, field_index: int) -> int:
        """A count of a request as the compiled scheduler keeps it (0 state, 1 computed tokens,
        2 tokens on the way, 3 generated tokens, 4 preemptions, 5 remaining tokens)."""
        return self._lib.ni_sched_get(self._h, request_id, field_index)

    def add_request(self, req: InferenceRequest) -> None:
        if type(req.request_id) is not int or req.request_id < 0:
            raise ValueError("request ids are non-negative integers")
        if self._lib.ni_sched_add(self._h, req.request_id, len(req.prompt_tokens), req.max_new_tokens) != 0:
            raise ValueError(f"request {req.request_id} cannot be added (id in use, empty prompt or no tokens to generate)")
        self.requests[req.request_id] = req
        req._scheduler = self

    def has_work(self) -> bool:
        return bool(self._lib.ni_sched_has_work(self._h))

    def _result(self, what: int) -> List[int]:
        n = self._lib.ni_sched_result(self._h, what, self._buf, len(self._buf))
        return list(self._buf[:n])

    # ---- one scheduling decision ----------------------------------------------------------
    def schedule(self) -> ScheduledBatch:
        batch = ScheduledBatch()
        n = self._lib.ni_sched_schedule(self._h)
        if n:
            ids, counts = self._result(0), self._result(1)
            batch.entries = [(self.requests[i], c) for i, c in zip(ids, counts)]
        batch.preempted = [self.requests[i] for i in self._result(2)]
        for i in self._result(3):
            req = self.requests[i]
            req.fail("out_of_pages")
            batch.failed.append(req)
        return batch

    # ---- after the forward pass -----------------------------------------------------------
    def advance(self, batch: ScheduledBatch, emitting) -> None:
        """The batch has been launched: its tokens count as computed, and every request in
        ``emitting`` has one sampled token on the way (known to the host at ``commit``)."""
        n = len(batch.entries)
        counts = (ctypes.c_int32 * max(n, 1))(*[c for _, c in batch.entries])
        emit = [r.request_id for r in emitting]
        rc = self._lib.ni_sched_advance(self._h, n, _ids([r.request_id for r, _ in batch.entries]), counts,
                                        len(emit), _ids(emit))
        if rc != 0:
            raise RuntimeError("the scheduler does not know a request of this batch")

    def commit(self, sampled: Dict[int, int]) -> List[InferenceRequest]:
        """``sampled[request_id]`` is the token drawn for a request whose token was on the way.
        A request that finished or was dropped meanwhile ignores it.  Returns the requests that
        finished; their pages and slots are given back."""
        finished = []
        for rid, tok in sampled.items():
            req = self.requests[rid]
            if req.is_finished() or req.num_pending == 0:
                continue
            alive = req.add_token(tok)
            self._lib.ni_sched_commit(self._h, rid, 0 if alive else 1)
            if not alive:
                finished.append(req)
        return finished

    def abort(self, req: InferenceRequest, reason: str) -> bool:
        """End a request as failed, whatever its state; its pages and slot are given back.
        Returns False if it had ended before."""
        if self._lib.ni_sched_abort(self._h, req.request_id) != 1:
            return False
        req.fail(reason)
        return True

    def running_requests(self) -> List[InferenceRequest]:
        return [r for r in self.requests.values() if r._ended is None and self.request_field(r.request_id, 0) == 1]

    def update_after_step(self, batch: ScheduledBatch, sampled: Dict[int, int]) -> List[InferenceRequest]:
        """advance + commit in one call, for a step whose tokens are read at once."""
        self.advance(batch, [req for req, _ in batch.entries if req.request_id in sampled])
        return self.commit(sampled)

    def can_continue_decoding(self, previous: ScheduledBatch) -> bool:
        """True if the next decision is known without the tokens of ``previous``, the batch
        still in flight: it held every running request, all of them get their token from it
        and go on decoding, nobody waits for admission, and every page they need is free - so
        the next batch is the same requests in the same order, one token each."""
        ids = [r.request_id for r, _ in previous.entries]
        return bool(self._lib.ni_sched_can_continue(self._h, _ids(ids), len(ids)))

    @property
    def num_preemptions(self) -> int:
        return self._lib.ni_sched_stat(self._h, 4)

    @property
    def num_finished(self) -> int:
        return self._lib.ni_sched_stat(self._h, 2)

    def stats(self) -> SchedulerStats:
        st = self._lib.ni_sched_stat
        return SchedulerStats(st(self._h, 0), st(self._h, 1), st(self._h, 2), st(self._h, 3), st(self._h, 4))
