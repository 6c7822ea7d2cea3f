"""The step function: one forward pass over a batch of (request, its next tokens).

A step runs only the tokens it is given - portions of prompts beside single decoded
tokens, cut anywhere - against the cache that earlier steps left, and returns FP32 logits
at the wanted places.  The reference runs every prefilling request alone and the decoding
ones as a second batch (src/engine/engine.cpp:215-250), with one prefill flag per batch
(include/nanoinfer/model/model.h:19-31), and computes logits for every row
(src/engine/engine.cpp:312-330).

``ModelRunner`` owns the device side of the cache (page tensors per layer run, state
tensors) next to the host-side ``CacheManager``; generation (scheduler + sampling) and
trace replay both drive this one class.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, GroupSpec, OutOfPages
from ..config.model_config import ModelConfig
from ..parts.base import PagedKVNeed, StateNeed
from .model import DecoderModel
from .runtime import Runtime


class StepError(ValueError):
    """A step's entries are invalid (bad token id, too long, unknown request...)."""


@dataclass
class StepEntry:
    """One request's part of a step: its next tokens and the places (indices into these
    tokens) whose logits are wanted."""
    request: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class CacheView:
    """What a mixer sees of the cache for one layer run."""
    group: int = -1
    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    writable: bool = True


@dataclass
class StepContext:
    """Device-side description of a step, shared by all layers.

    tokens, positions, seq_of_token: int32 [T];  cu_q: int32 [B+1] token offsets per
    request;  kv_len: int32 [B] cached length after this step;  slots: int32 [B] state slot
    per request;  logit_rows: int32 [R];  block_tables[g]: int32 [B, W] of group g.
    The host_* fields hold the same numbers for decisions made on the host.
    """
    n_tokens: int
    n_seqs: int
    n_logit_rows: int
    tokens: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    cu_q: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    block_tables: List[torch.Tensor]
    host_q_lens: List[int] = field(default_factory=list)
    host_kv_lens: List[int] = field(default_factory=list)
    host_slots: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0


def reserve_entries(cache: CacheManager, entries: Sequence[StepEntry], admit) -> List[int]:
    """Take slots and pages for every entry of a step, all or nothing.

    Every group's pool and the slot count are checked before anything is taken, so a step
    that does not fit raises OutOfPages (or StepError) and leaves the cache unchanged.
    ``admit(request)`` is called for requests the cache does not know yet.  Returns each
    entry's start position (its cached length before this step).
    """
    need = [0] * len(cache.groups)
    new_requests = 0
    for e in entries:
        if cache.has(e.request):
            per_group = cache.pages_needed(e.request, len(e.tokens))
        else:
            per_group = cache.pages_for_new_request(len(e.tokens))
            new_requests += 1
        need = [a + b for a, b in zip(need, per_group)]
    if new_requests > cache.num_free_slots:
        raise StepError(f"{new_requests} new requests but only {cache.num_free_slots} free slots")
    for g, n in enumerate(need):
        if n > cache.num_free_pages(g):
            raise OutOfPages(f"group {g}: the step needs {n} more pages, "
                             f"{cache.num_free_pages(g)} are free")
    for e in entries:
        if not cache.has(e.request):
            admit(e.request)
    starts = [cache.length(e.request) for e in entries]
    for e in entries:
        cache.append(e.request, len(e.tokens))
    return starts


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class ModelRunner:
    def __init__(self, config: ModelConfig, weights: Dict[str, torch.Tensor], *, dtype,
                 page_size: int = 16, num_pages: int = 1024, max_requests: int = 8,
                 max_tokens_per_request: Optional[int] = None, device: str = "cuda:0") -> None:
        from .runtime import parse_dtype
        self.config = config
        self.rt = Runtime(device=torch.device(device), dtype=parse_dtype(dtype), page_size=page_size)
        self.model = DecoderModel(config, weights, self.rt)
        if max_tokens_per_request is None:
            max_tokens_per_request = min(config.max_position_embeddings, num_pages * page_size)
        self.max_tokens_per_request = min(max_tokens_per_request, config.max_position_embeddings)

        # cache groups: one per distinct need among the runs that own a cache
        needs = self.model.cache_needs()
        group_specs: List[GroupSpec] = []
        self.caches: List[Optional[CacheView]] = [None] * len(needs)
        self._state_runs: List[int] = []
        for r, need in enumerate(needs):
            if isinstance(need, PagedKVNeed):
                spec = GroupSpec(need.num_kv_heads, need.head_dim, need.window)
                if spec not in group_specs:
                    group_specs.append(spec)
                self.caches[r] = CacheView(group=group_specs.index(spec))
            elif isinstance(need, StateNeed):
                self.caches[r] = CacheView()
                self._state_runs.append(r)
            elif need is not None:
                raise StepError(f"run {r}: unknown cache need {need!r}")
        if not group_specs:
            group_specs.append(GroupSpec(0, 0, None))  # bookkeeping of lengths only
        self.cache = CacheManager(group_specs, [num_pages] * len(group_specs), page_size,
                                  max_requests, self.max_tokens_per_request)
        rt = self.rt
        for r, need in enumerate(needs):
            view = self.caches[r]
            if isinstance(need, PagedKVNeed):
                shape = (num_pages, need.num_kv_heads, page_size, need.head_dim)
                view.k_pages = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
                view.v_pages = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
            elif isinstance(need, StateNeed):
                dt = rt.dtype if need.dtype == "compute" else getattr(torch, need.dtype)
                view.state = torch.zeros((max_requests,) + tuple(need.shape), dtype=dt, device=rt.device)
        for r, run in enumerate(config.schedule):
            if run.cache_of is not None:
                src = self.caches[run.cache_of]
                self.caches[r] = CacheView(group=src.group, k_pages=src.k_pages, v_pages=src.v_pages,
                                           state=src.state, writable=False)
        self._pinned: List[torch.Tensor] = []
        self._pinned_events: List[torch.cuda.Event] = []
        self._pinned_next = 0
        self._dev_meta: Optional[torch.Tensor] = None

    # ---- metadata -------------------------------------------------------------------------
    def _upload(self, host: np.ndarray) -> torch.Tensor:
        n = host.size
        if self._dev_meta is None or self._dev_meta.numel() < n:
            cap = max(4096, _round_up(n * 2, 1024))
            self._dev_meta = torch.empty(cap, dtype=torch.int32, device=self.rt.device)
            self._pinned = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._pinned_events = [torch.cuda.Event() for _ in range(4)]
            self._pinned_used = [False] * 4
        i = self._pinned_next
        self._pinned_next = (i + 1) % len(self._pinned)
        if self._pinned_used[i]:
            self._pinned_events[i].synchronize()
        self._pinned[i][:n].numpy()[:] = host
        self._dev_meta[:n].copy_(self._pinned[i][:n], non_blocking=True)
        self._pinned_events[i].record()
        self._pinned_used[i] = True
        return self._dev_meta

    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.config.vocab_size
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r}: an entry needs at least one token")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise StepError(f"request {e.request!r}: token id {t} is outside [0, {vocab})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            held = self.cache.length(e.request) if self.cache.has(e.request) else 0
            if held + n > self.max_tokens_per_request:
                raise StepError(f"request {e.request!r} would reach {held + n} tokens, more than "
                                f"the limit of {self.max_tokens_per_request}")

    def admit(self, request) -> int:
        slot = self.cache.admit(request)
        for r in self._state_runs:
            self.caches[r].state[slot].zero_()
        return slot

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Take pages for the entries' tokens and upload the step's metadata."""
        cache = self.cache
        starts = reserve_entries(cache, entries, self.admit)
        q_lens = [len(e.tokens) for e in entries]
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        slots = [cache.slot(e.request) for e in entries]
        n_tokens, n_seqs = sum(q_lens), len(entries)
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(starts, q_lens)])
        seq_of_token = np.repeat(np.arange(n_seqs, dtype=np.int32), q_lens)
        cu_q = np.zeros(n_seqs + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu_q[1:])
        rows = [int(cu_q[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
        width = max(1, -(-max(kv_lens) // cache.page_size))
        tables = [cache.table_rows(g, slots, width).reshape(-1) for g in range(len(cache.groups))]
        parts = [tokens, positions, seq_of_token, cu_q, np.asarray(kv_lens, dtype=np.int32),
                 np.asarray(slots, dtype=np.int32), np.asarray(rows, dtype=np.int32)] + tables
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += _round_up(max(p.size, 1), 4)
        host = np.zeros(total, dtype=np.int32)
        for o, p in zip(offsets, parts):
            host[o:o + p.size] = p
        dev = self._upload(host)

        def view(i):
            return dev[offsets[i]:offsets[i] + parts[i].size]

        return StepContext(
            n_tokens=n_tokens, n_seqs=n_seqs, n_logit_rows=len(rows), tokens=view(0),
            positions=view(1), seq_of_token=view(2), cu_q=view(3), kv_len=view(4), slots=view(5),
            logit_rows=view(6),
            block_tables=[view(7 + g).view(n_seqs, width) for g in range(len(cache.groups))],
            host_q_lens=q_lens, host_kv_lens=kv_lens, host_slots=slots, max_q_len=max(q_lens),
            max_kv_len=max(kv_lens))

    # ---- the step -------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns FP32 logits [number of wanted places, vocab] on the device,
        ordered by entry and then by ``want``."""
        self._validate(entries)
        ctx = self.build_context(entries)
        logits = self.model.forward(ctx, self.caches)
        for e in entries:
            self.cache.release_passed(e.request)
        return logits

    def end(self, request) -> None:
        """The request is finished: give back its pages and its slot."""
        self.cache.free(request)
