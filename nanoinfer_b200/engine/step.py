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

import gc
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, GroupSpec, OutOfPages
from ..config.model_config import ModelConfig
from ..parts.base import PagedKVNeed, PagedNeed, StateNeed, StepPlan, planes_of
from .model import DecoderModel
from .request import PENDING_TOKEN
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
    """What a mixer sees of the cache for one layer run: the page tensors of its planes by name
    (``k_pages`` / ``v_pages`` are the planes "k" and "v"), or its state tensor."""
    group: int = -1
    pages: Dict[str, torch.Tensor] = field(default_factory=dict)
    state: Optional[torch.Tensor] = None
    writable: bool = True

    @property
    def k_pages(self) -> Optional[torch.Tensor]:
        return self.pages.get("k")

    @property
    def v_pages(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")


@dataclass
class DevicePlan:
    """A part's StepPlan after the upload: its arrays as int32 device tensors, its integers."""
    arrays: Dict[str, torch.Tensor]
    scalars: Dict[str, int]


@dataclass
class StepContext:
    """Device-side description of a step, shared by all layers.

    tokens, positions, seq_of_token: int32 [T];  cu_q: int32 [B+1] token offsets per
    request;  kv_len: int32 [B] cached length after this step;  slots: int32 [B] state slot
    per request;  logit_rows: int32 [R];  block_tables[g]: int32 [B, W] of group g.
    The host_* fields hold the same numbers for decisions made on the host (empty in a step
    that is replayed from a graph).  decode_only: every request brings exactly one token.
    plans: what the parts' own plan_step hooks returned for this step, by the class that defines
    the hook; a part reads its own with plan_of(self).
    read_after: the weight matrices that will be read after the part that is running, in order
    (set by the model and the arrangement as they go); a part whose kernels leave the memory system
    room may ask the head of them into L2 (``Runtime.warm``).
    norm_after: the norm part that reads the residual stream after the running block, if it can come
    prepared by the kernel that last adds into the stream (``ops.NormHandoff``); else None.
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
    decode_only: bool = False
    plans: Dict[type, DevicePlan] = field(default_factory=dict)
    read_after: tuple = ()
    norm_after: object = None

    def plan_of(self, part) -> DevicePlan:
        owner = plan_owner(type(part))
        if owner is None or owner not in self.plans:
            raise StepError(f"{type(part).__name__} has no plan in this step (no plan_step hook, or the "
                            f"context was built without it)")
        return self.plans[owner]


def plan_owner(cls) -> Optional[type]:
    """The class in ``cls``'s ancestry that defines plan_step (one plan per such class and step)."""
    for c in cls.__mro__:
        if "plan_step" in c.__dict__:
            return c
    return None


def upload_plans(parts, q_lens: Sequence[int], starts: Sequence[int], device) -> Dict[type, DevicePlan]:
    """The plans of the given parts for one step, each array copied to the device on its own (for
    contexts built by hand; the runner packs them into its single metadata copy instead)."""
    out: Dict[type, DevicePlan] = {}
    for part in parts:
        owner = plan_owner(type(part))
        if owner is not None and owner not in out:
            plan = owner.plan_step(list(q_lens), list(starts))
            out[owner] = DevicePlan({k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.int32)).to(device)
                                     for k, v in plan.arrays.items()}, dict(plan.scalars))
    return out


def reserve_entries(cache: CacheManager, entries: Sequence[StepEntry], admit) -> List[int]:
    """Take slots and pages for every entry of a step, all or nothing.

    Every group's pool and the slot count are checked before anything is taken, so a step
    that does not fit raises OutOfPages (or StepError) and leaves the cache unchanged.
    ``admit(request)`` is called for requests the cache does not know yet.  Returns each
    entry's start position (its cached length before this step).
    """
    if all(len(e.tokens) == 1 and cache.has(e.request) for e in entries):
        # the decode loop: at most one new page per request, the same in every group
        n_new_pages = sum(1 for e in entries if cache.needs_page_for_one(e.request))
        for g in range(len(cache.groups)):
            if n_new_pages > cache.num_free_pages(g):
                raise OutOfPages(f"group {g}: the step needs {n_new_pages} more pages, "
                                 f"{cache.num_free_pages(g)} are free")
        starts = [cache.length(e.request) for e in entries]
        for e in entries:
            cache.append_one(e.request)
        return starts
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
                 page_size: int = 16, num_pages=1024, max_requests: int = 8,
                 max_tokens_per_request: Optional[int] = None, max_portion_tokens: Optional[int] = None,
                 device: str = "cuda:0", fused_decode: bool = False, beyond_model_limit: bool = False) -> None:
        """``num_pages``: pages of every cache group's pool, or one count per group (in the order
        the groups first appear in the schedule).  With one count, a windowed group gets no more
        pages than its requests can ever hold at once, if ``max_portion_tokens`` (the most tokens
        a request brings in one step) is given: max_requests * (window + portion) tokens.
        ``fused_decode``: run steps of up to 8 single tokens as one persistent kernel
        (csrc/decode_fused.cu) where the model is a plain stack of attention + SwiGLU blocks.  Off by
        default: measured slower than the chain of per-part kernels (1.68 ms against 0.86 ms per
        step at batch 8 of the 1B sizes; five grid barriers per layer are what it cannot hide).
        ``beyond_model_limit``: let a request grow past the model's max_position_embeddings, up to
        ``max_tokens_per_request`` (for replaying given tokens: positions are computed, not looked up,
        so nothing breaks there; serving keeps the model's limit)."""
        from .runtime import parse_dtype
        self.config = config
        self.rt = Runtime(device=torch.device(device), dtype=parse_dtype(dtype), page_size=page_size,
                          fused_decode=fused_decode)
        # compile (in parallel) and load what this precision needs before the first step
        from ..kernels import ops
        common = ["elementwise", "rope_kv", "attention_generic"]
        ops.preload(common + (["gemm_f32"] if self.rt.dtype == torch.float32 else
                              ["gemv_bf16", "gemv_ksplit", "gemm_tc", "gemm_tc2", "gemm_swap_tc", "attention_prefill", "attention_prefill_tc", "attention_decode"]
                              + (["decode_fused"] if fused_decode else [])))
        self.model = DecoderModel(config, weights, self.rt)

        # cache groups: one per distinct need among the runs that own a cache
        needs = self.model.cache_needs()
        group_keys: List[tuple] = []
        group_specs: List[GroupSpec] = []
        self.caches: List[Optional[CacheView]] = [None] * len(needs)
        self._state_runs: List[int] = []
        for r, need in enumerate(needs):
            if isinstance(need, (PagedKVNeed, PagedNeed)):
                key = (planes_of(need), need.window)
                if key not in group_keys:
                    group_keys.append(key)
                    kv = isinstance(need, PagedKVNeed)
                    group_specs.append(GroupSpec(need.num_kv_heads if kv else 0, need.head_dim if kv else 0, need.window))
                self.caches[r] = CacheView(group=group_keys.index(key))
            elif isinstance(need, StateNeed):
                self.caches[r] = CacheView()
                self._state_runs.append(r)
            elif need is not None:
                raise StepError(f"run {r}: unknown cache need {need!r}")
        if not group_specs:
            group_specs.append(GroupSpec(0, 0, None))  # bookkeeping of lengths only
        pages_per_group = self._pages_per_group(num_pages, group_specs, page_size, max_requests, max_portion_tokens)
        if max_tokens_per_request is None:
            full = [n for n, g in zip(pages_per_group, group_specs) if g.window is None] or pages_per_group
            max_tokens_per_request = min(config.max_position_embeddings, min(full) * page_size)
        self.max_tokens_per_request = max_tokens_per_request if beyond_model_limit else \
            min(max_tokens_per_request, config.max_position_embeddings)
        self.cache = CacheManager(group_specs, pages_per_group, page_size, max_requests, self.max_tokens_per_request)
        rt = self.rt
        for r, need in enumerate(needs):
            view = self.caches[r]
            if isinstance(need, (PagedKVNeed, PagedNeed)):
                n_pages = pages_per_group[view.group]
                for name, row in planes_of(need):
                    shape = (n_pages,) + tuple(row[:-1]) + (page_size, row[-1])
                    view.pages[name] = torch.zeros(shape, dtype=rt.dtype, device=rt.device)
            elif isinstance(need, StateNeed):
                dt = rt.dtype if need.dtype == "compute" else getattr(torch, need.dtype)
                view.state = torch.zeros((max_requests,) + tuple(need.shape), dtype=dt, device=rt.device)
        for r, run in enumerate(config.schedule):
            if run.cache_of is not None:
                src = self.caches[run.cache_of]
                self.caches[r] = CacheView(group=src.group, pages=src.pages, state=src.state, writable=False)
        # hooks of the parts: who plans its own work per step, and what may be captured into a graph
        parts = [p for b in self.model.blocks for p in (getattr(b, "mixer", None), getattr(b, "feed_forward", None))
                 if p is not None] + [self.model.embedding, self.model.head]
        self.planners: List[type] = []
        for part in parts:
            owner = plan_owner(type(part))
            if owner is not None and owner not in self.planners:
                self.planners.append(owner)
        safety = {getattr(p, "graph_safe", "none") for p in parts}
        self.decode_graphs_ok = safety <= {"decode", "all"}
        self.portion_graphs_ok = safety <= {"all"}
        self.error_word = ops.error_word(self.rt.device)   # non-zero once a kernel gave up a bounded wait
        self.use_graphs = True
        self.h2d_bytes = 0            # bytes of step metadata copied to the device so far
        self.max_graph_batch = 256
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._portion_graphs: Dict[tuple, "_PortionGraph"] = {}       # by step shape, least recently used first
        self._portion_seen: Dict[tuple, int] = {}
        self.max_portion_graphs = 8
        # A captured shape gives its place to a new one only after it has not come for this many steps:
        # with more recurring shapes than places, taking turns would capture every step anew (a serving
        # workload with 20 prompt-step shapes per round, repeated: 50 ms of capture for each 11 ms step).
        self.portion_graph_idle = 512
        self._step_no = 0
        # A capture costs about three runs of the step (an eager run that sizes the workspaces, the
        # capture, the first replay) and a replay saves only the launch overhead, so a shape must
        # have come back a few times before it is worth one.
        self.portion_graph_after = 4
        # The same holds for a batch size of single tokens, though a replay saves more there (the
        # step is short): a size is captured when it comes for the third time.  Sizes that pass
        # once or twice (a batch that shrinks as its requests end) run without a graph.
        self.decode_graph_after = 3
        self._decode_seen: Dict[int, int] = {}
        self._pinned: List[torch.Tensor] = []
        self._pinned_events: List[torch.cuda.Event] = []
        self._pinned_next = 0
        self._dev_meta: Optional[torch.Tensor] = None

    @staticmethod
    def _pages_per_group(num_pages, group_specs, page_size, max_requests, max_portion_tokens) -> List[int]:
        if not isinstance(num_pages, int):
            counts = [int(n) for n in num_pages]
            if len(counts) != len(group_specs):
                raise StepError(f"{len(counts)} page counts for {len(group_specs)} cache groups")
            return counts
        counts = []
        for g in group_specs:
            n = num_pages
            if g.window is not None and max_portion_tokens is not None:
                # a request holds its window, the portion being appended, and two partly used pages
                per_request = -(-(g.window + max_portion_tokens) // page_size) + 2
                n = min(n, max_requests * per_request)
            counts.append(n)
        return counts

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
        self.h2d_bytes += host.nbytes
        self._pinned[i][:n].numpy()[:] = host
        self._dev_meta[:n].copy_(self._pinned[i][:n], non_blocking=True)
        self._pinned_events[i].record()
        self._pinned_used[i] = True
        return self._dev_meta

    def _validate(self, entries: Sequence[StepEntry], pending_ok: bool = False) -> None:
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
            if n == 1:
                t = e.tokens[0]
                if not 0 <= t < vocab and not (pending_ok and t == PENDING_TOKEN):
                    raise StepError(f"request {e.request!r}: token id {t} is outside [0, {vocab})")
            elif min(e.tokens) < 0 or max(e.tokens) >= vocab:
                bad = next(t for t in e.tokens if not 0 <= t < vocab)
                raise StepError(f"request {e.request!r}: token id {bad} is outside [0, {vocab})")
            for w in e.want:
                if not 0 <= w < n:
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

    N_FIXED = 7      # tokens, positions, request of each token, row offsets, kv lengths, slots, logit rows

    def _layout(self, entries: Sequence[StepEntry], starts: Sequence[int], full_width: bool):
        """The step's metadata as host arrays, in the order they lie in one buffer: tokens,
        positions, request of each token, row offsets, kv lengths, slots, logit rows, block tables
        per group, then the arrays of the parts' own plans.  ``full_width``: tables at the cache's
        full width (what a captured graph needs) instead of the width this step uses."""
        cache = self.cache
        q_lens = [len(e.tokens) for e in entries]
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        slots = [cache.slot(e.request) for e in entries]
        n_seqs = len(entries)
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(starts, q_lens)])
        seq_of_token = np.repeat(np.arange(n_seqs, dtype=np.int32), q_lens)
        cu_q = np.zeros(n_seqs + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu_q[1:])
        rows = [int(cu_q[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
        width = cache.table_width if full_width else max(1, -(-max(kv_lens) // cache.page_size))
        tables = [cache.table_rows(g, slots, width).reshape(-1) for g in range(len(cache.groups))]
        plans = [owner.plan_step(q_lens, list(starts)) for owner in self.planners]
        parts = [tokens, positions, seq_of_token, cu_q, np.asarray(kv_lens, dtype=np.int32),
                 np.asarray(slots, dtype=np.int32), np.asarray(rows, dtype=np.int32)] + tables
        for plan in plans:
            parts += [np.asarray(a, dtype=np.int32) for a in plan.arrays.values()]
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += _round_up(max(p.size, 1), 4)
        return parts, offsets, total, q_lens, kv_lens, slots, width, plans

    def _context(self, dev: torch.Tensor, parts, offsets, q_lens, kv_lens, slots, width, max_kv_len, plans) -> StepContext:
        """Views of the uploaded buffer ``dev`` as a StepContext."""
        n_seqs, n_groups = len(q_lens), len(self.cache.groups)

        def view(i):
            return dev[offsets[i]:offsets[i] + parts[i].size]

        at = self.N_FIXED + n_groups
        device_plans: Dict[type, DevicePlan] = {}
        for owner, plan in zip(self.planners, plans):
            arrays = {}
            for name in plan.arrays:
                arrays[name] = view(at)
                at += 1
            device_plans[owner] = DevicePlan(arrays, dict(plan.scalars))
        return StepContext(
            n_tokens=sum(q_lens), n_seqs=n_seqs, n_logit_rows=parts[6].size, tokens=view(0),
            positions=view(1), seq_of_token=view(2), cu_q=view(3), kv_len=view(4), slots=view(5),
            logit_rows=view(6),
            block_tables=[view(self.N_FIXED + g).view(n_seqs, width) for g in range(n_groups)],
            host_q_lens=q_lens, host_kv_lens=kv_lens, host_slots=slots, max_q_len=max(q_lens),
            max_kv_len=max_kv_len, decode_only=all(q == 1 for q in q_lens), plans=device_plans)

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Take pages for the entries' tokens and upload the step's metadata."""
        starts = reserve_entries(self.cache, entries, self.admit)
        parts, offsets, total, q_lens, kv_lens, slots, width, plans = self._layout(entries, starts, full_width=False)
        host = np.zeros(total, dtype=np.int32)
        for o, p in zip(offsets, parts):
            host[o:o + p.size] = p
        dev = self._upload(host)
        return self._context(dev, parts, offsets, q_lens, kv_lens, slots, width, max(kv_lens), plans)

    # ---- the step -------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch; returns FP32 logits [number of wanted places, vocab] on the device,
        ordered by entry and then by ``want``.  The tensor is valid until the next step.
        ``device_tokens`` (int32 on the device, one per entry): the tokens of a step of single
        tokens that the host has not read yet (entries then carry PENDING_TOKEN)."""
        self._validate(entries, pending_ok=device_tokens is not None)
        self._step_no += 1
        if device_tokens is not None and not (self._graphable(entries) and device_tokens.numel() == len(entries)):
            raise StepError("tokens can be fed from the device only to a replayed step of single tokens")
        if self._graphable(entries) and (device_tokens is not None or self._decode_graph_due(len(entries), count=True)):
            starts = reserve_entries(self.cache, entries, self.admit)
            logits = self._decode_graph(len(entries)).run(entries, starts, device_tokens)
        elif self._portion_graphable(entries):
            starts = reserve_entries(self.cache, entries, self.admit)
            logits = self._portion_graph(entries).run(entries, starts)
        else:
            ctx = self.build_context(entries)
            logits = self.model.forward(ctx, self.caches)
        for e in entries:
            self.cache.release_passed(e.request)
        return logits

    # ---- decode steps as CUDA graphs ------------------------------------------------------
    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        """A step of single tokens that all want their logits can be captured once per batch size
        and replayed, if every mixer and feed-forward of the model says that its forward finds
        what changes between steps in device memory (graph_safe)."""
        return (self.use_graphs and self.decode_graphs_ok and len(entries) <= self.max_graph_batch
                and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    # ---- steps with prompt portions as CUDA graphs -------------------------------------------
    def _portion_graphable(self, entries: Sequence[StepEntry]) -> bool:
        """A step's launches depend only on how many tokens each entry brings and how many logit
        rows it wants (everything else is metadata in device memory), so a shape that comes back -
        the same portion size step after step while a prompt is cut into portions - is captured at
        its ``portion_graph_after``-th appearance and replayed from then on."""
        if not self.use_graphs or not self.portion_graphs_ok or self.rt.dtype != torch.bfloat16:
            return False
        sig = tuple((len(e.tokens), len(e.want)) for e in entries)
        if sig in self._portion_graphs:
            return True
        seen = self._portion_seen.get(sig, 0) + 1
        self._portion_seen[sig] = seen
        if len(self._portion_seen) > 4096:
            self._portion_seen.clear()
        if seen < self.portion_graph_after:
            return False
        if len(self._portion_graphs) >= self.max_portion_graphs:
            oldest = next(iter(self._portion_graphs.values()))                # least recently used
            if self._step_no - oldest.last_used < self.portion_graph_idle:
                return False                                                  # every place is in use: this shape runs without a graph
        return True

    def _portion_graph(self, entries: Sequence[StepEntry]) -> "_PortionGraph":
        sig = tuple((len(e.tokens), len(e.want)) for e in entries)
        g = self._portion_graphs.pop(sig, None)
        if g is None:
            if len(self._portion_graphs) >= self.max_portion_graphs:       # drop the least recently used
                self._portion_graphs.pop(next(iter(self._portion_graphs)))
            g = _PortionGraph(self)
        self._portion_graphs[sig] = g                                      # most recently used last
        return g

    def _decode_graph_due(self, n: int, count: bool) -> bool:
        """True if a step of ``n`` single tokens runs as a graph: the size has a graph already, or
        comes for the ``decode_graph_after``-th time.  ``count``: this call is such a step."""
        if n in self._graphs:
            return True
        seen = self._decode_seen.get(n, 0) + 1
        if count:
            self._decode_seen[n] = seen
        return seen >= self.decode_graph_after

    def can_feed_device_tokens(self, n: int) -> bool:
        """True if the next step of ``n`` single tokens can take its tokens from a device tensor
        (it then runs as a replayed graph, whose token buffer they are copied into)."""
        return (self.use_graphs and self.decode_graphs_ok and 0 < n <= self.max_graph_batch
                and self._decode_graph_due(n, count=False))

    def _decode_graph(self, n: int) -> "_DecodeGraph":
        g = self._graphs.get(n)
        if g is None:
            g = self._graphs[n] = _DecodeGraph(self, n)
        return g

    def greedy_decode_on_device(self, requests: Sequence[object], last_tokens: Sequence[int],
                                n_steps: int) -> torch.Tensor:
        """Decode ``n_steps`` greedy tokens for each request without touching the host between
        steps: arg-max, token feedback and position advance are part of the replayed graph.
        ``last_tokens[i]`` is the token of request i that has not been run yet.  Pages for all
        steps are taken up front.  Returns int32 [n_steps, len(requests)] on the device; the
        token that the last step samples is returned but not yet run."""
        if not self.decode_graphs_ok:
            raise StepError("device-side decoding needs a model whose parts can be captured into a graph")
        for r in requests:
            self.cache.append(r, n_steps)
        n = len(requests)
        g = self._decode_graph(n)
        starts = [self.cache.length(r) - n_steps for r in requests]
        entries = [StepEntry(r, [int(t)], [0]) for r, t in zip(requests, last_tokens)]
        return g.run_greedy(entries, starts, n_steps)

    def end(self, request) -> None:
        """The request is finished: give back its pages and its slot."""
        self.cache.free(request)


from ..kernels import ops  # noqa: E402  (after the classes above: no import cycle)


class _quiet_collector:
    """Stream capture must not be disturbed by the garbage collector: if it frees an older CUDA
    graph (or anything else whose release is a CUDA call) while a stream is capturing, the capture
    is invalidated.  Collect first, then keep the collector off until the capture has ended."""

    def __enter__(self):
        gc.collect()
        self.was_enabled = gc.isenabled()
        gc.disable()

    def __exit__(self, *exc):
        if self.was_enabled:
            gc.enable()
        return False


class _PortionGraph:
    """The forward pass of one step shape (tokens and wanted rows per entry), captured once and
    replayed: metadata in a static device buffer refreshed by one copy from pinned memory, block
    tables at their full width, split counts chosen for the longest request the cache allows."""

    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.host = self.host_np = self.dev = None
        self.copied = torch.cuda.Event()
        self.copy_pending = False
        self.last_used = runner._step_no

    def run(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> torch.Tensor:
        runner = self.runner
        self.last_used = runner._step_no
        parts, offsets, total, q_lens, kv_lens, slots, width, plans = runner._layout(entries, starts, full_width=True)
        if self.host is None:
            self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
            self.host_np = self.host.numpy()
            self.dev = torch.zeros(total, dtype=torch.int32, device=runner.rt.device)
        if self.copy_pending:
            self.copied.synchronize()
        for o, p in zip(offsets, parts):
            self.host_np[o:o + p.size] = p
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record(ops.current_stream_object())
        self.copy_pending = True
        runner.h2d_bytes += total * 4
        if self.graph is None:
            ctx = runner._context(self.dev, parts, offsets, q_lens, kv_lens, slots, width,
                                  runner.max_tokens_per_request, plans)
            ctx.host_q_lens, ctx.host_kv_lens, ctx.host_slots = [], [], []     # a replay has no host numbers
            # This step runs eagerly (which also loads what is missing and sizes the workspaces);
            # the same launches are then captured for the steps to come.  Every step's kernels run once.
            logits = runner.model.forward(ctx, runner.caches)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with _quiet_collector(), torch.cuda.graph(self.graph):
                self.logits = runner.model.forward(ctx, runner.caches)
            return logits
        self.graph.replay()
        return self.logits


class _DecodeGraph:
    """The forward pass of ``n`` single-token requests, captured once and replayed.

    All metadata lives in one static device buffer at fixed offsets (block tables at their
    full width), refreshed by one copy from pinned host memory before each replay; grids do
    not depend on context lengths.  A second capture adds arg-max, token feedback and the
    advance of positions, for decoding without the host in the loop.
    """

    def __init__(self, runner: ModelRunner, n: int) -> None:
        self.runner, self.n = runner, n
        cache = runner.cache
        self.width = cache.table_width
        n_groups = len(cache.groups)
        # the parts' plans for n single tokens: sizes are fixed by the step's shape, contents are
        # refreshed with the positions (a plan may order its work by cached length)
        plans = [owner.plan_step([1] * n, [0] * n) for owner in runner.planners]
        self.plan_sizes = [[np.asarray(a).size for a in plan.arrays.values()] for plan in plans]
        flat_plan_sizes = [sz for ps in self.plan_sizes for sz in ps]
        # what changes every step comes first (one small copy): tokens, positions, request of each
        # token, row offsets, kv lengths, plan arrays; then slots, logit rows and the block tables
        names = ["tokens", "positions", "seq_of_token", "cu_q", "kv_len"] + [f"plan{i}" for i in range(len(flat_plan_sizes))] + \
                ["slots", "logit_rows"] + [f"table{g}" for g in range(n_groups)]
        sizes = [n, n, n, n + 1, n] + flat_plan_sizes + [n, n] + [n * self.width] * n_groups
        self.off, total = {}, 0
        for name, sz in zip(names, sizes):
            self.off[name] = total
            total += _round_up(max(sz, 1), 4)
        self.small = self.off["slots"]
        dev = runner.rt.device
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.copied = torch.cuda.Event()
        self.copy_pending = False
        self.last_ids: Optional[list] = None     # requests and table version of the last full refresh
        self.last_version = -1
        o = self.off
        self.host_np[o["seq_of_token"]:o["seq_of_token"] + n] = np.arange(n)
        self.host_np[o["cu_q"]:o["cu_q"] + n + 1] = np.arange(n + 1)
        self.host_np[o["logit_rows"]:o["logit_rows"] + n] = np.arange(n)            # all rows are wanted

        def view(name, sz):
            return self.dev[o[name]:o[name] + sz]

        at = 0
        device_plans: Dict[type, DevicePlan] = {}
        for owner, plan in zip(runner.planners, plans):
            arrays = {}
            for name, a in plan.arrays.items():
                arrays[name] = view(f"plan{at}", np.asarray(a).size)
                at += 1
            device_plans[owner] = DevicePlan(arrays, dict(plan.scalars))
        self.has_plan_arrays = any(sz > 0 for sz in flat_plan_sizes)
        self.ctx = StepContext(
            n_tokens=n, n_seqs=n, n_logit_rows=n, tokens=view("tokens", n), positions=view("positions", n),
            seq_of_token=view("seq_of_token", n), cu_q=view("cu_q", n + 1), kv_len=view("kv_len", n),
            slots=view("slots", n), logit_rows=view("logit_rows", n),
            block_tables=[view(f"table{g}", n * self.width).view(n, self.width) for g in range(n_groups)],
            max_q_len=1, max_kv_len=runner.max_tokens_per_request, decode_only=True, plans=device_plans)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.greedy_graph: Optional[torch.cuda.CUDAGraph] = None
        self.greedy_out: Optional[torch.Tensor] = None
        self.greedy_launches = 0

    def _fill(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> None:
        """Refresh the step's metadata on the device: tokens, positions and lengths every step
        (one small copy); slots and block tables only when a request joined or left or a page
        was taken since the last fill (a second copy)."""
        n, o, cache = self.n, self.off, self.runner.cache
        if self.copy_pending:
            self.copied.synchronize()
        h = self.host_np
        h[o["tokens"]:o["tokens"] + n] = [e.tokens[0] for e in entries]
        h[o["positions"]:o["positions"] + n] = starts
        h[o["kv_len"]:o["kv_len"] + n] = h[o["positions"]:o["positions"] + n] + 1
        if self.has_plan_arrays:          # the parts' plans may depend on the cached lengths
            at = 0
            for owner, sizes in zip(self.runner.planners, self.plan_sizes):
                plan = owner.plan_step([1] * n, list(starts))
                for a, sz in zip(plan.arrays.values(), sizes):
                    a = np.asarray(a, dtype=np.int32)
                    if a.size != sz:
                        raise StepError(f"{owner.__name__}.plan_step: the size of an array changed with the positions")
                    h[o[f"plan{at}"]:o[f"plan{at}"] + sz] = a
                    at += 1
        ids = [e.request for e in entries]
        small = self.small
        if ids != self.last_ids or cache.table_version != self.last_version:
            slots = [cache.slot(r) for r in ids]
            h[o["slots"]:o["slots"] + n] = slots
            for g in range(len(cache.groups)):
                h[o[f"table{g}"]:o[f"table{g}"] + n * self.width] = cache.table_rows(g, slots).reshape(-1)
            self.last_ids, self.last_version = ids, cache.table_version
            self.dev.copy_(self.host, non_blocking=True)
            self.runner.h2d_bytes += self.host.numel() * 4
        else:
            self.dev[:small].copy_(self.host[:small], non_blocking=True)
            self.runner.h2d_bytes += small * 4
        self.copied.record(ops.current_stream_object())
        self.copy_pending = True

    def _capture(self) -> torch.Tensor:
        """Runs this step eagerly (which also compiles and loads what is missing and sizes the
        workspaces) and captures the same launches for the steps to come; returns this step's
        logits.  Every step's kernels run exactly once, so a part that updates state of its own
        is not run twice for the step that is captured."""
        runner = self.runner
        logits = runner.model.forward(self.ctx, runner.caches)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with _quiet_collector(), torch.cuda.graph(self.graph):
            self.logits = runner.model.forward(self.ctx, runner.caches)
        return logits

    def run(self, entries: Sequence[StepEntry], starts: Sequence[int],
            device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        self._fill(entries, starts)
        if device_tokens is not None:
            self.ctx.tokens.copy_(device_tokens)      # after the host's copy, before the replay
        if self.graph is None:
            return self._capture()
        self.graph.replay()
        return self.logits

    def run_greedy(self, entries: Sequence[StepEntry], starts: Sequence[int], n_steps: int) -> torch.Tensor:
        runner, ctx = self.runner, self.ctx
        self._fill(entries, starts)
        out = torch.empty(n_steps, self.n, dtype=torch.int32, device=runner.rt.device)
        first = 0
        if self.greedy_graph is None:
            # the first step runs eagerly, feedback included; the graph is captured for the others
            self.greedy_out = torch.zeros(self.n, dtype=torch.int32, device=runner.rt.device)
            ops.argmax(runner.model.forward(ctx, runner.caches), self.greedy_out)
            ctx.tokens.copy_(self.greedy_out)
            ctx.positions.add_(1)
            ctx.kv_len.add_(1)
            out[0].copy_(self.greedy_out)
            first = 1
            torch.cuda.synchronize()
            self.greedy_graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with _quiet_collector(), torch.cuda.graph(self.greedy_graph):
                logits = runner.model.forward(ctx, runner.caches)
                ops.argmax(logits, self.greedy_out)
                ctx.tokens.copy_(self.greedy_out)
                ctx.positions.add_(1)
                ctx.kv_len.add_(1)
            self.greedy_launches = ops.launch_count() - before   # this package's kernels per step
        for i in range(first, n_steps):
            self.greedy_graph.replay()
            out[i].copy_(self.greedy_out)
        return out
