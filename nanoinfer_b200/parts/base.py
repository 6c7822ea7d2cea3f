"""Contracts of the parts a model is assembled from.

No part knows which model it is in: it receives its own spec (sizes and constants),
its weights by slot name, and the runtime (device, compute dtype, kernels).

Every part class has
    weight_slots(spec, hidden_size) -> {slot: WeightSlot}      (static; no GPU needed)
    __init__(self, spec, hidden_size, weights: {slot: tensor}, rt: Runtime)

Norm            forward(h, delta, rows=None) -> x
                    h: fp32 residual stream [T, d], updated in place to h + delta when
                    delta is given; x = norm(h) in the compute dtype.  ``rows`` (int32
                    device tensor [R]) restricts the output to those rows of h.
PositionEncoding  owns the constants a mixer needs to encode positions (for rotary:
                    inverse frequencies, rotary_dim, pairing); table() returns them.
Mixer           cache_need() -> PagedKVNeed | PagedNeed | StateNeed | None
                forward(x, ctx: StepContext, cache: CacheView | None) -> y [T, d]
                    x: normed activations [T, d] in the compute dtype.  Must only use
                    ctx (positions, segments, block tables, state slots) to find what
                    belongs to which request; must give the same result for a token
                    however the step was cut.
FeedForward     forward(x, ctx) -> y [T, d]
                A mixer or feed-forward with the class attribute ``adds_into_residual = True``
                is called with ``residual=h`` as well and may add its output into h itself
                and return None (a fused epilogue).

Embedding       forward(tokens, h) -> None
                    tokens int32 [T] on the device; fills the FP32 residual stream h [T, d].
                    ``table`` (optional attribute): its [vocab, d] matrix on the device, which a
                    tied head is handed as its "weight".
Head            forward(h, delta, norm, ctx) -> FP32 logits [ctx.n_logit_rows, vocab]
                    for rows ctx.logit_rows of h (+ delta, still pending); ``norm`` is the model's
                    final norm.  Its spec says ``tied``; then weight_slots is empty.

Two optional hooks, on mixers, feed-forwards, embeddings and heads alike:

plan_step       a static method plan_step(q_lens, starts) -> StepPlan.  Called once per step and
                per class that defines it, on the host, with every entry's number of tokens and
                cached length before the step.  It returns what the part's kernels need to find
                their work (tile lists, token lists, counts): int32 arrays, which the runner
                uploads with the step's other metadata in the same pinned copy and hands to the
                part as device tensors (``ctx.plan_of(self)``), and host integers.  The arrays'
                sizes may depend on ``q_lens`` only (a captured step is replayed with other
                ``starts``).  The step function itself knows nothing about tilings.
graph_safe      "none" (default), "decode" or "all": whether the part's forward may be captured
                into a CUDA graph and replayed for other steps of the same shape - that is, whether
                it finds everything that changes from step to step (tokens, positions, slots, block
                tables, plans) in device memory through ctx, and decides nothing on the host from
                ctx's host_* fields.  "decode": only for steps in which every request brings one
                token.  The runner runs every step's kernels exactly once (the pass that precedes a
                capture IS that step), so a part with state of its own may be graph-safe too.
Arrangement     (a block) forward(h, delta, ctx, caches) -> delta'
                    runs its norms, mixer and feed-forward; returns the addition that
                    is still pending on the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class WeightSlot:
    """Shape and initialisation rule of one weight of a part.

    init "normal": N(0, std) in random-weights mode; "ones": 1.0 (norm gains).
    """
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token, in pages; ``window`` = how many most recent
    tokens stay reachable (None = all)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class PagedNeed:
    """Paged per-token storage of any layout: ``planes`` names each tensor a token has a row in
    and that row's shape, e.g. (("latent", (96,)),) for one compressed vector per token, or keys
    and values of different widths.  The page tensor of a plane with row shape (a, ..., z) is
    [pages, a, ..., page_size, z].  ``window`` as in PagedKVNeed."""
    planes: Tuple[Tuple[str, Tuple[int, ...]], ...]
    window: Optional[int] = None


def planes_of(need) -> Tuple[Tuple[str, Tuple[int, ...]], ...]:
    """The planes of a paged need: keys and values [Hkv, hd] each for a PagedKVNeed."""
    if isinstance(need, PagedKVNeed):
        row = (need.num_kv_heads, need.head_dim)
        return (("k", row), ("v", row))
    return tuple((name, tuple(shape)) for name, shape in need.planes)


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request: ``shape`` elements of ``dtype`` ("float32" or
    the string "compute"), zeroed when a request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class StepPlan:
    """What a part's plan_step returns: int32 arrays for the device and integers for the host."""
    arrays: Dict[str, "object"] = field(default_factory=dict)
    scalars: Dict[str, int] = field(default_factory=dict)


class Part:
    """Base of all parts; subclasses override what their category needs."""

    graph_safe = "none"

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        return {}

    def weights_in_order(self) -> tuple:
        """The part's large weight matrices on the device, in the order its kernels read them
        (what the parts before it may ask into L2 ahead of time); () if it has none."""
        return ()

    def __init__(self, spec, hidden_size: int, weights: Dict[str, "object"], rt) -> None:
        self.spec = spec
        self.hidden_size = hidden_size
        self.rt = rt
