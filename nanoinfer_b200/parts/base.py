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
Mixer           cache_need() -> PagedKVNeed | StateNeed | None
                forward(x, ctx: StepContext, cache: CacheView | None) -> y [T, d]
                    x: normed activations [T, d] in the compute dtype.  Must only use
                    ctx (positions, segments, block tables, state slots) to find what
                    belongs to which request; must give the same result for a token
                    however the step was cut.
FeedForward     forward(x, ctx) -> y [T, d]
                A mixer or feed-forward with the class attribute ``adds_into_residual = True``
                is called with ``residual=h`` as well and may add its output into h itself
                and return None (a fused epilogue).
Arrangement     (a block) forward(h, delta, ctx, caches) -> delta'
                    runs its norms, mixer and feed-forward; returns the addition that
                    is still pending on the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass
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
class StateNeed:
    """A fixed-size state per request: ``shape`` elements of ``dtype`` ("float32" or
    the string "compute"), zeroed when a request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Base of all parts; subclasses override what their category needs."""

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        return {}

    def __init__(self, spec, hidden_size: int, weights: Dict[str, "object"], rt) -> None:
        self.spec = spec
        self.hidden_size = hidden_size
        self.rt = rt
