"""Parts a model is assembled from; importing this package registers the built-in kinds."""
from . import block, embedding, feed_forward, head, mixer, norm, position  # noqa: F401
from .base import PagedKVNeed, PagedNeed, Part, StateNeed, StepPlan, WeightSlot

__all__ = ["PagedKVNeed", "PagedNeed", "Part", "StateNeed", "StepPlan", "WeightSlot"]
