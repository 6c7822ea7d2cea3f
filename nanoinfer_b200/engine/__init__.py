from .step import CacheView, ModelRunner, StepContext, StepEntry, StepError

__all__ = ["CacheView", "ModelRunner", "StepContext", "StepEntry", "StepError"]
