from .engine import Engine, EngineConfig, StepOutput
from .request import InferenceRequest, RequestState
from .scheduler import ScheduledBatch, Scheduler, SchedulerStats
from .step import CacheView, ModelRunner, StepContext, StepEntry, StepError, reserve_entries

__all__ = ["Engine", "EngineConfig", "StepOutput", "InferenceRequest", "RequestState",
           "ScheduledBatch", "Scheduler", "SchedulerStats", "CacheView", "ModelRunner",
           "StepContext", "StepEntry", "StepError", "reserve_entries"]
