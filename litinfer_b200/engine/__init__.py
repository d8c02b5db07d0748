from .batch import GroupView, StepContext, StepItem, context_from, pack_step
from .engine import Engine, EngineConfig
from .scheduler import Request, RequestRefused, ScheduledItem, Scheduler, SchedulerConfig
from .step import ModelRunner

__all__ = [
    "Engine",
    "EngineConfig",
    "GroupView",
    "ModelRunner",
    "Request",
    "RequestRefused",
    "ScheduledItem",
    "Scheduler",
    "SchedulerConfig",
    "StepContext",
    "StepItem",
    "context_from",
    "pack_step",
]
