from .engine import Engine
from .runner import BadToken, ContextFull, ModelRunner, StepError, StepItem, TooManyRows
from .scheduler import Request, ScheduledItem, Scheduler

__all__ = ["Engine", "BadToken", "ContextFull", "ModelRunner", "StepError", "StepItem", "TooManyRows",
           "Request", "ScheduledItem", "Scheduler"]
