from .step import ModelRunner, StepContext, StepEntry, StepError
from .scheduler import Event, PlanItem, Request, Scheduler
from .engine import Engine

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepError", "Event", "PlanItem", "Request",
           "Scheduler", "Engine"]
