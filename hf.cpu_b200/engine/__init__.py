from . import measure
from .step import Engine, GroupMeta, StepContext, StepEntry, Workspace
from .scheduler import FinishEvent, Request, RequestError, Scheduler, StepPlan, TokenEvent

__all__ = ["measure", "Engine", "StepEntry", "StepContext", "GroupMeta", "Workspace", "Scheduler", "Request", "RequestError",
           "TokenEvent", "FinishEvent", "StepPlan"]
