from .context import StepContext, Workspace
from .llm_engine import LLMEngine, RequestOutput
from .runner import ModelRunner, StepItem
from .scheduler import Request, ScheduledItem, Scheduler, SchedulerOutput

__all__ = ["StepContext", "Workspace", "LLMEngine", "RequestOutput", "ModelRunner", "StepItem", "Request", "ScheduledItem",
           "Scheduler", "SchedulerOutput"]
