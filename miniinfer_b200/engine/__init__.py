from .context import StepContext, Workspace
from .runner import ModelRunner, StepItem

__all__ = ["StepContext", "Workspace", "ModelRunner", "StepItem"]
