from .batch import GroupMeta, StepContext, StepEntry, build_context
from .step import StepError, StepFunction

__all__ = ["GroupMeta", "StepContext", "StepEntry", "build_context", "StepError", "StepFunction"]
