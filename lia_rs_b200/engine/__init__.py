from .engine import Engine
from .step import StepContext, StepEntry, StepError, StepRuntime

__all__ = ["Engine", "StepContext", "StepEntry", "StepError", "StepRuntime"]
