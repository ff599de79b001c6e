from .engine import Engine
from .step import StepContext, StepEntry, StepError

__all__ = ["Engine", "StepContext", "StepEntry", "StepError"]
