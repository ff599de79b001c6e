from .engine import Engine
from .step import StepContext, StepEntry, StepError, StepRuntime
from .trace import TraceRunner, replay

__all__ = ["Engine", "StepContext", "StepEntry", "StepError", "StepRuntime", "TraceRunner", "replay"]
