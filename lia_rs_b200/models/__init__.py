from .decoder import DecoderModel, ModelSpec, ScheduleEntry
from . import minicpm5_llama  # noqa: F401  (registers the architecture)

__all__ = ["DecoderModel", "ModelSpec", "ScheduleEntry"]
