"""lia_rs_b200: a small, whole inference engine for one B200, for the MiniCPM5 Llama
architecture of Heltion/lia.rs: configuration and registry, safetensors weights, layers built
from parts, a paged cache manager, one step function, a scheduler, sampling, a command line and
`generate()`; every forward operation is a hand-written sm_100a CUDA kernel."""
from . import models as _models  # noqa: F401  (registers the built-in architecture)
from .config import ConfigError, LlamaConfig, register_architecture, resolve_architecture
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "register_architecture", "resolve_architecture", "WeightError",
           "write_random_model", "Engine", "StepEntry", "generate", "replay", "Sampling"]


def __getattr__(name):
    if name in ("Engine", "StepEntry", "StepError", "replay"):
        from . import engine
        return getattr(engine, name)
    if name in ("generate", "Generator"):
        from .engine import generate as _g
        return getattr(_g, name)
    if name in ("Sampling",):
        from . import sampling
        return getattr(sampling, name)
    raise AttributeError(name)
