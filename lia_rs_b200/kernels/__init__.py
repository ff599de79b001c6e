from . import build, ops
from .ops import KernelError

__all__ = ["build", "ops", "KernelError"]
