"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, the weight used as stored
(src/gpu/kernels/normalization.rs:46-112).  Parameters: hidden, eps."""
from __future__ import annotations

from ..weights import TensorSpec
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # rows in, rows out: only the number of tokens matters

    @staticmethod
    def tensor_specs(params, prefix):
        return [TensorSpec(prefix + "weight", (params["hidden"],), kind="norm")]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.weight = tensors[prefix + "weight"]     # bfloat16 or, if stored so, float32

    def forward(self, ctx, x, out, rows_index=None, out_scale=1.0):
        self.runtime.ops.rmsnorm(x, self.weight, out, self.eps, out_scale, rows_index)

    def rms_record(self):
        return self.weight, self.eps
