"""Dense SwiGLU feed-forward: act = up * gate / (1 + exp(-gate)), f = act Wd^T, no biases
(src/inference/moe.rs:31-61, src/gpu/kernels/basic.rs:150-157).  Gate and up are one product
against [Wg; Wu] whose epilogue applies the activation (the reference's gated kernel does the
same with two matrices: src/gpu/kernels/llama_gated.rs:181-222); the down product adds into the
residual stream.  Parameters: hidden, intermediate."""
from __future__ import annotations

import torch

from ..weights import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import ACCUM, SWIGLU, linear, prepare_weight


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # rows in, rows out: only the number of tokens matters
    takes_deferred_norm = True

    @staticmethod
    def tensor_specs(params, prefix):
        h, i = params["hidden"], params["intermediate"]
        return [TensorSpec(prefix + "gate_proj.weight", (i, h)),
                TensorSpec(prefix + "up_proj.weight", (i, h)),
                TensorSpec(prefix + "down_proj.weight", (h, i))]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.w_gate_up = prepare_weight(torch.cat([tensors[prefix + "gate_proj.weight"],
                                                   tensors[prefix + "up_proj.weight"]], dim=0), runtime)
        self.w_down = prepare_weight(tensors[prefix + "down_proj.weight"], runtime)

    def forward(self, ctx, x, residual, scale):
        rt, n = self.runtime, x.shape[0]
        act = ctx.buffer("ffn.act", (n, self.intermediate), rt.compute_dtype)
        linear(rt, SWIGLU, x, self.w_gate_up, act, error_flag=ctx.error_flag, name="gate_up")
        linear(rt, ACCUM, act, self.w_down, residual, scale, error_flag=ctx.error_flag, name="down")
