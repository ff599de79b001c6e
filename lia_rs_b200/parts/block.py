"""Arrangements of a layer's parts.

`prenorm`: r = h + s * mixer(norm1(h)); h' = r + s * ffn(norm2(r))
(src/inference/llama_fusion.rs:41-117; s is MiniCPM's scale_depth / sqrt(layers), 1 for plain
Llama).  Checkpoint names: input_layernorm, self_attn, post_attention_layernorm, mlp
(src/inference/huggingface/minicpm5.rs:31-68); a layer spec may override them."""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, Arrangement, PartSpec, lookup,
                   register_arrangement)


@dataclass(frozen=True)
class LayerSpec:
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    arrangement: str = "prenorm"
    residual_scale: float = 1.0
    names: dict = field(default_factory=lambda: {"norm1": "input_layernorm.", "mixer": "self_attn.",
                                                 "norm2": "post_attention_layernorm.", "feed_forward": "mlp."},
                        hash=False, compare=False)


@register_arrangement("prenorm")
class PreNormBlock(Arrangement):
    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str) -> list:
        n = spec.names
        return (lookup(NORMS, spec.norm.kind, "norm").tensor_specs(spec.norm.params, prefix + n["norm1"])
                + lookup(MIXERS, spec.mixer.kind, "mixer").tensor_specs(spec.mixer.params, prefix + n["mixer"])
                + lookup(NORMS, spec.norm.kind, "norm").tensor_specs(spec.norm.params, prefix + n["norm2"])
                + lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward").tensor_specs(
                    spec.feed_forward.params, prefix + n["feed_forward"]))

    def __init__(self, spec: LayerSpec, tensors: dict, prefix: str, runtime):
        n = spec.names
        self.runtime = runtime
        self.scale = float(spec.residual_scale)
        self.norm1 = lookup(NORMS, spec.norm.kind, "norm")(spec.norm.params, tensors, prefix + n["norm1"], runtime)
        self.mixer = lookup(MIXERS, spec.mixer.kind, "mixer")(spec.mixer.params, tensors, prefix + n["mixer"], runtime)
        self.norm2 = lookup(NORMS, spec.norm.kind, "norm")(spec.norm.params, tensors, prefix + n["norm2"], runtime)
        self.feed_forward = lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward")(
            spec.feed_forward.params, tensors, prefix + n["feed_forward"], runtime)
        self.graph_safe = all(part.graph_safe for part in (self.norm1, self.mixer, self.norm2, self.feed_forward))

    def stack_record(self):
        parts = [self.norm1.stack_record(), self.mixer.stack_record(), self.norm2.stack_record(),
                 self.feed_forward.stack_record()]
        if any(part is None for part in parts):
            return None
        return dict(kind="prenorm", norm1=parts[0], mixer=parts[1], norm2=parts[2], feed_forward=parts[3],
                    residual_scale=self.scale)

    def forward(self, ctx, residual, kv=None, state=None):
        x = ctx.buffer("block.x", tuple(residual.shape), self.runtime.compute_dtype)
        self.norm1.forward(ctx, residual, x)
        self.mixer.forward(ctx, x, residual, self.scale, kv=kv, state=state)
        self.norm2.forward(ctx, residual, x)
        self.feed_forward.forward(ctx, x, residual, self.scale)


def build_layer(spec: LayerSpec, tensors: dict, prefix: str, runtime):
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement")(spec, tensors, prefix, runtime)


def layer_tensor_specs(spec: LayerSpec, prefix: str) -> list:
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement").tensor_specs(spec, prefix)
