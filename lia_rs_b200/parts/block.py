"""Arrangements of a layer's parts.

`prenorm`: r = h + s * mixer(norm1(h)); h' = r + s * ffn(norm2(r))
(src/inference/llama_fusion.rs:41-117; s is MiniCPM's scale_depth / sqrt(layers), 1 for plain
Llama).  Checkpoint names: input_layernorm, self_attn, post_attention_layernorm, mlp
(src/inference/huggingface/minicpm5.rs:31-68); a layer spec may override them."""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, Arrangement, DeferredNorm, PartSpec, lookup,
                   register_arrangement)


@dataclass(frozen=True)
class LayerSpec:
    """`norm` is the norm at every place of the arrangement; `norms` names other norms for single places
    (for the pre-norm arrangement the places are "norm1" and "norm2")."""
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    arrangement: str = "prenorm"
    residual_scale: float = 1.0
    norms: dict = field(default_factory=dict, hash=False, compare=False)
    names: dict = field(default_factory=lambda: {"norm1": "input_layernorm.", "mixer": "self_attn.",
                                                 "norm2": "post_attention_layernorm.", "feed_forward": "mlp."},
                        hash=False, compare=False)

    def norm_at(self, place: str) -> PartSpec:
        return self.norms.get(place, self.norm)


@register_arrangement("prenorm")
class PreNormBlock(Arrangement):
    supports_rows = True

    @staticmethod
    def _classes(spec: LayerSpec):
        norm1, norm2 = spec.norm_at("norm1"), spec.norm_at("norm2")
        return ((lookup(NORMS, norm1.kind, "norm"), norm1.params), (lookup(MIXERS, spec.mixer.kind, "mixer"), spec.mixer.params),
                (lookup(NORMS, norm2.kind, "norm"), norm2.params),
                (lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward"), spec.feed_forward.params))

    @staticmethod
    def check(spec: LayerSpec) -> None:
        for cls, params in PreNormBlock._classes(spec):
            cls.check_params(params)

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str) -> list:
        n = spec.names
        places = (n["norm1"], n["mixer"], n["norm2"], n["feed_forward"])
        return [t for (cls, params), place in zip(PreNormBlock._classes(spec), places)
                for t in cls.tensor_specs(params, prefix + place)]

    def __init__(self, spec: LayerSpec, tensors: dict, prefix: str, runtime):
        n = spec.names
        self.runtime = runtime
        self.scale = float(spec.residual_scale)
        places = (n["norm1"], n["mixer"], n["norm2"], n["feed_forward"])
        self.norm1, self.mixer, self.norm2, self.feed_forward = (
            cls(params, tensors, prefix + place, runtime) for (cls, params), place in zip(self._classes(spec), places))
        self.graph_safe = all(part.graph_safe for part in (self.norm1, self.mixer, self.norm2, self.feed_forward))

    def graph_key(self, ctx) -> tuple:
        return (self.norm1.graph_key(ctx) + self.mixer.graph_key(ctx) + self.norm2.graph_key(ctx) +
                self.feed_forward.graph_key(ctx))

    def _normed(self, ctx, norm, part, source):
        """The input of `part`: `norm(source)`, left to the part's first product where the part can take that."""
        deferred = DeferredNorm(ctx, norm, source)
        return deferred if part.takes_deferred_norm else deferred.tensor()

    def forward(self, ctx, residual, kv=None, state=None, rows=None, n_rows=None):
        x = self._normed(ctx, self.norm1, self.mixer, residual)
        if rows is None:
            self.mixer.forward(ctx, x, residual, self.scale, kv=kv, state=state)
            self.feed_forward.forward(ctx, self._normed(ctx, self.norm2, self.feed_forward, residual), residual, self.scale)
            return None
        # Only `rows` matter after this layer (the reference prunes the last layer the same way:
        # src/inference/llama_fusion.rs:45-60): the mixer brings the cache up to date for every token; the output
        # projection, the second norm, the feed-forward and both residual sums run on the picked rows alone.
        picked = ctx.buffer("block.picked", (n_rows, residual.shape[1]), residual.dtype)
        if n_rows and self.mixer.supports_rows:
            self.runtime.ops.gather_rows(residual, rows, picked)
        if self.mixer.supports_rows:
            self.mixer.forward(ctx, x, picked, self.scale, kv=kv, state=state, rows=rows, n_rows=n_rows)
        else:
            self.mixer.forward(ctx, x, residual, self.scale, kv=kv, state=state)
            if n_rows:
                self.runtime.ops.gather_rows(residual, rows, picked)
        if n_rows:
            self.feed_forward.forward(ctx, self._normed(ctx, self.norm2, self.feed_forward, picked), picked, self.scale)
        return picked


def build_layer(spec: LayerSpec, tensors: dict, prefix: str, runtime):
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement")(spec, tensors, prefix, runtime)


def check_layer(spec: LayerSpec) -> None:
    """Raise ValueError if a part of the layer refuses its parameters (no device needed)."""
    arrangement = lookup(ARRANGEMENTS, spec.arrangement, "arrangement")
    if hasattr(arrangement, "check"):
        arrangement.check(spec)


def layer_tensor_specs(spec: LayerSpec, prefix: str) -> list:
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement").tensor_specs(spec, prefix)
