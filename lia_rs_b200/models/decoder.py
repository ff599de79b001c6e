"""A decoder as data: an embedding, a list of layers, the ORDER in which layers run, a final
norm and an output head.  The model builder of an architecture fills a `ModelSpec` from its
configuration; `DecoderModel` builds the parts and runs a step.  Nothing here knows an
architecture's name.

The order is a list of `ScheduleEntry`: which layer runs, which cache it uses and whether it
appends to it.  The default is each layer once with a cache of its own; a list may name a layer
twice (with a second cache) or let a layer read a cache that an earlier entry wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parts import NORMS, PartSpec, build_layer, check_layer, layer_tensor_specs, lookup, MIXERS
from ..parts.linear import STORE, linear, prepare_weight
from ..weights import TensorSpec


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache: Optional[int] = None     # id of the cache this entry uses (None: the mixer has none)
    writes: bool = True             # False: read a cache that another entry fills


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: list
    final_norm: PartSpec
    schedule: list = field(default_factory=list)
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    embedding_name: str = "model.embed_tokens.weight"
    head_name: Optional[str] = "lm_head.weight"     # None: tied to the embedding table
    layer_prefix: str = "model.layers.{}."
    final_norm_prefix: str = "model.norm."
    eos_token_ids: tuple = ()

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [
                ScheduleEntry(i, i if self._mixer(i).cache_request(self.layers[i].mixer.params) else None)
                for i in range(len(self.layers))]
        for entry in self.schedule:
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.layers)}")
        for layer in self.layers:
            check_layer(layer)                      # a size that a part or its kernels cannot take is refused here
        requests = {}
        writers = set()
        for entry in self.schedule:
            request = self._mixer(entry.layer).cache_request(self.layers[entry.layer].mixer.params)
            if (request is None) != (entry.cache is None):
                raise ValueError(f"schedule entry {entry}: the mixer's cache need and the entry disagree")
            if entry.cache is None:
                continue
            if requests.setdefault(entry.cache, request) != request:
                raise ValueError(f"cache {entry.cache} is shared by layers with different needs")
            if entry.writes:
                if entry.cache in writers:
                    raise ValueError(f"cache {entry.cache} is written by two schedule entries")
                writers.add(entry.cache)
            elif entry.cache not in writers:
                raise ValueError(f"cache {entry.cache} is read before any entry writes it")

    def _mixer(self, layer: int):
        return lookup(MIXERS, self.layers[layer].mixer.kind, "mixer")

    def tensor_specs(self) -> list:
        specs = [TensorSpec(self.embedding_name, (self.vocab_size, self.hidden_size))]
        for i, layer in enumerate(self.layers):
            specs += layer_tensor_specs(layer, self.layer_prefix.format(i))
        specs += lookup(NORMS, self.final_norm.kind, "norm").tensor_specs(self.final_norm.params,
                                                                           self.final_norm_prefix)
        if self.head_name is not None:
            specs.append(TensorSpec(self.head_name, (self.vocab_size, self.hidden_size)))
        return specs

    def cache_requests(self) -> dict:
        """cache id -> KVCacheRequest."""
        out = {}
        for entry in self.schedule:
            if entry.cache is not None:
                out[entry.cache] = self._mixer(entry.layer).cache_request(self.layers[entry.layer].mixer.params)
        return out

    def state_requests(self) -> dict:
        """schedule position -> StateRequest, for mixers that keep per-request state."""
        out = {}
        for position, entry in enumerate(self.schedule):
            request = self._mixer(entry.layer).state_request(self.layers[entry.layer].mixer.params)
            if request is not None:
                out[position] = request
        return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: dict, runtime):
        self.spec, self.runtime = spec, runtime
        device = runtime.device

        def on_device(names):
            return {n: tensors[n].to(device) for n in names}

        table = tensors[spec.embedding_name].to(device)
        self.embedding = prepare_weight(table, runtime)
        self.layers = []
        for i, layer in enumerate(spec.layers):
            prefix = spec.layer_prefix.format(i)
            names = [s.name for s in layer_tensor_specs(layer, prefix)]
            self.layers.append(build_layer(layer, on_device(names), prefix, runtime))
        norm_cls = lookup(NORMS, spec.final_norm.kind, "norm")
        names = [s.name for s in norm_cls.tensor_specs(spec.final_norm.params, spec.final_norm_prefix)]
        self.final_norm = norm_cls(spec.final_norm.params, on_device(names), spec.final_norm_prefix, runtime)
        if spec.head_name is None:
            self.head = self.embedding
        else:
            self.head = prepare_weight(tensors[spec.head_name].to(device), runtime)
        # layers of one description launch alike: one of each answers for all when a step's graph key is made
        distinct = {}
        for layer_spec, layer in zip(spec.layers, self.layers):
            distinct.setdefault(repr(layer_spec), layer)
        self._key_layers = list(distinct.values()) + [self.final_norm]
        # decode steps may be captured in CUDA graphs only if every part launches the same way each step
        self.graph_safe = all(layer.graph_safe for layer in self.layers) and bool(self.final_norm.graph_safe)

    def graph_key(self, ctx) -> tuple:
        """What a captured step is good for: the step's numbers of tokens, of wanted rows, of single-token entries
        and of portions, its context bucket, and whatever else of its shape the parts say their launches depend on
        (each distinct answer once)."""
        seen, extra = set(), []
        for layer in self._key_layers:
            key = layer.graph_key(ctx)
            if key and key not in seen:
                seen.add(key)
                extra.append(key)
        return (ctx.n_tokens, ctx.n_out, ctx.context_bucket, ctx.n_single, ctx.n_prefill_segments, tuple(extra))

    def forward(self, ctx) -> torch.Tensor:
        """Run the step described by `ctx`; returns 32-bit logits [ctx.n_out, vocab] (device).  When fewer rows
        are wanted than the step brings, the last entry of the schedule is told which (an arrangement that can
        then computes only what those rows need and hands back their residual rows; the reference's pruning of
        the last layer, src/inference/llama_fusion.rs:45-60, src/gpu/kernels/llama.rs:185-198)."""
        rt, spec = self.runtime, self.spec
        n = ctx.n_tokens
        h = ctx.buffer("model.h", (n, spec.hidden_size), torch.float32)
        rt.ops.embedding(ctx.tokens, self.embedding, h, spec.embedding_scale, ctx.error_flag)
        picked = None
        last = len(spec.schedule) - 1
        for position, entry in enumerate(spec.schedule):
            kv = ctx.kv_view(entry.cache, entry.writes) if entry.cache is not None else None
            layer = self.layers[entry.layer]
            if position == last and ctx.n_out < n and getattr(layer, "supports_rows", False):
                picked = layer.forward(ctx, h, kv=kv, state=ctx.state(position), rows=ctx.out_rows, n_rows=ctx.n_out)
            else:
                layer.forward(ctx, h, kv=kv, state=ctx.state(position))
        if ctx.n_out == 0:
            return ctx.logits_buffer(0, spec.vocab_size)
        y = ctx.buffer("model.y", (ctx.n_out, spec.hidden_size), rt.compute_dtype)
        if picked is not None:
            self.final_norm.forward(ctx, picked, y)
        else:
            self.final_norm.forward(ctx, h, y, rows_index=ctx.out_rows)
        logits = ctx.logits_buffer(ctx.n_out, spec.vocab_size)
        linear(rt, STORE, y, self.head, logits, spec.logit_scale, error_flag=ctx.error_flag, name="head")
        return logits
