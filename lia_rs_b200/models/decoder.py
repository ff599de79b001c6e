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

from ..parts import NORMS, PartSpec, build_layer, layer_tensor_specs, lookup, MIXERS
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


class DecodeStack:
    """The persistent decode kernel (csrc/decode_stack.cu) over the whole schedule, when every layer is a
    pre-norm arrangement of RMSNorm, grouped-query attention (rotary or no position encoding) and SwiGLU
    with the same sizes, scale and eps, in bfloat16.  It is built from the layers' `stack_record`s, so it
    knows parts by their kind, never an architecture.  `plan(ctx)` says whether a step can use it."""

    def __init__(self, model):
        self.model = model
        self.records = None
        self.layers_device = None
        self.tables = None
        self.timeline = None          # int64 [layers, 16] on the device: set it to have CTA 0 write its phase times
        self.usable = self._collect()

    def _collect(self) -> bool:
        model = self.model
        if model.runtime.compute_dtype != torch.bfloat16 or not model.spec.schedule:
            return False
        records = []
        for entry in model.spec.schedule:
            record = model.layers[entry.layer].stack_record()
            if (record is None or entry.cache is None or record["kind"] != "prenorm"
                    or record["norm1"]["kind"] != "rmsnorm" or record["norm2"]["kind"] != "rmsnorm"
                    or record["mixer"]["kind"] != "gqa_attention" or record["feed_forward"]["kind"] != "swiglu"):
                return False
            records.append(record)
        if model.spec.state_requests():
            return False
        first = records[0]
        mixer, ffn = first["mixer"], first["feed_forward"]

        def same(a, b):
            return a is b or (a is not None and b is not None and torch.equal(a, b))

        for r in records:
            m = r["mixer"]
            if (r["residual_scale"] != first["residual_scale"] or r["norm1"]["eps"] != first["norm1"]["eps"]
                    or r["norm2"]["eps"] != first["norm1"]["eps"]
                    or any(m[k] != mixer[k] for k in ("heads", "kv_heads", "head_dim", "rotary_dim", "attn_scale"))
                    or not same(m["inv_freq"], mixer["inv_freq"])
                    or r["feed_forward"]["intermediate"] != ffn["intermediate"]
                    or r["norm1"]["weight"].dtype != first["norm1"]["weight"].dtype
                    or r["norm2"]["weight"].dtype != first["norm1"]["weight"].dtype):
                return False
        self.records = records
        return True

    def splits(self, ctx, runtime_step) -> int:
        """Ranges of keys per token: the (token, kv head, range) items fill the CTAs once; no range is
        shorter than 256 keys at the step's context bucket."""
        mixer = self.records[0]["mixer"]
        items = max(1, ctx.n_tokens * mixer["kv_heads"])
        return max(1, min(runtime_step.sm_count // items, 32, ctx.context_bucket // 256))

    def plan(self, ctx, runtime_step):
        """The number of key ranges if this step can run through the kernel, else None."""
        if not (self.usable and ctx.decode_only) or len(self.records) > 64:      # the kernel keeps 64 layer records
            return None
        mixer, ffn = self.records[0]["mixer"], self.records[0]["feed_forward"]
        n_splits = self.splits(ctx, runtime_step)
        ops = self.model.runtime.ops
        if not ops.decode_stack_accepts(ctx.n_tokens, self.model.spec.hidden_size, mixer["heads"], mixer["kv_heads"],
                                        mixer["head_dim"], ffn["intermediate"], mixer["rotary_dim"], n_splits):
            return None
        return n_splits

    def _layer_array(self, ctx):
        views = [ctx.kv_view(entry.cache, entry.writes) for entry in self.model.spec.schedule]
        key = tuple((v.k_pages.data_ptr(), v.block_table.data_ptr(), v.writes) for v in views)
        if self.tables != key:
            rows = []
            for record, view in zip(self.records, views):
                rows.append(dict(norm1=record["norm1"]["weight"], norm2=record["norm2"]["weight"],
                                 wqkv=record["mixer"]["wqkv"], wo=record["mixer"]["wo"],
                                 wgu=record["feed_forward"]["wgu"], wd=record["feed_forward"]["wd"],
                                 k_pages=view.k_pages, v_pages=view.v_pages, block_table=view.block_table,
                                 window=record["mixer"]["window"], writes=view.writes))
            self.layers_device = self.model.runtime.ops.decode_stack_layers(rows, self.model.runtime.device)
            self.tables = key
        return self.layers_device

    def forward(self, ctx, h, n_splits):
        rt, spec = self.model.runtime, self.model.spec
        first = self.records[0]
        mixer, ffn = first["mixer"], first["feed_forward"]
        nq, nkv, d = mixer["heads"], mixer["kv_heads"], mixer["head_dim"]
        n = ctx.n_tokens
        step = ctx.runtime
        qkv = ctx.buffer("stack.qkv", (n, (nq + 2 * nkv) * d), torch.float32)
        attn = ctx.buffer("stack.attn", (n, nq * d), torch.bfloat16)
        act = ctx.buffer("stack.act", (n, ffn["intermediate"]), torch.bfloat16)
        partial = step.scratch("stack.partial", n * nq * n_splits * (d + 1), torch.float32)
        counters = step.counters(n * nkv)
        rt.ops.decode_stack(self._layer_array(ctx), len(self.records), h, qkv, attn, act, partial, counters,
                            ctx.positions, ctx.slots, step.stack_barrier(), nq, nkv, d, ffn["intermediate"],
                            mixer["rotary_dim"], mixer["inv_freq"], first["norm1"]["eps"], first["residual_scale"],
                            mixer["attn_scale"], n_splits, step.sm_count, ctx.error_flag, self.timeline)


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
        # decode steps may be captured in CUDA graphs only if every part launches the same way each step
        self.graph_safe = all(layer.graph_safe for layer in self.layers) and bool(self.final_norm.graph_safe)
        self.decode_stack = DecodeStack(self)       # the layers as one persistent kernel, for decode steps it accepts
        self.use_decode_stack = True
        self.stack_steps = 0                        # steps that went through it

    def forward(self, ctx) -> torch.Tensor:
        """Run the step described by `ctx`; returns 32-bit logits [ctx.n_out, vocab] (device)."""
        rt, spec = self.runtime, self.spec
        n = ctx.n_tokens
        h = ctx.buffer("model.h", (n, spec.hidden_size), torch.float32)
        rt.ops.embedding(ctx.tokens, self.embedding, h, spec.embedding_scale, ctx.error_flag)
        n_splits = self.decode_stack.plan(ctx, ctx.runtime) if self.use_decode_stack else None
        if n_splits is not None:
            self.decode_stack.forward(ctx, h, n_splits)
            self.stack_steps += 1
        else:
            for position, entry in enumerate(spec.schedule):
                kv = ctx.kv_view(entry.cache, entry.writes) if entry.cache is not None else None
                self.layers[entry.layer].forward(ctx, h, kv=kv, state=ctx.state(position))
        if ctx.n_out == 0:
            return ctx.logits_buffer(0, spec.vocab_size)
        y = ctx.buffer("model.y", (ctx.n_out, spec.hidden_size), rt.compute_dtype)
        self.final_norm.forward(ctx, h, y, rows_index=ctx.out_rows)
        logits = ctx.logits_buffer(ctx.n_out, spec.vocab_size)
        linear(rt, STORE, y, self.head, logits, spec.logit_scale)
        return logits
