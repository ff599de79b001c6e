"""Interfaces of the parts a decoder layer is put together from, and one registry per kind.

A layer is an *arrangement* (how norms, mixer, feed-forward and the residual stream are wired)
of four kinds of parts:

  mixer              moves information between positions (attention here); may own a cache
                     (keys and values in pages) and/or per-request state of fixed size
  feed-forward       acts on each position alone (dense SwiGLU here; experts elsewhere)
  norm               normalises rows of the residual stream
  position encoding  how positions enter the mixer (rotary here)

Every part is built from a `PartSpec` (its kind and its parameters: all sizes and constants)
and from the tensors it declared.  No part knows which model it is in: the model builder
(`models/`) chooses the parts layer by layer from the configuration.

The residual stream is always a 32-bit tensor [tokens, hidden].  Mixers and feed-forwards obey
one contract: `forward(ctx, x, residual, scale, ...)` ADDS `scale * f(x)` into `residual`
in place, where x is the normalised input in the compute element type.  This lets a part fuse
the residual sum into its last kernel, and lets a toy part do `residual.add_(y, alpha=scale)`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class KVCacheRequest:
    """What a mixer needs from the paged cache: `kv_heads` x `head_dim` keys and values per
    token, all of them (`window` None) or the last `window` of them."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-request state of fixed size: one tensor of `shape` and `dtype` per live request,
    zeroed when the request is admitted."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Runtime:
    """Device and compute element type of one engine; parts launch kernels through `ops`."""

    def __init__(self, device, compute_dtype: torch.dtype):
        from ..kernels import ops
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("compute element type must be float32 or bfloat16")
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.ops = ops


class Part:
    """Base of all parts.  `tensor_specs` declares the checkpoint tensors (names relative to
    `prefix`); `__init__` receives them already on the device, in their storage element type.

    `graph_safe`: the part's `forward` launches the same kernels with the same arguments in every step
    whose entries have the same numbers of tokens, with the same number of wanted rows and the same
    `ctx.context_bucket`; whatever else differs between such steps (token ids, positions, the portions'
    starts, slots, pages) it reads on the device, from `ctx.tokens`, `ctx.positions`, `ctx.slots`,
    `ctx.prefill_segments` and the block tables, never on the host.  Only when every part of a model says
    so are its steps captured in CUDA graphs and replayed; a part that looks at the starts in
    `ctx.segments` in Python, or allocates, leaves this False and the model runs launch by launch.

    Rows of nobody: a step of many single tokens may bring `ctx.padding` extra rows at its end (token 0, position 0,
    slot -1 in `ctx.slots`), counted in `ctx.n_tokens`, `ctx.n_out` and `ctx.decode_rows` but not listed in
    `ctx.segments`.  A part's kernels run them like any row, except that nothing is read from or written to a
    cache or a state for a negative slot; what they compute is dropped."""

    graph_safe = False

    def graph_key(self, ctx) -> tuple:
        """What else of a step's shape this part's launches depend on, beyond the step's number of tokens, of
        wanted rows, of single-token entries and of portions, and its context bucket: two steps that agree in all
        of these replay one captured graph.  The answer that is always right is the number of tokens of every
        entry, which is the default; a part whose launches do not look at them answers () (a part that cuts
        portions into tiles answers with its number of tiles)."""
        return tuple(count for _, _, count, _ in ctx.segments)

    @staticmethod
    def tensor_specs(params: dict, prefix: str) -> list:
        return []

    def __init__(self, params: dict, tensors: dict, prefix: str, runtime: Runtime):
        self.params = params
        self.runtime = runtime

    @staticmethod
    def check_params(params: dict) -> None:
        """Raise ValueError for parameters this part (or the kernels behind it) cannot take.  Called when a
        model's description is put together, before any tensor is read and without a device, so that an
        unsupported size is refused with its reason at the earliest place."""


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, rows_index=None, out_scale: float = 1.0):
        """out[r] = norm(x[rows_index[r]] or x[r]) * out_scale; x 32-bit, out compute type."""
        raise NotImplementedError

    def rms_record(self):
        """`(weight, eps)` if this norm is exactly y = x / sqrt(mean(x^2) + eps) * weight (a product kernel
        can then norm its input rows itself, see `DeferredNorm`), else None."""
        return None


class DeferredNorm:
    """A normalised input that has not been computed yet: `norm` applied to the 32-bit rows `source`.  An
    arrangement hands it, in place of the tensor, to a mixer or feed-forward that says `takes_deferred_norm`;
    such a part gives it to `parts.linear.linear` as the product's input, which either lets the product's
    kernel norm the rows as it reads them (a norm with an `rms_record`, few tokens) or calls `tensor()`.
    `tensor()` runs the norm's own kernel once and returns the rows in the compute element type."""

    def __init__(self, ctx, norm: Norm, source: torch.Tensor, buffer_name: str = "block.x"):
        self.ctx, self.norm, self.source, self.buffer_name = ctx, norm, source, buffer_name
        self.shape = source.shape
        self._tensor = None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            out = self.ctx.buffer(self.buffer_name, tuple(self.source.shape), self.norm.runtime.compute_dtype)
            self.norm.forward(self.ctx, self.source, out)
            self._tensor = out
        return self._tensor


class PositionEncoding(Part):
    """Owned by a mixer.  Encodes q and k in place of the mixer and appends k, v to the cache."""

    def encode_and_store(self, ctx, qkv: torch.Tensor, q_out: torch.Tensor, kv, nq: int, nkv: int, d: int):
        raise NotImplementedError

    def rotate_half(self):
        """`(rotary_dim, inv_freq)` if this encoding is exactly "rotate-half over the first rotary_dim elements
        of every q and k head by angle position * inv_freq[i]" (rotary_dim 0, inv_freq None: nothing is
        encoded), else None.  The decode attention kernel can apply such an encoding itself, together with
        the append to the cache; every other encoding (interleaved pairs, sections, learned tables) answers
        None and runs its own `encode_and_store` ahead of the attention kernel, at every step."""
        return None


class Mixer(Part):
    # True: `forward` takes `rows` / `n_rows` (only those tokens' outputs are needed, `residual` holds those rows
    # alone; cache and state are still updated for every token).  False: the arrangement runs the mixer for every
    # token and picks the rows afterwards.
    supports_rows = False
    # True: `x` may be a `DeferredNorm` (the part only ever gives it to `linear`, or calls its `tensor()`).
    takes_deferred_norm = False

    @staticmethod
    def cache_request(params: dict) -> Optional[KVCacheRequest]:
        return None

    @staticmethod
    def state_request(params: dict) -> Optional[StateRequest]:
        return None

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, scale: float, kv=None, state=None):
        """residual += scale * mixer(x).  `kv` is the layer's `cache.KVView` (or None), `state`
        the tensor [slots, *shape] of its per-request state (or None)."""
        raise NotImplementedError


class FeedForward(Part):
    takes_deferred_norm = False      # as for Mixer

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, scale: float):
        """residual += scale * feed_forward(x)."""
        raise NotImplementedError


class Arrangement:
    """How one layer wires its parts around the residual stream.  `graph_safe` as for `Part`: true
    when all its parts are."""

    graph_safe = False

    def graph_key(self, ctx) -> tuple:
        """As `Part.graph_key`, for the layer: what its parts answer, put together.  The default is the answer that
        is always right."""
        return tuple(count for _, _, count, _ in ctx.segments)

    @staticmethod
    def tensor_specs(layer_spec, prefix: str) -> list:
        raise NotImplementedError

    def __init__(self, layer_spec, tensors: dict, prefix: str, runtime: Runtime):
        raise NotImplementedError

    # True: `forward` takes `rows` / `n_rows` and then returns the residual rows of those tokens alone.
    supports_rows = False

    def forward(self, ctx, residual: torch.Tensor, kv=None, state=None, rows=None, n_rows=None):
        """Run the layer on the residual stream in place.  With `rows` (device int32 batch indices, `n_rows` of
        them; only an arrangement that says `supports_rows` is given them) nothing after this layer needs the
        other tokens: the layer still brings cache and state up to date for every token, but may compute the
        rest for these rows only, and returns their residual rows [n_rows, hidden] in the order of `rows`.
        Without `rows` it returns None."""
        raise NotImplementedError


MIXERS: dict = {}
FEED_FORWARDS: dict = {}
NORMS: dict = {}
POSITION_ENCODINGS: dict = {}
ARRANGEMENTS: dict = {}


def _register(table: dict, kind: str):
    def decorate(cls):
        table[kind] = cls
        cls.kind = kind
        return cls
    return decorate


def register_mixer(kind: str):
    return _register(MIXERS, kind)


def register_feed_forward(kind: str):
    return _register(FEED_FORWARDS, kind)


def register_norm(kind: str):
    return _register(NORMS, kind)


def register_position_encoding(kind: str):
    return _register(POSITION_ENCODINGS, kind)


def register_arrangement(kind: str):
    return _register(ARRANGEMENTS, kind)


def lookup(table: dict, kind: str, what: str):
    if kind not in table:
        raise KeyError(f"unknown {what} {kind!r}; registered: {sorted(table)}")
    return table[kind]
