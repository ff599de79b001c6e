"""Grouped-query attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T without biases (src/inference/llama.rs:92-112), computed as
one product with the concatenated matrix [Wq; Wk; Wv] (src/inference/llama_weights.rs:100-135);
position encoding of q and k and append of k, v to the pages; q-head h attends through kv-head
h div (heads/kv_heads) to the keys j <= position of its own request, scores scaled by
1/sqrt(head_dim), softmax in 32-bit (src/gpu/kernels/llama.rs:62-159); output projection
(src/inference/llama.rs:290-298) added into the residual stream.

Parameters: hidden, heads, kv_heads, head_dim, window (None = all keys), position (a PartSpec).
"""
from __future__ import annotations

import math

import torch

from ..weights import TensorSpec
from .base import KVCacheRequest, Mixer, POSITION_ENCODINGS, lookup, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight
from .paged_attention import PagedAttention


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    graph_safe = True
    supports_rows = True
    takes_deferred_norm = True

    @staticmethod
    def check_params(params):
        PagedAttention.check(int(params["heads"]), int(params["kv_heads"]), int(params["head_dim"]))
        position = params["position"]
        lookup(POSITION_ENCODINGS, position.kind, "position encoding").check_params(position.params)

    @staticmethod
    def tensor_specs(params, prefix):
        h, nq, nkv, d = params["hidden"], params["heads"], params["kv_heads"], params["head_dim"]
        return [TensorSpec(prefix + "q_proj.weight", (nq * d, h)),
                TensorSpec(prefix + "k_proj.weight", (nkv * d, h)),
                TensorSpec(prefix + "v_proj.weight", (nkv * d, h)),
                TensorSpec(prefix + "o_proj.weight", (h, nq * d))]

    @staticmethod
    def cache_request(params):
        return KVCacheRequest(params["kv_heads"], params["head_dim"], params.get("window"))

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden = int(params["hidden"])
        self.nq, self.nkv, self.d = int(params["heads"]), int(params["kv_heads"]), int(params["head_dim"])
        self.window = params.get("window")
        self.scale = 1.0 / math.sqrt(self.d)
        self.w_qkv = prepare_weight(torch.cat([tensors[prefix + "q_proj.weight"],
                                               tensors[prefix + "k_proj.weight"],
                                               tensors[prefix + "v_proj.weight"]], dim=0), runtime)
        self.w_o = prepare_weight(tensors[prefix + "o_proj.weight"], runtime)
        position = params["position"]
        self.position = lookup(POSITION_ENCODINGS, position.kind, "position encoding")(
            position.params, tensors, prefix, runtime)
        self.graph_safe = bool(self.position.graph_safe)
        # the kernels that will serve this attention are chosen here, once; sizes they cannot take are refused here
        self.attention = PagedAttention(runtime.compute_dtype, self.nq, self.nkv, self.d, self.window, self.scale,
                                        rotate_half=self.position.rotate_half())

    def graph_key(self, ctx) -> tuple:
        return self.position.graph_key(ctx) + self.attention.graph_key(ctx)

    def forward(self, ctx, x, residual, scale, kv=None, state=None, rows=None, n_rows=None):
        """`rows` (device int32, `n_rows` of them): only these tokens' outputs are needed.  `residual` then holds
        those rows alone ([n_rows, hidden]); keys and values of every token are still appended."""
        rt, n = self.runtime, x.shape[0]
        nq, nkv, d = self.nq, self.nkv, self.d
        flag = ctx.error_flag
        qkv = ctx.buffer("attn.qkv", (n, (nq + 2 * nkv) * d), torch.float32)
        linear(rt, STORE, x, self.w_qkv, qkv, error_flag=flag, name="qkv")
        o = ctx.buffer("attn.o", (n, nq * d), rt.compute_dtype)
        if rows is None:
            if not self.attention.forward_fused(ctx, qkv, kv, o):
                q = ctx.buffer("attn.q", (n, nq * d), rt.compute_dtype)
                self.position.encode_and_store(ctx, qkv, q, kv, nq, nkv, d)
                self.attention.forward(ctx, q, kv, o)
            linear(rt, ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
            return
        q = ctx.buffer("attn.q", (n, nq * d), rt.compute_dtype)
        self.position.encode_and_store(ctx, qkv, q, kv, nq, nkv, d)       # the cache takes every token
        if n_rows == 0:
            return
        if n_rows * 8 <= n:
            self.attention.forward(ctx, q, kv, o, rows=rows, n_rows=n_rows)   # few rows: only they attend
        else:
            self.attention.forward(ctx, q, kv, o)
        picked = ctx.buffer("attn.o_rows", (n_rows, nq * d), rt.compute_dtype)
        rt.ops.gather_rows(o, rows, picked)
        linear(rt, ACCUM, picked, self.w_o, residual, scale, error_flag=flag, name="o")
