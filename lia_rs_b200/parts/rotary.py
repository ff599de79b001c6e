"""Rotary position encoding, rotate-half over the first `rotary_dim` elements of each head
(src/gpu/kernels/llama.rs:44-55): inv_i = theta^(-2i/rotary_dim), angle = position * inv_i.
The inverse frequencies are computed in 64-bit on the host and rounded once to 32-bit; angle,
sine and cosine are 32-bit on the device.  Fused with the append of keys and values to the cache.
Parameters: theta, rotary_dim.  `none` encodes nothing and only appends."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # positions are read on the device

    @staticmethod
    def check_params(params):
        rotary_dim, theta = int(params["rotary_dim"]), float(params["theta"])
        if rotary_dim % 2 or rotary_dim <= 0 or not theta > 0:
            raise ValueError("rotary encoding needs an even positive rotary_dim and theta > 0")

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.rotary_dim = int(params["rotary_dim"])
        theta = float(params["theta"])
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv = 1.0 / (theta ** (2.0 * i / self.rotary_dim))
        self.inv_freq = inv.to(torch.float32).to(runtime.device)

    def rotate_half(self):
        return self.rotary_dim, self.inv_freq

    def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d):
        self.runtime.ops.rope_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                       kv.v_pages, nq, nkv, d, self.rotary_dim, self.inv_freq,
                                       write_kv=kv.writes, error_flag=ctx.error_flag)


@register_position_encoding("none")
class NoEncoding(PositionEncoding):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # positions are read on the device

    def rotate_half(self):
        return 0, None

    def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d):
        self.runtime.ops.rope_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                       kv.v_pages, nq, nkv, d, 0, None, write_kv=kv.writes,
                                       error_flag=ctx.error_flag)
