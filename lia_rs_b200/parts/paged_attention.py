"""Causal softmax attention of a step's tokens over a paged cache: which kernel serves which rows.

A mixer builds one `PagedAttention` from its sizes when it is built; the choice of kernels is made there,
once, and an unsupported size is refused there with its reason.  The kernels (csrc/):

  variant "tensor"   bfloat16 with head size 32, 64 or 128: single decoded tokens go to the split-key kernel
                     (attention_decode.cu), prompt portions to the tcgen05 kernel (attention_prefill_tc.cu) where it
                     takes the head size and group, else to the mma.sync kernel (attention_prefill.cu), else
                     (more than 64 query heads per kv head) to the kernel for every size;
  variant "generic"  everything else: the 32-bit path, and bfloat16 with another head size
                     (attention_generic.cu: a warp per token and head, 32-bit probabilities).  On the bfloat16
                     path this is a slow road, so it is said once when such a mixer is built.

Head sizes are multiples of 16 up to 256 (what attention_generic.cu takes); `check` refuses others.
The reference chooses between its scalar and tensor attention kernels per call from the row count and the
context (src/inference/llama.rs:15-35,131-151, src/inference/llama_plan.rs:76-99).
"""
from __future__ import annotations

import sys

import torch

from ..kernels import ops

_told = set()


class PagedAttention:
    @staticmethod
    def check(heads: int, kv_heads: int, head_dim: int) -> None:
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ValueError("attention: heads must be a positive multiple of kv_heads")
        if head_dim <= 0 or head_dim % ops.ATTENTION_HEAD_DIM_STEP or head_dim > ops.ATTENTION_HEAD_DIM_MAX:
            raise ValueError(f"attention: head_dim {head_dim} is not a multiple of {ops.ATTENTION_HEAD_DIM_STEP} of at "
                             f"most {ops.ATTENTION_HEAD_DIM_MAX} (what the attention kernels take)")

    def __init__(self, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, window, scale: float,
                 rotate_half=None):
        """`rotate_half`: what the mixer's position encoding answers to `rotate_half()`; with it (and the
        tensor variant, and at most 16 query heads per kv head) decode-only steps encode, append and attend in
        one kernel (`forward_fused`)."""
        self.check(heads, kv_heads, head_dim)
        self.nq, self.nkv, self.d = int(heads), int(kv_heads), int(head_dim)
        self.window, self.scale = window, float(scale)
        self.group = self.nq // self.nkv
        self.variant = "tensor" if dtype == torch.bfloat16 and self.d in ops.DECODE_HEAD_DIMS else "generic"
        if dtype == torch.bfloat16 and self.variant == "generic" and self.d not in _told:
            _told.add(self.d)
            print(f"[lia_rs_b200] bfloat16 attention with head size {self.d} runs on the kernel for every size "
                  f"(32-bit probabilities, a warp per token and head); the tensor-core kernels take "
                  f"{ops.DECODE_HEAD_DIMS}", file=sys.stderr, flush=True)
        self.rotate_half = rotate_half if (self.variant == "tensor" and self.group <= 16) else None
        self._prefill = None          # (kernel, tokens per tile), asked of the library at the first prompt portion
        self._decode_plans = {}       # (rows, wanted ranges) -> (ranges, as clusters)
        self._ctas_per_sm = None      # CTAs of the decode kernel that an SM holds, asked of the library at the first decode step

    # ---- how a decode row's keys are cut ----
    def decode_splits(self, ctx, rows: int) -> int:
        """Into how many ranges the decode kernel cuts each token's keys: as many as fill the CTAs that the SMs
        hold at once (two an SM at head size 128, four at 64: 64 tokens of 16/2 heads of 64 over ~2,250 keys take
        25.6 us in two ranges, 16.3 in four), in one round; no more than 32 (the last CTA of a token reads them
        all) and none shorter than 256 keys at the step's longest context.  It depends on the number of rows and
        on the context bucket alone (each token then cuts its own span, on the device), so a captured step serves
        every step of its shape and bucket."""
        groups = self.nkv * ((self.group + 15) // 16)
        ctas = max(1, rows * groups)
        if self._ctas_per_sm is None:
            self._ctas_per_sm = ops.attention_decode_ctas_per_sm(self.d, self.group) or 2
        wanted = (self._ctas_per_sm * ctx.runtime.sm_count) // ctas
        return max(1, min(wanted, 32, ctx.context_bucket // 256))

    def decode_plan(self, ctx, rows: int):
        """(ranges per token, whether a token's ranges form a thread-block cluster).  As clusters (2, 4, 8 or 16
        ranges, all clusters on the device at once) the ranges meet in distributed shared memory; otherwise
        through scratch memory, the CTA that finishes a token last combining them."""
        wanted = self.decode_splits(ctx, rows)
        plan = self._decode_plans.get((rows, wanted))
        if plan is None:
            groups = self.nkv * ((self.group + 15) // 16)
            clustered = ops.attention_decode_cluster_splits(self.d, self.group, rows * groups, wanted) if wanted >= 2 else 1
            plan = self._decode_plans[(rows, wanted)] = (clustered, True) if clustered >= 2 else (wanted, False)
        return plan

    def prefill_splits(self, ctx, tiles: int) -> int:
        """Into how many ranges the tcgen05 prompt kernel cuts the keys of each of its CTAs: as many as give every
        SM a CTA, none shorter than 1,024 keys at the step's context bucket (so none before 1,024 tokens), at most 16.  A whole prompt has CTAs
        enough and is not cut; a short portion late in a long prompt is (the reference cuts a tile's keys into parts
        of 4,096 and merges them: src/inference/llama_plan.rs:76-99).  It depends on the portions' lengths and the
        context bucket alone, as a captured step needs."""
        ctas = max(1, tiles * self.nkv)
        return max(1, min(ctx.runtime.sm_count // ctas, 16, ctx.context_bucket // 1024))

    def _decode_scratch(self, ctx, rows: int, n_splits: int):
        if n_splits <= 1:
            return None, None
        partial = ctx.runtime.scratch("attn.partial", ctx.n_tokens * self.nq * n_splits * (self.d + 1), torch.float32)
        counters = ctx.runtime.counters(rows * self.nkv * ((self.group + 15) // 16))
        return partial, counters

    def _work(self, ctx, element_size: int):
        """(cache bytes the single-token rows must read, flops of the prompt portions), for the profile only."""
        if ops._profiler is None:
            return 0, 0
        def visible(position):
            return position + 1 if self.window is None else min(position + 1, self.window)
        keys = sum(visible(start) for _, start, count, _ in ctx.segments if count == 1)
        pairs = sum(visible(start + i) for _, start, count, _ in ctx.segments if count > 1 for i in range(count))
        return keys * 2 * self.nkv * self.d * element_size, 4 * self.nq * self.d * pairs

    def _prefill_kernel(self):
        """(kernel, tokens per tile) for prompt portions, asked of the library once."""
        if self._prefill is None:
            per_tile = ops.attention_prefill_tc_tokens_per_tile(self.group, self.d)
            if per_tile:
                self._prefill = (ops.attention_prefill_tc, per_tile)
            else:
                self._prefill = (ops.attention_prefill, ops.attention_prefill_tokens_per_tile(self.group))
        return self._prefill

    def graph_key(self, ctx) -> tuple:
        """What of a step's shape the launches below depend on beyond the numbers of tokens, single-token entries and
        portions and the context bucket: into how many tiles the prompt kernel cuts the portions.  (Where the
        portions begin and how long each is, the kernels read on the device.)"""
        if self.variant != "tensor" or not ctx.n_prefill_segments:
            return ()
        per_tile = self._prefill_kernel()[1]
        if not per_tile:
            return ()
        return (per_tile, sum((count + per_tile - 1) // per_tile for _, _, count, _ in ctx.segments if count > 1))

    # ---- the step's attention ----
    def forward(self, ctx, q, kv, out, rows=None, n_rows=None):
        """out[t] = attention of token t's encoded queries `q[t]` over the cache `kv` (keys and values of this
        step already appended), for every token of the step, or only for the tokens whose batch indices the
        device tensor `rows` lists (`n_rows` of them; the other rows of `out` are left as they are)."""
        nq, nkv, d = self.nq, self.nkv, self.d
        if rows is not None:
            if n_rows == 0:
                return
            if self.variant == "generic":
                ops.attention_generic(q, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table, out, nq, nkv,
                                      d, self.window, self.scale, rows=rows[:n_rows], error_flag=ctx.error_flag)
            else:
                # (the wanted rows of a step with prompt portions are those portions' last tokens: the kernels ahead
                # have written keys anywhere before them, not just their own)
                self._decode(ctx, q, kv, out, rows[:n_rows], n_rows, all_new=ctx.n_prefill_segments > 0)
            return
        work_bytes, work_flops = self._work(ctx, q.element_size())
        if self.variant == "generic":
            ops.attention_generic(q, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table, out, nq, nkv, d,
                                  self.window, self.scale, error_flag=ctx.error_flag, work_bytes=work_bytes)
            return
        if ctx.decode_rows.numel():
            self._decode(ctx, q, kv, out, ctx.decode_rows, ctx.decode_rows.numel(), work_bytes)
        if ctx.n_prefill_segments:
            kernel, per_tile = self._prefill_kernel()
            if per_tile:
                tiles = sum((count + per_tile - 1) // per_tile for _, _, count, _ in ctx.segments if count > 1)
                more = {}
                if kernel is ops.attention_prefill_tc:
                    splits = self.prefill_splits(ctx, tiles)
                    if splits > 1:
                        words = ops.attention_prefill_tc_partial_floats(ctx.n_tokens, nq, d, splits)
                        more = dict(splits=splits, partial=ctx.runtime.scratch("attn.prefill_partial", words, torch.float32))
                kernel(q, kv.k_pages, kv.v_pages, ctx.prefill_segments, ctx.n_prefill_segments, tiles, ctx.slots,
                       kv.block_table, out, nq, nkv, d, self.window, self.scale, ctx.error_flag, work_flops=work_flops,
                       **more)
            else:
                ops.attention_generic(q, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table, out, nq, nkv,
                                      d, self.window, self.scale, rows=ctx.prefill_rows, error_flag=ctx.error_flag)

    def _decode(self, ctx, q, kv, out, rows, n_rows, work_bytes=0, all_new=False):
        n_splits, clustered = self.decode_plan(ctx, n_rows)
        partial, counters = (None, None) if clustered else self._decode_scratch(ctx, n_rows, n_splits)
        ops.attention_decode(q, kv.k_pages, kv.v_pages, rows, ctx.positions, ctx.slots, kv.block_table, out, partial,
                             self.nq, self.nkv, self.d, self.window, self.scale, 0, n_splits, counters,
                             error_flag=ctx.error_flag, work_bytes=work_bytes, cluster=clustered, all_new=all_new)

    def forward_fused(self, ctx, qkv, kv, out) -> bool:
        """For a step of single decoded tokens and a rotate-half (or no) position encoding: encoding of q and k,
        append of k and v to `kv`, and attention, in one kernel.  Returns False, having done nothing, when the
        step or this attention is not of that kind; the caller then encodes and attends separately."""
        if self.rotate_half is None or not ctx.decode_only or kv.k_pages.dtype != torch.bfloat16:
            return False
        rotary_dim, inv_freq = self.rotate_half
        n_splits, clustered = self.decode_plan(ctx, ctx.n_tokens)
        partial, counters = (None, None) if clustered else self._decode_scratch(ctx, ctx.n_tokens, n_splits)
        ops.attention_decode(None, kv.k_pages, kv.v_pages, ctx.decode_rows, ctx.positions, ctx.slots, kv.block_table,
                             out, partial, self.nq, self.nkv, self.d, self.window, self.scale, 0, n_splits, counters,
                             qkv=qkv, inv_freq=inv_freq, rotary_dim=rotary_dim, write_kv=kv.writes,
                             error_flag=ctx.error_flag, label="fused", work_bytes=self._work(ctx, 2)[0], cluster=clustered)
        return True
