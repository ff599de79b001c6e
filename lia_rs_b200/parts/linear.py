"""Matrix products of the parts: out (op)= alpha * a @ w^T with an epilogue.

`prepare_weight` brings a checkpoint matrix to the compute element type once, at load.
`linear` chooses the kernel for a bfloat16 product (measured on a B200, in TB/s of weights streamed):
* up to 16 tokens the persistent kernel that keeps the tokens' rows on the SM and streams the weights
  through a ring (csrc/gemm_stream.cu; a 2B-class layer's four products at 8 tokens: 23.7 us against 30.0 for
  the one-CTA-per-16-rows kernel below; the output head, 73,448 x 2,048, at 8 tokens: 47.6 us = 6.3 TB/s against
  60.3 us for the tcgen05 kernel), which can also norm its input rows itself (`a` a `DeferredNorm`: no norm
  kernel runs then);
* beyond that, a product whose output tiles alone occupy the SMs (the output head, a wide gate/up matrix) goes
  to the persistent tcgen05 kernel (csrc/gemm_tc.cu) at every number of tokens (the head at 24 tokens: 60 us
  against 169 for the few-token kernel);
* otherwise, where the persistent few-token kernel does not take the sizes, up to 16 tokens the kernel that
  streams the weights once with one CTA per 16 rows (csrc/gemm_skinny.cu); beyond 16 tokens, the tcgen05 kernel that cuts K over a cluster (csrc/gemm_cluster.cu)
  while it applies (16 tokens of a 2B-class layer: 58 us with the few-token kernel, 63 us with the cluster
  kernel; 24 tokens: 82 against 66; 32 tokens: 91 against 70: every CTA of the few-token kernel reads all the
  tokens' rows from L2) and up to 256 tokens; then the persistent tcgen05 kernel, which cuts K through scratch
  memory up to 128 tokens and beyond that cuts the tokens into tiles as narrow as fills the SMs (a 2B-class
  layer's four products at 512 tokens: 90 us, at 256 tokens 70 us with the cluster kernel for three of them);
* what TMA cannot address goes to the few-token kernel if it can take it, else, and always for the 32-bit
  path, to the product on the 32-bit pipes (csrc/gemm_simt.cu)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import DeferredNorm

STORE, ACCUM, SWIGLU = ops.GEMM_STORE, ops.GEMM_ACCUM, ops.GEMM_SWIGLU


def prepare_weight(weight: torch.Tensor, runtime) -> torch.Tensor:
    return weight.to(runtime.compute_dtype).contiguous()


SKINNY_BEST_TOKENS = 16
CLUSTER_MAX_TOKENS = 256        # beyond, narrow tiles of the persistent kernel are as fast or faster (2,048 x 2,048 at 512 tokens: 14.9 against 18.2 us)


_TC, _SKINNY, _CLUSTER, _SIMT, _STREAM = range(5)
_choices = {}          # what decides the choice -> the kernel chosen (the checks cost more than the lookup)


def _choose(mode, a, w, out) -> int:
    tensor_cores = ops.gemm_tc_accepts(mode, a, w, out)
    few = ops.gemm_skinny_accepts(mode, a, w, out)
    if a.shape[0] <= ops.STREAM_MAX_TOKENS and ops.gemm_stream_accepts(mode, a, w, out):
        return _STREAM
    if tensor_cores and ops.gemm_tc_tiles_fill_the_sms(a, out):
        return _TC
    if few and a.shape[0] <= SKINNY_BEST_TOKENS:
        return _SKINNY
    if tensor_cores and a.shape[0] <= CLUSTER_MAX_TOKENS and ops.gemm_cluster_accepts(mode, a, w, out):
        return _CLUSTER
    if tensor_cores:
        return _TC
    return _SKINNY if few else _SIMT


def linear(runtime, mode: int, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0,
           error_flag=None, name=None):
    """`name`: what the product is to its caller ("qkv", "down", ...), for the per-kernel-class profile.
    `error_flag` (int32[1] on the device, a step's `ctx.error_flag`): a tensor-core kernel that gives up on one
    of its bounded waits raises it to 3, and the step's caller then learns that the result is not to be used."""
    if isinstance(a, DeferredNorm):
        # few tokens of a norm that a product kernel can apply itself: the norm's own kernel does not run
        record = a.norm.rms_record() if a.source.shape[0] <= ops.STREAM_MAX_TOKENS and w.dtype == torch.bfloat16 else None
        if record is not None:
            source, (norm_weight, eps) = a.source, record
            key = ("norm", mode, source.shape, source.stride(), source.data_ptr() & 15, w.shape, w.stride(), w.data_ptr() & 15,
                   out.shape[1], out.stride(), out.dtype, norm_weight.dtype, norm_weight.data_ptr() & 15, source.device.index)
            fused = _choices.get(key)
            if fused is None:
                fused = _choices[key] = (norm_weight.is_contiguous() and norm_weight.data_ptr() % 16 == 0
                                         and norm_weight.dtype in (torch.bfloat16, torch.float32)
                                         and ops.gemm_stream_accepts(mode, source, w, out, norm=True))
            if fused:
                ops.gemm_stream(mode, source, w, out, alpha, error_flag, label=name, norm_weight=norm_weight, eps=eps)
                return
        a = a.tensor()
    if a.dtype != torch.bfloat16:
        ops.gemm_simt(mode, a, w, out, alpha, label=name)
        return
    # everything the kernels' acceptance looks at: sizes, row strides, element types, 16-byte alignment of the bases
    key = (mode, a.shape, a.stride(), a.data_ptr() & 15, w.shape, w.stride(), w.dtype, w.data_ptr() & 15,
           out.shape[1], out.stride(), out.dtype, out.data_ptr() & 15, a.device.index)
    choice = _choices.get(key)
    if choice is None:
        choice = _choices[key] = _choose(mode, a, w, out)
    if choice == _TC:
        ops.gemm_tc(mode, a, w, out, alpha, error_flag, label=name)
    elif choice == _STREAM:
        ops.gemm_stream(mode, a, w, out, alpha, error_flag, label=name)
    elif choice == _SKINNY:
        ops.gemm_skinny(mode, a, w, out, alpha, error_flag, label=name)
    elif choice == _CLUSTER:
        ops.gemm_cluster(mode, a, w, out, alpha, error_flag, label=name)
    else:
        ops.gemm_simt(mode, a, w, out, alpha, label=name)
