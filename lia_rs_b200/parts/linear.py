"""Matrix products of the parts: out (op)= alpha * a @ w^T with an epilogue.

`prepare_weight` brings a checkpoint matrix to the compute element type once, at load.
`linear` chooses the kernel.  bfloat16: up to 16 tokens the kernel that streams the weights once with
no meeting of CTAs (csrc/gemm_skinny.cu); beyond that, while the product has too few output tiles to
fill the SMs, the tcgen05 kernel that cuts K over a cluster (csrc/gemm_cluster.cu); with many output
tiles the few-token kernel again up to its 32 tokens (the output head), then the persistent tcgen05
kernel (csrc/gemm_tc.cu), when the shape allows them; else, and always for the 32-bit path, the product
on the 32-bit pipes.  (Measured per 2B-class layer: 16 tokens 58 us with the few-token kernel, 63 us with
the cluster kernel; 24 tokens 82 against 66; 32 tokens 91 against 70: every CTA of the few-token kernel
reads all the tokens' rows from L2.)"""
from __future__ import annotations

import torch

from ..kernels import ops

STORE, ACCUM, SWIGLU = ops.GEMM_STORE, ops.GEMM_ACCUM, ops.GEMM_SWIGLU


def prepare_weight(weight: torch.Tensor, runtime) -> torch.Tensor:
    return weight.to(runtime.compute_dtype).contiguous()


SKINNY_BEST_TOKENS = 16


def linear(runtime, mode: int, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0):
    few = a.dtype == torch.bfloat16 and ops.gemm_skinny_accepts(mode, a, w, out)
    if few and (a.shape[0] <= SKINNY_BEST_TOKENS or not ops.gemm_cluster_accepts(mode, a, w, out)):
        ops.gemm_skinny(mode, a, w, out, alpha)
    elif a.dtype == torch.bfloat16 and ops.gemm_cluster_accepts(mode, a, w, out):
        ops.gemm_cluster(mode, a, w, out, alpha)
    elif a.dtype == torch.bfloat16 and ops.gemm_tc_accepts(mode, a, w, out):
        ops.gemm_tc(mode, a, w, out, alpha)
    else:
        ops.gemm_simt(mode, a, w, out, alpha)
