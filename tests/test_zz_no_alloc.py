"""lia_gemm_tc_noalloc, called through its exported C symbol, against the ordinary entry point.

The entry point serves hosts that must not call cudaMalloc when they need a product (a frozen memory
pool, a plug-in whose host owns device memory): its split-K scratch is a static array inside the
library.  This file is collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It must pass alone in a fresh process and after the other tests."""
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ERR_SCRATCH = -6
SCRATCH_FLOATS = (8 << 20) // 4


def entry_points():
    from lia_rs_b200.kernels import build
    lib = build.load()
    fn = lib.lia_gemm_tc_noalloc
    fn.argtypes = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                   c_int, c_void_p, c_void_p]
    fn.restype = c_int
    need = lib.lia_gemm_tc_noalloc_scratch_floats
    need.argtypes = [c_int, c_int, c_int, c_int, c_int]
    need.restype = c_longlong
    lib.lia_gemm_tc_noalloc_reset.argtypes = [c_void_p]
    lib.lia_gemm_tc_noalloc_reset.restype = c_int
    return fn, need


def reset(stream=None):
    from lia_rs_b200.kernels import build
    return build.load().lia_gemm_tc_noalloc_reset(stream or torch.cuda.current_stream().cuda_stream)


def free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info(DEV)[0]          # the driver's count: cudaMalloc by anyone in the process shows here


def call(fn, mode, a, w, out, alpha, flag, sms):
    from lia_rs_b200.kernels import ops
    M, K = a.shape
    N = out.shape[1]
    return fn(mode, a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), ops.dtype_code(out.dtype),
              out.stride(0), M, N, K, alpha, sms, flag.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_no_alloc_product_equals_the_ordinary_one_on_two_calls_in_a_row():
    from lia_rs_b200.kernels import ops
    fn, need = entry_points()
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    # a first call, so that the address lookup (and whatever the driver loads for it) lies behind us
    warm_a = torch.randn(4, 512, device=DEV).to(torch.bfloat16)
    warm_w = torch.randn(256, 512, device=DEV).to(torch.bfloat16)
    assert call(fn, ops.GEMM_STORE, warm_a, warm_w, torch.empty(4, 256, device=DEV), 1.0, flag, sms) == 0
    # two different split-K shapes back to back: the second finds the first one's partial sums in the array
    for call_index, (mode, M, N, K) in enumerate([(ops.GEMM_STORE, 8, 2560, 2048), (ops.GEMM_SWIGLU, 5, 1000, 6144),
                                                  (ops.GEMM_ACCUM, 3, 200, 2048)]):
        torch.manual_seed(call_index)
        a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        rows = 2 * N if mode == ops.GEMM_SWIGLU else N
        w = (torch.randn(rows, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
        assert need(mode, M, N, K, sms) > 0, "the shape was meant to split K and use the scratch"
        base = torch.randn(M, N, device=DEV)
        want, got = base.clone(), base.clone()
        ops.gemm_tc(mode, a, w, want, 0.5, flag)
        held, free = torch.cuda.memory_allocated(DEV), free_bytes()
        assert call(fn, mode, a, w, got, 0.5, flag, sms) == 0
        assert free_bytes() == free and torch.cuda.memory_allocated(DEV) == held      # neither the driver nor torch gave memory out
        exact = a.double() @ w.double().T
        if mode == ops.GEMM_SWIGLU:
            gate, up = exact[:, :N], exact[:, N:]
            exact = up * gate / (1 + torch.exp(-gate))
        elif mode == ops.GEMM_ACCUM:
            exact = base.double() + 0.5 * exact
        else:
            exact = 0.5 * exact
        scale = max(1.0, float(exact.abs().max()))
        limit = 2e-5 * scale * math.sqrt(K / 64)                  # the tolerance of the product's own test
        assert float((got.double() - want.double()).abs().max()) <= limit
        assert float((got.double() - exact).abs().max()) <= limit
    assert flag.item() == 0


def test_no_alloc_refuses_what_its_array_cannot_hold():
    from lia_rs_b200.kernels import ops
    fn, need = entry_points()
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    M, N, K = 128, 12288, 2048                                     # two ranges or more x 128 x 12288 floats > 8 MiB
    assert need(ops.GEMM_STORE, M, N, K, sms) > SCRATCH_FLOATS
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    out = torch.full((M, N), 3.0, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert call(fn, ops.GEMM_STORE, a, w, out, 1.0, flag, sms) == ERR_SCRATCH
    torch.cuda.synchronize()
    assert float((out - 3.0).abs().max()) == 0.0                    # nothing ran


def test_no_alloc_reset_zeroes_the_counters_and_products_go_on():
    from lia_rs_b200.kernels import ops
    fn, need = entry_points()
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.manual_seed(3)
    M, N, K = 8, 2560, 2048
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    assert need(ops.GEMM_STORE, M, N, K, sms) > 0
    exact = a.double() @ w.double().T
    limit = 2e-5 * max(1.0, float(exact.abs().max())) * math.sqrt(K / 64)
    for _ in range(2):
        out = torch.zeros(M, N, device=DEV)
        free = free_bytes()
        assert reset() == 0
        assert call(fn, ops.GEMM_STORE, a, w, out, 1.0, flag, sms) == 0
        assert free_bytes() == free
        assert float((out.double() - exact).abs().max()) <= limit
    assert flag.item() == 0
