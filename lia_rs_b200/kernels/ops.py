"""Python faces of the CUDA entry points.  Every function takes CUDA tensors, checks what the
kernel assumes, launches on the current stream and raises on a refusal; there is no CPU or
library fallback here."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUM, GEMM_SWIGLU = 0, 1, 2

_ERRORS = {-1: "a size the kernel refuses", -2: "a pointer or stride that is not aligned as required",
           -3: "the launch failed (cudaGetLastError)", -4: "a driver entry point is missing or failed",
           -5: "no instantiation for this combination of element types"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = build.load()
        for name in dir(_Signatures):
            if name.startswith("lia_"):
                fn = getattr(_lib, name)
                fn.argtypes = getattr(_Signatures, name)
                fn.restype = c_int
    return _lib


class _Signatures:
    lia_embedding = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    lia_rmsnorm = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p]
    lia_rope_kv_write = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_gemm_simt = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                     c_int, c_int, c_float, c_void_p]
    lia_attention_generic = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]
    lia_gather_rows = [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong,
                       ctypes.c_longlong, c_void_p]
    lia_wait_probe = [c_int, c_void_p, c_void_p, c_void_p]
    lia_attention_decode = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_attention_decode_cluster_splits = [c_int, c_int, c_int, c_int]
    lia_attention_decode_ctas_per_sm = [c_int, c_int]
    lia_gemm_tc = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                   c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p]
    lia_gemm_cluster = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                        c_int, c_void_p, c_void_p]
    lia_gemm_cluster_splits = [c_int, c_int, c_int, c_int, c_int]
    lia_gemm_skinny = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                       c_void_p, c_void_p]
    lia_gemm_stream = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                       c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_gemm_stream_stages = [c_int, c_int, c_int, c_int, c_int, c_int]
    lia_attention_prefill = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]
    lia_attention_prefill_tc = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_void_p]
    lia_attention_prefill_tc_tokens_per_tile = [c_int, c_int]
    lia_select_tokens = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                         ctypes.c_longlong, c_void_p]
    lia_select_tokens_scratch_floats = [c_int, c_int]
    lia_select_candidates = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, ctypes.c_longlong, c_void_p]
    lia_select_candidates_scratch_floats = [c_int, c_int, c_int]


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dtype} has no kernel")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels need contiguous CUDA tensors (there is no CPU path)")


def _p(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle.  Asked for at every launch (a graph capture runs on a stream of its own), so through
    torch's direct call where this torch has it: building a Stream object each time cost several microseconds a launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def kernel_launches() -> int:
    """Kernels this library has launched since it was loaded, counted at the launch sites in C.  A
    replay of a captured CUDA graph runs its kernels again without passing a launch site: the engine
    adds those (`Engine.stats['kernels']`)."""
    fn = lib().lia_kernel_launches
    fn.restype = ctypes.c_longlong
    fn.argtypes = []
    return int(fn())


def _check(code: int, what: str):
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, code)}")


class Profiler:
    """Device time per kernel class, from CUDA events around every launch of this library while it is
    installed (`set_profiler`).  The reference's counterpart is LIA_PROFILE: a synchronisation and a host timer
    around every product, name, shape and seconds printed (src/inference/operations.rs:85-90,303-310); like it,
    this cannot run under a captured graph.  Events between launches also keep a kernel from starting under its
    predecessor's tail, so the times are those of a launch-by-launch step: read them as shares."""

    def __init__(self):
        self.records = []                        # (class, start event, end event, bytes, flops)

    def summary(self) -> dict:
        """class -> {calls, ms, bytes, flops} over what was recorded since the last call; waits for the device."""
        torch.cuda.synchronize()
        out = {}
        for key, start, end, nbytes, flops in self.records:
            entry = out.setdefault(key, {"calls": 0, "ms": 0.0, "bytes": 0, "flops": 0})
            entry["calls"] += 1
            entry["ms"] += start.elapsed_time(end)
            entry["bytes"] += int(nbytes)
            entry["flops"] += int(flops)
        self.records = []
        return out


class _Timed:
    __slots__ = ("key", "nbytes", "flops", "start")

    def __init__(self, key, nbytes, flops):
        self.key, self.nbytes, self.flops = key, nbytes, flops

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        if _profiler is not None:
            _profiler.records.append((self.key, self.start, end, self.nbytes, self.flops))
        return False


class _NotTimed:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_profiler = None
_NOT_TIMED = _NotTimed()


def set_profiler(profiler) -> None:
    """Install (or, with None, remove) the profiler that every launch of this library reports to."""
    global _profiler
    _profiler = profiler


def _timed(kernel: str, label=None, nbytes=0, flops=0, work=None):
    """`work`: a function giving (bytes, flops), asked only while a profiler listens."""
    if _profiler is None:
        return _NOT_TIMED
    if work is not None:
        nbytes, flops = work()
    return _Timed(f"{kernel}:{label}" if label else kernel, nbytes, flops)


def _gemm_work(a, w, out):
    """(bytes, flops) of a product as the roofline counts them: every operand once."""
    return (a.numel() * a.element_size() + w.numel() * w.element_size() + out.numel() * out.element_size(),
            2 * a.shape[0] * w.shape[0] * a.shape[1])


def embedding(tokens, table, out, scale: float, error_flag=None):
    _cuda(tokens, table, out, error_flag)
    n, hidden = out.shape
    with _timed("embedding"):
        _check(lib().lia_embedding(_p(tokens), _p(table), dtype_code(table.dtype), _p(out), n, hidden,
                                   table.shape[0], scale, _p(error_flag), _stream()), "embedding")


def rmsnorm(x, weight, out, eps: float, out_scale: float = 1.0, rows_index=None):
    _cuda(x, weight, out, rows_index)
    rows, hidden = out.shape
    if x.dtype != torch.float32 or x.shape[1] != hidden:
        raise KernelError("rmsnorm takes 32-bit rows of the same width as its output")
    with _timed("rmsnorm"):
        _check(lib().lia_rmsnorm(_p(x), _p(rows_index), _p(weight), dtype_code(weight.dtype), _p(out),
                                 dtype_code(out.dtype), rows, hidden, eps, out_scale, _stream()), "rmsnorm")


def rope_kv_write(qkv, positions, slots, block_table, q_out, k_pages, v_pages, nq, nkv, d, rotary_dim,
                  inv_freq, write_kv=True, error_flag=None):
    _cuda(qkv, positions, slots, block_table, q_out, k_pages, v_pages, inv_freq, error_flag)
    n = qkv.shape[0]
    if qkv.dtype != torch.float32 or qkv.shape[1] != (nq + 2 * nkv) * d:
        raise KernelError("rope_kv_write takes 32-bit q|k|v rows")
    if q_out.dtype != k_pages.dtype or k_pages.dtype != v_pages.dtype:
        raise KernelError("rope_kv_write: q and the cache must have one element type")
    num_pages, page_size = k_pages.shape[0], k_pages.shape[1]
    with _timed("rope_kv_write"):
        _check(lib().lia_rope_kv_write(_p(qkv), _p(positions), _p(slots), _p(block_table), block_table.shape[1],
                                       _p(q_out), _p(k_pages), _p(v_pages), dtype_code(q_out.dtype), n, nq, nkv, d,
                                       rotary_dim, _p(inv_freq), page_size, num_pages, 1 if write_kv else 0,
                                       _p(error_flag), _stream()), "rope_kv_write")


def gather_rows(src, index, dst):
    """dst[r] = src[index[r]] for 2-D tensors of one element type and width (rows copied as they are; a negative
    index gives zeros); see csrc/elementwise.cu."""
    _cuda(index)
    if not (src.is_cuda and dst.is_cuda) or src.dim() != 2 or dst.dim() != 2 or src.dtype != dst.dtype \
            or src.shape[1] != dst.shape[1] or src.stride(1) != 1 or dst.stride(1) != 1 or index.dtype != torch.int32 \
            or index.numel() < dst.shape[0]:
        raise KernelError("gather_rows: 2-D CUDA tensors of one type and width, int32 index of at least dst's rows")
    size = src.element_size()
    with _timed("gather_rows"):
        _check(lib().lia_gather_rows(_p(src), _p(index), _p(dst), dst.shape[0], src.shape[0], src.stride(0) * size,
                                     dst.stride(0) * size, src.shape[1] * size, _stream()), "gather_rows")


def wait_probe(polls: int, error_flag, gave_up=None):
    """One thread waits on an mbarrier that nobody arrives at, gives up after `polls` polls (at most 65,536) and
    raises error flag 3, exactly as the tensor-core kernels' bounded waits do; see csrc/library.cu."""
    _cuda(error_flag, gave_up)
    _check(lib().lia_wait_probe(int(polls), _p(error_flag), _p(gave_up), _stream()), "wait_probe")


def reset_scratch(device) -> None:
    """Zero the counters at the head of this device's split-K scratch: a product that gave up may have left
    them mid-count (every product that runs to its end leaves them at zero)."""
    key = torch.device(device).index or 0
    if key in _scratch:
        _scratch[key][:COUNTER_WORDS].zero_()


def gemm_simt(mode, a, w, out, alpha: float = 1.0, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the 32-bit pipes; see csrc/gemm_simt.cu."""
    _cuda(a, w, out)
    M, K = a.shape
    N = out.shape[1]
    rows_w = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or rows_w != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    with _timed("gemm_simt", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_simt(mode, _p(a), dtype_code(a.dtype), a.stride(0), _p(w), dtype_code(w.dtype),
                                   w.stride(0), _p(out), dtype_code(out.dtype), out.stride(0), M, N, K, alpha,
                                   _stream()), "gemm_simt")


_SCRATCH_FLOATS = 16 << 20          # 64 MB of split-K scratch per device, allocated (zeroed) at first use
COUNTER_WORDS = 4096                # its first words are the split-K tile counters (csrc/gemm_tc.cu)
_scratch = {}
_sm_count = {}


def _device_scratch(device):
    key = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    if key not in _scratch:
        # zeroed: the first words are tile counters that every product leaves at zero again
        _scratch[key] = torch.zeros(_SCRATCH_FLOATS, dtype=torch.float32, device=device)
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _scratch[key], _sm_count[key]


def gemm_tc_accepts(mode, a, w, out) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16 operands, K and the row strides
    multiples of 8 elements (TMA needs 16-byte rows), 16-byte aligned bases."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_tiles_fill_the_sms(a, out) -> bool:
    """Whether the product's output tiles (128 features each, all tokens of up to 256 in one) are at least
    three quarters as many as the device has SMs: the tcgen05 kernel then streams the weights with every SM at
    work without cutting K, whatever the number of tokens."""
    _, sms = _device_scratch(a.device)
    return 4 * ((out.shape[1] + 127) // 128) >= 3 * sms


def gemm_tc(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the tensor cores; see csrc/gemm_tc.cu.  Products
    with few tiles split K and use this device's scratch, so calls on one device must not overlap."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    scratch, sms = _device_scratch(a.device)
    with _timed("gemm_tc", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_tc(mode, _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                 out.stride(0), M, N, K, alpha, _p(scratch), scratch.numel(), sms, _p(error_flag),
                                 _stream()), "gemm_tc")


def gemm_cluster_accepts(mode, a, w, out) -> bool:
    """Whether the cluster kernel takes this product: what the tcgen05 kernel takes, and so few output
    tiles that at least two CTAs of a cluster can share each one's K."""
    if not gemm_tc_accepts(mode, a, w, out):
        return False
    _, sms = _device_scratch(a.device)
    return lib().lia_gemm_cluster_splits(mode, a.shape[0], out.shape[1], a.shape[1], sms) >= 2


def gemm_cluster(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the tensor cores with K cut over the CTAs of a
    thread-block cluster, partial sums meeting in distributed shared memory; see csrc/gemm_cluster.cu."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _, sms = _device_scratch(a.device)
    with _timed("gemm_cluster", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_cluster(mode, _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                      out.stride(0), M, N, K, alpha, sms, _p(error_flag), _stream()), "gemm_cluster")


SKINNY_MAX_TOKENS = 32


def gemm_skinny_accepts(mode, a, w, out) -> bool:
    """Whether the few-token kernel takes this product: bfloat16 operands, at most 32 tokens, K and the
    row strides multiples of 8 elements, 16-byte aligned bases (bulk copies and 16-byte loads)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    M, K = a.shape
    return (M <= SKINNY_MAX_TOKENS and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T for M <= 32 tokens: each CTA streams 16 rows of w over
    the whole of K; see csrc/gemm_skinny.cu."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    with _timed("gemm_skinny", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_skinny(mode, _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                     out.stride(0), M, N, K, alpha, _p(error_flag), _stream()), "gemm_skinny")


STREAM_MAX_TOKENS = 16
STREAM_NORM_MAX_K = 4096


def gemm_stream_accepts(mode, a, w, out, norm=False) -> bool:
    """Whether the persistent few-token kernel takes this product: bfloat16 weights, at most 16 tokens whose rows
    fit in shared memory beside a ring of two stages, K and the row strides multiples of 8 elements, 16-byte
    aligned bases.  `norm`: `a` is the 32-bit rows that the kernel norms itself (K at most 4,096)."""
    if w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    if a.dtype != (torch.float32 if norm else torch.bfloat16):
        return False
    M, K = a.shape
    if not (M <= STREAM_MAX_TOKENS and K % 64 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return False
    _, sms = _device_scratch(a.device)
    return lib().lia_gemm_stream_stages(mode, M, out.shape[1], K, 1 if norm else 0, sms) > 0


def gemm_stream(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None, norm_weight=None, eps: float = 0.0,
                stages_cap: int = 0, early_stages: int = 0):
    """out[M, N] (op)= alpha * x[M, K] @ w[N, K]^T for M <= 16 tokens, one persistent CTA per SM with the
    tokens' rows resident in shared memory; see csrc/gemm_stream.cu.  Without `norm_weight`, x = a (bfloat16);
    with it, a is 32-bit and x = RMSNorm(a; norm_weight, eps) rounded to bfloat16, computed inside the kernel."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _, sms = _device_scratch(a.device)
    if norm_weight is None:
        x, ldx, src, ld_src, nw, nw_code = _p(a), a.stride(0), None, 0, None, 0
    else:
        if a.dtype != torch.float32 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_stream with a norm takes 32-bit rows and a weight of K elements")
        x, ldx, src, ld_src, nw, nw_code = None, 0, _p(a), a.stride(0), _p(norm_weight), dtype_code(norm_weight.dtype)
    with _timed("gemm_stream", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_stream(mode, x, ldx, _p(w), w.stride(0), _p(out), dtype_code(out.dtype), out.stride(0),
                                     M, N, K, alpha, src, ld_src, nw, nw_code, eps, sms, stages_cap, early_stages, _p(error_flag),
                                     _stream()), "gemm_stream")


ATTENTION_HEAD_DIM_STEP, ATTENTION_HEAD_DIM_MAX = 16, 256      # what csrc/attention_generic.cu takes


def attention_generic(q, k_pages, v_pages, positions, slots, block_table, out, nq, nkv, d, window, scale,
                      rows=None, error_flag=None, label=None, work_bytes=0):
    """Attention for every token of the batch, or for the tokens whose batch indices `rows` lists (row t of
    `out` is written for token t either way).  A visible key whose block-table entry names no page counts
    for nothing and raises error flag 2."""
    _cuda(q, k_pages, v_pages, positions, slots, block_table, out, rows, error_flag)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("attention: q, cache and out must have one element type")
    n = q.shape[0] if rows is None else rows.shape[0]
    with _timed("attention_generic", label, work_bytes):
        _check(lib().lia_attention_generic(_p(q), _p(k_pages), _p(v_pages), dtype_code(q.dtype), _p(positions),
                                           _p(slots), _p(block_table), block_table.shape[1], _p(rows), _p(out), n, nq,
                                           nkv, d, k_pages.shape[1], int(window or 0), scale, k_pages.shape[0],
                                           _p(error_flag), _stream()),
               "attention_generic")


DECODE_HEAD_DIMS = (32, 64, 128)       # head sizes the tensor-core attention kernels are built for


def attention_decode(q, k_pages, v_pages, rows, positions, slots, block_table, out, partial, nq, nkv, d, window,
                     scale, split_len, n_splits, counters=None, qkv=None, inv_freq=None, rotary_dim=0, write_kv=True,
                     error_flag=None, label=None, work_bytes=0, cluster=False, all_new=False):
    """Split-key decode attention (bfloat16) for the single-token rows of the batch; see
    csrc/attention_decode.cu.  `partial` is 32-bit scratch for the ranges' partial results.
    `split_len` 0: every row cuts its own visible span into `n_splits` ranges.  `counters` (int32, at
    least rows * kv_heads * ceil(group / 16) words, zero before the first call; every call leaves them
    zero) lets the CTA that finishes a token last combine its ranges; without them (or with more than
    128 ranges) a second kernel does.  With `qkv` (32-bit q|k|v rows of the step, at most 16 query heads per
    kv head) `q` may be None: the kernel takes the queries from `qkv`, applies the rotary encoding
    (`inv_freq`, `rotary_dim`; 0: none) and, if `write_kv`, appends each token's key and value to the cache
    itself, so no separate position-encoding kernel runs.  `cluster`: `n_splits` came from
    `attention_decode_cluster_splits`; the ranges of a token then meet in distributed shared memory and neither
    `partial` nor `counters` is used.  `all_new`: the rows may be tokens of this step's prompt portions, so any of
    their keys may have been written by the kernels ahead (otherwise only a row's own key is taken to be of this step,
    and the kernel fetches older tiles before it waits for those kernels)."""
    _cuda(q, k_pages, v_pages, rows, positions, slots, block_table, out, partial, counters, qkv, inv_freq, error_flag)
    if qkv is not None:
        if qkv.dtype != torch.float32 or qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError("attention_decode: qkv must be 32-bit q|k|v rows")
        q = out if q is None else q             # unused by the kernel then; only its element type is checked
    if counters is not None and (counters.dtype != torch.int32
                                 or counters.numel() < rows.shape[0] * nkv * ((nq // nkv + 15) // 16)):
        raise KernelError("attention_decode: counters must be int32, one per row and head group")
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_decode is a bfloat16 kernel")
    with _timed("attention_decode", label, work_bytes):
        _check(lib().lia_attention_decode(_p(q), _p(k_pages), _p(v_pages), _p(rows), rows.shape[0], _p(positions),
                                          _p(slots), _p(block_table), block_table.shape[1], _p(out), _p(partial),
                                          0 if partial is None else partial.numel(), _p(counters), q.shape[0], nq, nkv, d,
                                          k_pages.shape[1], int(window or 0), scale, split_len, n_splits, _p(qkv), _p(inv_freq),
                                          int(rotary_dim), 1 if write_kv else 0, k_pages.shape[0], 1 if cluster else 0, 1 if all_new else 0,
                                          _p(error_flag),
                                          _stream()),
               "attention_decode")


def attention_decode_cluster_splits(d: int, group: int, clusters: int, wanted: int) -> int:
    """Ranges per token (2, 4, 8 or 16, at most `wanted`) with which `attention_decode(..., cluster=True)` can
    serve `clusters` (token, head group) pairs at once; 1: it cannot (one range, or too many clusters for the device)."""
    return int(lib().lia_attention_decode_cluster_splits(d, group, clusters, wanted))


def attention_decode_ctas_per_sm(d: int, group: int) -> int:
    """CTAs of `attention_decode` that one SM holds at once for this head size (0: unknown)."""
    return int(lib().lia_attention_decode_ctas_per_sm(d, group))


def attention_prefill_tokens_per_tile(group: int) -> int:
    """Tokens of a portion that one CTA of the prefill kernel takes (0: group size not supported)."""
    return 64 // group if 1 <= group <= 64 else 0


def attention_prefill(q, k_pages, v_pages, segments, n_segments, n_tiles, slots, block_table, out, nq, nkv, d,
                      window, scale, error_flag=None, label=None, work_flops=0):
    """Tensor-core attention (bfloat16) for the prompt portions listed in `segments`
    ([n_segments, 3] int32: first batch index, first position, count); see csrc/attention_prefill.cu."""
    _cuda(q, k_pages, v_pages, segments, slots, block_table, out, error_flag)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_prefill is a bfloat16 kernel")
    with _timed("attention_prefill", label, 0, work_flops):
        _check(lib().lia_attention_prefill(_p(q), _p(k_pages), _p(v_pages), _p(segments), n_segments, n_tiles,
                                           _p(slots), _p(block_table), block_table.shape[1], _p(out), nq, nkv, d,
                                           k_pages.shape[1], int(window or 0), scale, k_pages.shape[0], _p(error_flag),
                                           _stream()), "attention_prefill")


def attention_prefill_tc_tokens_per_tile(group: int, d: int) -> int:
    """Tokens of a portion that one CTA of the tcgen05 prefill kernel takes (0: it does not take this group
    size or head size)."""
    return int(lib().lia_attention_prefill_tc_tokens_per_tile(group, d))


def attention_prefill_tc(q, k_pages, v_pages, segments, n_segments, n_tiles, slots, block_table, out, nq, nkv, d,
                         window, scale, error_flag=None, label=None, work_flops=0, splits=1, partial=None):
    """Prompt-portion attention on the tcgen05 tensor cores (bfloat16, head size 64 or 128, heads per kv head a
    divisor of 128); see csrc/attention_prefill_tc.cu.  Arguments as `attention_prefill`.  `splits` > 1 cuts every
    CTA's keys into that many ranges that run side by side and are merged by a second kernel; `partial` is their
    32-bit scratch, `attention_prefill_tc_partial_floats` words long."""
    _cuda(q, k_pages, v_pages, segments, slots, block_table, out, error_flag, partial)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_prefill_tc is a bfloat16 kernel")
    splits = int(splits)
    if splits > 1 and (partial is None or partial.dtype != torch.float32
                       or partial.numel() < attention_prefill_tc_partial_floats(q.shape[0], nq, d, splits)):
        raise KernelError("attention_prefill_tc: the ranges need 32-bit scratch of attention_prefill_tc_partial_floats words")
    with _timed("attention_prefill_tc", label, 0, work_flops):
        _check(lib().lia_attention_prefill_tc(_p(q), _p(k_pages), _p(v_pages), _p(segments), n_segments, n_tiles,
                                              _p(slots), _p(block_table), block_table.shape[1], _p(out), nq, nkv, d,
                                              k_pages.shape[1], int(window or 0), scale, k_pages.shape[0], splits,
                                              _p(partial) if splits > 1 else None, q.shape[0], _p(error_flag), _stream()),
               "attention_prefill_tc")


def attention_prefill_tc_partial_floats(n_tokens: int, nq: int, d: int, splits: int) -> int:
    return int(splits) * int(n_tokens) * int(nq) * (int(d) + 2)


_select_scratch = {}


def select_tokens(logits, out, temperature=None, seeds=None, positions=None):
    _cuda(logits, out, temperature, seeds, positions)
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("select_tokens takes 32-bit logits and writes int32 tokens")
    if temperature is not None and (seeds is None or positions is None):
        raise KernelError("select_tokens: temperature needs seeds and positions")
    key = torch.device(logits.device).index or 0
    fn = lib().lia_select_tokens_scratch_floats
    fn.restype = ctypes.c_longlong
    need = int(fn(rows, vocab))
    scratch = _select_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        # zeroed: its head holds the rows' counters, which every call leaves at zero
        scratch = _select_scratch[key] = torch.zeros(max(need, 1 << 18), dtype=torch.float32, device=logits.device)
    with _timed("select_tokens"):
        _check(lib().lia_select_tokens(_p(logits), logits.stride(0), vocab, _p(temperature), _p(seeds),
                                       _p(positions), _p(out), rows, _p(scratch), scratch.numel(), _stream()), "select_tokens")


CANDIDATES_MAX = 32


def select_candidates(logits, k: int, out_values, out_ids, nonfinite, temperature=None, mass=None):
    """The best k logits of every row and their token ids, best first (larger logit, then larger id; minus
    infinity is no candidate, missing ones have id -1): what the host's sampling rule needs of a row when it
    keeps at most k tokens.  `nonfinite` (int32[1]) is increased by the number of NaN and infinite logits.
    With `temperature` (float64 [rows]) also `mass` (float64 [rows, 2]): the row's largest logit and the sum of
    exp((x - largest) / temperature) over the whole row in 64-bit, which bounds what the candidates leave out."""
    _cuda(logits, out_values, out_ids, nonfinite)
    rows, vocab = logits.shape
    if (temperature is None) != (mass is None):
        raise KernelError("select_candidates: temperature and mass come together")
    if temperature is not None:
        _cuda(temperature, mass)
        if temperature.dtype != torch.float64 or mass.dtype != torch.float64 or temperature.numel() != rows \
                or tuple(mass.shape) != (rows, 2) or not mass.is_contiguous() or not temperature.is_contiguous():
            raise KernelError("select_candidates: temperature is float64 [rows], mass float64 [rows, 2]")
    if logits.dtype != torch.float32 or out_values.dtype != torch.float32 or out_ids.dtype != torch.int32:
        raise KernelError("select_candidates takes 32-bit logits and writes float32 values and int32 ids")
    if tuple(out_values.shape) != (rows, k) or tuple(out_ids.shape) != (rows, k) or nonfinite.dtype != torch.int32:
        raise KernelError("select_candidates: outputs must be [rows, k]")
    key = torch.device(logits.device).index or 0
    fn = lib().lia_select_candidates_scratch_floats
    fn.restype = ctypes.c_longlong
    need = int(fn(rows, vocab, k))
    scratch = _select_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        scratch = _select_scratch[key] = torch.zeros(max(need, 1 << 18), dtype=torch.float32, device=logits.device)
    with _timed("select_candidates"):
        _check(lib().lia_select_candidates(_p(logits), logits.stride(0), vocab, rows, k, _p(out_values), _p(out_ids),
                                           _p(nonfinite), _p(temperature), _p(mass), _p(scratch), scratch.numel(),
                                           _stream()), "select_candidates")
