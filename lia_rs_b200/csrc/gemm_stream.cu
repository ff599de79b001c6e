// Matrix product for a handful of tokens (a decode batch of up to 16): out[t, f] = sum_k X[t, k] * W[f, k],
// as a persistent kernel: one CTA per SM, the tokens' rows resident in shared memory, the weights streaming
// through a ring of stages that never stops.
//
// With so few tokens the product is the streaming of W, once, at memory speed.  What was measured on a B200 and
// shapes this kernel:
//   * memory serves requests in the order they were made, at about 7 TB/s over the device.  One SM can take in
//     110 GB/s, so 148 SMs are not needed to fill the pipe, but the pipe must never run empty: what is asked for
//     early (weights, which depend on nothing) is not lost time for what is asked for late (the tokens' rows),
//     it is work done;
//   * an SM issues about 12 million bulk copies a second whatever their size: 2 KB copies (a row of a K chunk)
//     hold a kernel at half the memory's speed, 16 KB copies do not.
//   * mma.sync is slow on this device: an SM completes one m16n8k16 about every 9 cycles.  With the 16 rows of W
//     as the MMA's M and eight tokens as its N, a 32 KB piece of W takes 64 instructions (600 cycles) against
//     1,300 cycles of memory time; with the tokens as M and 8 rows as N it takes twice that and binds the kernel.
//     An instruction's result comes some hundred cycles after its issue, so a warp keeps eight accumulators.
//   * reading both operands from shared memory costs more cycles than the memory time of the weights; a lane's
//     parts of the tokens' rows are the same for every block, so they stay in registers.
// A CTA takes every G-th block of 16 rows of W (G CTAs, one per SM) over the WHOLE of K, so no CTA's result meets
// another's: no scratch memory, no atomic, no second kernel.  Three kinds of warps:
//   * the producer: one thread asks for the next K chunk of the next block as soon as its stage is free.  Where
//     the rows of W are contiguous and a chunk is the whole of K (K up to 2,048), a stage is two copies of
//     eight rows (32 KB each at K = 2,048); else one copy per row.  The two halves of a stage lie 64 bytes
//     apart modulo 128, and the MMA's rows alternate between them, so a quarter-warp's 16-byte loads of two
//     rows fill all 32 banks.  The producer waits for no earlier kernel, so under programmatic dependent launch
//     weights are on their way while the kernel ahead drains; but memory serves in order, so only `early` stages
//     go out before the tokens' rows have been asked for, the rest of the ring right after;
//   * eight MMA warps: they wait for the kernel ahead, then fetch their parts of the tokens' rows ONCE, into
//     registers (or, for a K too long for that, into shared memory), as they are or, for the entry point with a
//     norm, from the 32-bit residual stream through RMSNorm: each CTA norms for itself, which costs no trip
//     to memory more where a kernel of its own costs a launch.  Each warp takes every eighth group of 32 k of a
//     chunk with mma.sync m16n8k16; operands are read 16 bytes per lane, which permutes k inside a group
//     identically for both operands.  At the end of a block a warp leaves its partial sums in one of two
//     buffers and goes on with the next block;
//   * the epilogue warp: adds the eight warps' sums in warp order (the result is the same in every run),
//     applies the epilogue and writes.  For ACCUM it has asked for the old values before the sums are there.
//
// Epilogues as in the other product kernels: STORE out = alpha*acc; ACCUM out += alpha*acc;
// SWIGLU: a block's 16 rows are 8 gate rows and the 8 matching up rows, out = up * gate/(1+exp(-gate)).
#include "common.cuh"

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int ROWS = 16;                 // rows of W per block: the MMA's M
constexpr int HALF_ROWS = 8;             // rows per half of a stage
constexpr int CHUNK_K = 2048;            // most elements of K per stage
constexpr int PAD_BYTES = 64;            // between the halves of a stage, and in the pitch of the tokens' rows
constexpr int MAX_STAGES = 4;
constexpr int MMA_WARPS = 8;
constexpr int PRODUCER_WARP = MMA_WARPS, EPILOGUE_WARP = MMA_WARPS + 1;
constexpr int THREADS = (MMA_WARPS + 2) * 32;
constexpr int FILL_THREADS = (MMA_WARPS + 1) * 32;     // the MMA warps and the epilogue warp bring in the tokens' rows
constexpr int TOKENS = 16;               // most tokens: two tiles of the MMA's N
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr uint64_t WAIT_LIMIT_NS = 4000000000ull;      // four seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded by time, not by polls (a poll may sleep for a while): a kernel ahead of this one under programmatic
// dependent launch may run for many milliseconds; after WAIT_LIMIT_NS the caller gives up and raises the error flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    uint64_t start = 0;
    for (uint32_t i = 0;; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 63u) == 63u) {
            const uint64_t now = global_timer_ns();
            if (start == 0) start = now;
            else if (now - start > WAIT_LIMIT_NS) return false;
        }
    }
}
// `bytes` (a multiple of 16) from global `src` to shared `dst`, both 16-byte aligned.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The MMA warps and the epilogue warp meet here; the producer does not.
__device__ __forceinline__ void fill_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(FILL_THREADS) : "memory"); }


struct Args {
    const __nv_bfloat16* W;
    const __nv_bfloat16* X;          // [M, K] bf16, or null with norm_src
    void* out;
    const float* norm_src;           // [M, K] 32-bit rows to be normed into X's place
    const void* norm_weight;         // [K] bf16 or f32
    int ldw, ldx, ldo, ld_norm, M, N, K;
    int stages, early, chunks, ck;   // ring; stages asked for before the tokens' rows; K chunks per block; elements of K per chunk (a multiple of 64)
    int blocks, x_pitch, stage_bytes, half_bytes;
    int norm, out_bf16;              // norm: 0 none, 1 weight bf16, 2 weight f32
    float alpha, eps;
    int* error_flag;
};

// Row of W in half `half` (0, 1), place `i` (0..7) of block `block` (-1: none).
template <int MODE>
__device__ __forceinline__ int weight_row(const Args& a, int block, int half, int i) {
    if (MODE == GEMM_SWIGLU) {
        const int f = block * HALF_ROWS + i;
        return f < a.N ? (half == 0 ? f : a.N + f) : -1;
    }
    const int f = block * ROWS + half * HALF_ROWS + i;
    return f < a.N ? f : -1;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// RMSNorm of row `src` (K 32-bit elements, K a multiple of 4, at most 128 * VPL) by one warp into `dst` (bf16),
// with the sums taken in the order of the stand-alone kernel (csrc/elementwise.cu), so the rows are the same bits.
template <typename TW, int VPL>
__device__ __forceinline__ void norm_row(const float* __restrict__ src, const TW* __restrict__ weight, uint8_t* dst, int K,
                                         float eps, int lane) {
    const int quads = K >> 2;
    float4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = lane + i * 32;
        v[i] = q < quads ? __ldcg(reinterpret_cast<const float4*>(src) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        sum = fmaf(v[i].x, v[i].x, sum);
        sum = fmaf(v[i].y, v[i].y, sum);
        sum = fmaf(v[i].z, v[i].z, sum);
        sum = fmaf(v[i].w, v[i].w, sum);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sqrtf(sum / (float)K + eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = lane + i * 32;
        if (q < quads) {
            float w0, w1, w2, w3;
            if (sizeof(TW) == 4) {
                const float4 w = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(weight) + 4 * q);
                w0 = w.x; w1 = w.y; w2 = w.z; w3 = w.w;
            } else {
                const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(weight) + 4 * q);
                w0 = __uint_as_float(w.x << 16); w1 = __uint_as_float(w.x & 0xffff0000u);
                w2 = __uint_as_float(w.y << 16); w3 = __uint_as_float(w.y & 0xffff0000u);
            }
            uint2 packed;
            packed.x = pack2(v[i].x * inv * w0 * 1.0f, v[i].y * inv * w1 * 1.0f);
            packed.y = pack2(v[i].z * inv * w2 * 1.0f, v[i].w * inv * w3 * 1.0f);
            *reinterpret_cast<uint2*>(dst + 8 * q) = packed;
        }
    }
}

// The tokens' rows into shared memory (bf16), as they are or through RMSNorm, by the FILL_THREADS threads of
// the MMA warps and the epilogue warp (`fill_tid` 0 .. FILL_THREADS - 1).
template <int X_ROWS>
__device__ __forceinline__ void fill_rows(const Args& a, uint8_t* x_s, int fill_tid, int lane) {
    if (a.norm == 0) {
        const int per_row = a.K >> 3;             // 16-byte pieces per row
        const int pieces = X_ROWS * per_row;
        for (int base = 0; base < pieces; base += FILL_THREADS * 8) {
            uint4 got[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + fill_tid + j * FILL_THREADS;
                const int t = i / per_row, piece = i - t * per_row;
                got[j] = (i < pieces && t < a.M) ? __ldcg(reinterpret_cast<const uint4*>(a.X + (size_t)t * a.ldx) + piece)
                                                 : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = base + fill_tid + j * FILL_THREADS;
                const int t = i / per_row, piece = i - t * per_row;
                if (i < pieces) *reinterpret_cast<uint4*>(x_s + (size_t)t * a.x_pitch + piece * 16) = got[j];
            }
        }
    } else {
        const int fill_warp = fill_tid >> 5;      // 0 .. 8
        for (int t = fill_warp; t < X_ROWS; t += MMA_WARPS + 1) {
            uint8_t* dst = x_s + (size_t)t * a.x_pitch;
            if (t < a.M) {
                const float* src = a.norm_src + (size_t)t * a.ld_norm;
                if (a.norm == 1) {
                    if (a.K <= 2048) norm_row<__nv_bfloat16, 16>(src, (const __nv_bfloat16*)a.norm_weight, dst, a.K, a.eps, lane);
                    else norm_row<__nv_bfloat16, 32>(src, (const __nv_bfloat16*)a.norm_weight, dst, a.K, a.eps, lane);
                } else {
                    if (a.K <= 2048) norm_row<float, 16>(src, (const float*)a.norm_weight, dst, a.K, a.eps, lane);
                    else norm_row<float, 32>(src, (const float*)a.norm_weight, dst, a.K, a.eps, lane);
                }
            } else {
                for (int i = lane; i < (a.K >> 3); i += 32) *reinterpret_cast<uint4*>(dst + i * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
}

// The MMA warps (and, where the tokens' rows go through shared memory, the epilogue warp) tell the producer that the
// tokens' rows have been asked for: it holds the rest of its ring back until then (see the kernel).
template <int COUNT> __device__ __forceinline__ void asked_arrive() { asm volatile("bar.arrive 2, %0;" ::"n"(COUNT) : "memory"); }
template <int COUNT> __device__ __forceinline__ void asked_wait() { asm volatile("bar.sync 2, %0;" ::"n"(COUNT) : "memory"); }
__device__ __forceinline__ void mma_warps_barrier() { asm volatile("bar.sync 3, %0;" ::"n"(MMA_WARPS * 32) : "memory"); }

__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

// Row m of the MMA is row (m >> 1) of half (m & 1) of the stage, that is row (m & 1) * 8 + (m >> 1) of the block.
__device__ __forceinline__ int mma_row_of(int block_row) { return (block_row & 7) * 2 + (block_row >> 3); }

// NT: tiles of eight tokens (1 or 2).
// CHUNKS, PW: 0, 0: the tokens' rows lie in shared memory and every MMA reads its part of them there (any K that is
//     a multiple of 64).  Else K is CHUNKS chunks of 256 * PW elements, a warp takes PW groups of 32 k of every chunk,
//     and a lane keeps its parts of the tokens' rows in registers for the whole kernel, so that shared memory serves
//     the weights alone; the loops over a block then have no condition in them, and a warp has all its loads of four
//     groups in flight before the first of their eight MMAs.
template <int MODE, int NT, int CHUNKS, int PW>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(Args a) {
    constexpr int XG = CHUNKS * PW;
    extern __shared__ __align__(128) uint8_t smem[];
    // dynamic: [stages][stage_bytes] ring, then (XG == 0) the tokens' rows [NT * 8][x_pitch]
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], sums_full[2], sums_empty[2];
    __shared__ float sums[2][MMA_WARPS][ROWS][NT * 8 + 1];
    __shared__ float squares[MMA_WARPS][TOKENS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* x_s = smem + (size_t)a.stages * a.stage_bytes;
    constexpr int X_ROWS = NT * 8;
    constexpr int ASKED = XG > 0 ? (MMA_WARPS + 1) * 32 : THREADS;      // the MMA warps (and the epilogue warp) and the producer warp
    constexpr bool NORM_IN_REGISTERS = XG > 0 && XG * NT <= 16;

    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), MMA_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sums_full[i]), MMA_WARPS);
            mbar_init(smem_u32(&sums_empty[i]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    const int grid = gridDim.x;

    if (warp == PRODUCER_WARP) {
        // ---- producer: lane 0 asks; the weights depend on no earlier kernel.  Memory serves requests in order, so
        //      what is asked for before the tokens' rows delays them: `early` stages go out at once (enough to keep
        //      memory at work until the kernel ahead has finished), the rest when the rows have been asked for.
        //      (The whole warp walks the loop, since a named barrier counts warps.) ----
        bool asked = false, ok = true;
        int it = 0, st = 0;
        uint32_t phase = 0;                                           // of the stage's use: counted along, not divided out
        const bool whole_rows = a.chunks == 1 && a.ldw == a.K;       // a half of a stage is one piece of memory
        for (int block = blockIdx.x; block < a.blocks && ok; block += grid) {
            for (int c = 0; c < a.chunks; ++c, ++it, st = (st + 1 == a.stages ? 0 : st + 1), phase ^= (st == 0 ? 1u : 0u)) {
                if (it == a.early && !asked) { __syncwarp(); asked_wait<ASKED>(); asked = true; }
                if (it >= a.stages) {
                    if (lane == 0) ok = mbar_wait(smem_u32(&empty_bar[st]), phase ^ 1u);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                if (lane == 0) {
                    const uint32_t full = smem_u32(&full_bar[st]);
                    const int k0 = c * a.ck;
                    const uint32_t bytes = (uint32_t)min(a.ck, a.K - k0) * 2u;
                    int rows = 0;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < HALF_ROWS; ++i) rows += weight_row<MODE>(a, block, h, i) >= 0;
                    mbar_expect_tx(full, bytes * (uint32_t)rows);
                    const uint32_t dst = smem_base + (uint32_t)(st * a.stage_bytes);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int first = weight_row<MODE>(a, block, h, 0), last = weight_row<MODE>(a, block, h, HALF_ROWS - 1);
                        if (whole_rows && last >= 0) {
                            bulk_copy(dst + (uint32_t)(h * a.half_bytes), a.W + (size_t)first * a.ldw, bytes * HALF_ROWS, full);
                        } else {
#pragma unroll
                            for (int i = 0; i < HALF_ROWS; ++i) {
                                const int row = weight_row<MODE>(a, block, h, i);
                                if (row >= 0)
                                    bulk_copy(dst + (uint32_t)(h * a.half_bytes + i * a.ck * 2), a.W + (size_t)row * a.ldw + k0, bytes, full);
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0 && a.error_flag) atomicExch(a.error_flag, 3);
        __syncwarp();
        if (!asked) asked_wait<ASKED>();
    } else if (warp == EPILOGUE_WARP) {
        pdl_wait();                                   // ACCUM's old values come from the kernels ahead
        if (XG == 0) {
            asked_arrive<ASKED>();
            fill_rows<X_ROWS>(a, x_s, (int)threadIdx.x - 32, lane);
            fill_barrier();
        }
        // ---- epilogue: a block's outputs are 16 rows (SWIGLU: 8 features) x NT * 8 tokens ----
        bool ok = true;
        int ui = 0;
        for (int block = blockIdx.x; block < a.blocks; block += grid, ++ui) {
            const int buf = ui & 1;
            constexpr int PER_LANE = (MODE == GEMM_SWIGLU ? HALF_ROWS : ROWS) * NT * 8 / 32;
            float old[PER_LANE];
            if (MODE == GEMM_ACCUM) {
#pragma unroll
                for (int j = 0; j < PER_LANE; ++j) {
                    const int i = lane + j * 32, token = i >> 4, f = block * ROWS + (i & 15);
                    old[j] = (token < a.M && f < a.N) ? __ldcg(reinterpret_cast<const float*>(a.out) + (size_t)token * a.ldo + f) : 0.f;
                }
            }
            if (!mbar_wait(smem_u32(&sums_full[buf]), (uint32_t)(ui >> 1) & 1u)) { ok = false; break; }
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j) {
                const int i = lane + j * 32;
                if (MODE == GEMM_SWIGLU) {
                    // row 2q of the MMA is gate row q of the block, row 2q + 1 its up row
                    const int token = i >> 3, q = i & 7, f = block * HALF_ROWS + q;
                    float gate = 0.f, up = 0.f;
#pragma unroll
                    for (int w = 0; w < MMA_WARPS; ++w) {
                        gate += sums[buf][w][2 * q][token];
                        up += sums[buf][w][2 * q + 1][token];
                    }
                    if (token < a.M && f < a.N) {
                        const float value = up * (gate / (1.0f + __expf(-gate)));
                        if (a.out_bf16) reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)token * a.ldo + f] = __float2bfloat16_rn(value);
                        else reinterpret_cast<float*>(a.out)[(size_t)token * a.ldo + f] = value;
                    }
                } else {
                    const int token = i >> 4, r = i & 15, f = block * ROWS + r, m = mma_row_of(r);
                    float total = 0.f;
#pragma unroll
                    for (int w = 0; w < MMA_WARPS; ++w) total += sums[buf][w][m][token];
                    if (token < a.M && f < a.N) {
                        const float value = MODE == GEMM_STORE ? a.alpha * total : old[j] + a.alpha * total;
                        if (a.out_bf16) reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)token * a.ldo + f] = __float2bfloat16_rn(value);
                        else reinterpret_cast<float*>(a.out)[(size_t)token * a.ldo + f] = value;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sums_empty[buf]));
        }
        if (!ok && lane == 0 && a.error_flag) atomicExch(a.error_flag, 3);
    } else {
        // ---- eight MMA warps: each takes every eighth group of 32 k ----
        const int g = lane >> 2, t = lane & 3;
        // rows g and g + 8 of the MMA: rows (g >> 1) and (g >> 1) + 4 of half (g & 1) of the stage
        const uint32_t w_offset = (uint32_t)((g & 1) * a.half_bytes + (g >> 1) * a.ck * 2 + t * 16);
        const uint32_t w_high = (uint32_t)(4 * a.ck * 2);
        const int groups_per_chunk = a.ck >> 5;
        constexpr int XR = XG > 0 ? XG : 1, PWR = PW > 0 ? PW : 1;
        uint4 xf[XR][NT];                              // [chunk * PW + group][tile]: token 8 * tile + g, this lane's 8 k of the group
        (void)xf;
        if (XG > 0) {
            // ---- this lane's parts of the tokens' rows: every load in flight at once, one trip to L2 ----
            const bool normed = a.norm != 0;
            uint4 nw[NORM_IN_REGISTERS ? XR : 1][2];                 // the norm's weights for this lane's k: they wait for no one
            (void)nw;
            if (NORM_IN_REGISTERS && normed) {
#pragma unroll
                for (int r = 0; r < XR; ++r) {
                    {
                        const int k = (r / PWR) * (PWR * 256) + (warp + (r % PWR) * MMA_WARPS) * 32 + t * 8;
                        if (a.norm == 1) nw[r][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.norm_weight) + k);
                        else {
                            nw[r][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.norm_weight) + k);
                            nw[r][1] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.norm_weight) + k + 4);
                        }
                    }
                }
            }
            pdl_wait();                               // the tokens' rows come from the kernel ahead
            if (!(NORM_IN_REGISTERS && normed)) {
#pragma unroll
                for (int r = 0; r < XR; ++r) {
                    {
                        const int k = (r / PWR) * (PWR * 256) + (warp + (r % PWR) * MMA_WARPS) * 32 + t * 8;
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            const int token = n * 8 + g;
                            xf[r][n] = token < a.M ? __ldcg(reinterpret_cast<const uint4*>(a.X + (size_t)token * a.ldx + k)) : make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                }
                asked_arrive<ASKED>();
            } else if (NORM_IN_REGISTERS) {
                // RMSNorm here: the 32-bit rows come in once; a token's sum of squares is added up over the lanes that
                // share it (t), then over the warps in warp order through shared memory.
                float4 raw[XR][NT][2];
#pragma unroll
                for (int r = 0; r < XR; ++r) {
                    {
                        const int k = (r / PWR) * (PWR * 256) + (warp + (r % PWR) * MMA_WARPS) * 32 + t * 8;
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            const int token = n * 8 + g;
                            const float4* src = reinterpret_cast<const float4*>(a.norm_src + (size_t)token * a.ld_norm + k);
                            raw[r][n][0] = token < a.M ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                            raw[r][n][1] = token < a.M ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
                asked_arrive<ASKED>();
                float sq[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) sq[n] = 0.f;
#pragma unroll
                for (int r = 0; r < XR; ++r) {
                    {
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                sq[n] = fmaf(raw[r][n][j].x, raw[r][n][j].x, sq[n]); sq[n] = fmaf(raw[r][n][j].y, raw[r][n][j].y, sq[n]);
                                sq[n] = fmaf(raw[r][n][j].z, raw[r][n][j].z, sq[n]); sq[n] = fmaf(raw[r][n][j].w, raw[r][n][j].w, sq[n]);
                            }
                    }
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    sq[n] += __shfl_xor_sync(0xffffffffu, sq[n], 1);
                    sq[n] += __shfl_xor_sync(0xffffffffu, sq[n], 2);
                    if (t == 0) squares[warp][n * 8 + g] = sq[n];
                }
                mma_warps_barrier();
                float inv[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float total = 0.f;
#pragma unroll
                    for (int w = 0; w < MMA_WARPS; ++w) total += squares[w][n * 8 + g];
                    inv[n] = 1.0f / sqrtf(total / (float)a.K + a.eps);
                }
#pragma unroll
                for (int r = 0; r < XR; ++r) {
                    {
                        float w[8];
                        if (a.norm == 1) {
                            w[0] = bf16_lo(nw[r][0].x); w[1] = bf16_hi(nw[r][0].x); w[2] = bf16_lo(nw[r][0].y); w[3] = bf16_hi(nw[r][0].y);
                            w[4] = bf16_lo(nw[r][0].z); w[5] = bf16_hi(nw[r][0].z); w[6] = bf16_lo(nw[r][0].w); w[7] = bf16_hi(nw[r][0].w);
                        } else {
                            w[0] = __uint_as_float(nw[r][0].x); w[1] = __uint_as_float(nw[r][0].y); w[2] = __uint_as_float(nw[r][0].z); w[3] = __uint_as_float(nw[r][0].w);
                            w[4] = __uint_as_float(nw[r][1].x); w[5] = __uint_as_float(nw[r][1].y); w[6] = __uint_as_float(nw[r][1].z); w[7] = __uint_as_float(nw[r][1].w);
                        }
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            xf[r][n].x = pack2(raw[r][n][0].x * inv[n] * w[0], raw[r][n][0].y * inv[n] * w[1]);
                            xf[r][n].y = pack2(raw[r][n][0].z * inv[n] * w[2], raw[r][n][0].w * inv[n] * w[3]);
                            xf[r][n].z = pack2(raw[r][n][1].x * inv[n] * w[4], raw[r][n][1].y * inv[n] * w[5]);
                            xf[r][n].w = pack2(raw[r][n][1].z * inv[n] * w[6], raw[r][n][1].w * inv[n] * w[7]);
                        }
                    }
                }
            }
        } else {
            pdl_wait();
            asked_arrive<ASKED>();
            fill_rows<X_ROWS>(a, x_s, (int)threadIdx.x, lane);
            fill_barrier();
        }
        const uint8_t* x_base = x_s + (size_t)g * a.x_pitch + t * 16;       // XG == 0: token g's part for this lane
        (void)x_base;

        bool ok = true;
        int it = 0, ui = 0, st = 0;
        uint32_t phase = 0;                                           // of the stage's use: counted along, not divided out
        for (int block = blockIdx.x; block < a.blocks && ok; block += grid, ++ui) {
            // Eight accumulators per tile of tokens: an mma.sync takes some hundred cycles from issue to result, so a
            // warp keeps eight of them in flight, none waiting for another (four groups of 32 k, two instructions each).
            float part[4][2][NT][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int n = 0; n < NT; ++n) part[i][j][n][0] = part[i][j][n][1] = part[i][j][n][2] = part[i][j][n][3] = 0.f;
            if (XG > 0) {
#pragma unroll
                for (int c = 0; c < (CHUNKS > 0 ? CHUNKS : 1); ++c) {
                    if (!mbar_wait(smem_u32(&full_bar[st]), phase)) { ok = false; break; }
                    const uint8_t* stage = smem + (size_t)st * a.stage_bytes + w_offset + warp * 64;
#pragma unroll
                    for (int i0 = 0; i0 < PWR; i0 += 4) {
                        uint4 lo[4], hi[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (i0 + i < PWR) {
                                lo[i] = *reinterpret_cast<const uint4*>(stage + (i0 + i) * (MMA_WARPS * 64));
                                hi[i] = *reinterpret_cast<const uint4*>(stage + (i0 + i) * (MMA_WARPS * 64) + w_high);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (i0 + i < PWR) {
#pragma unroll
                                for (int n = 0; n < NT; ++n) {
                                    mma_bf16(part[i][0][n], lo[i].x, hi[i].x, lo[i].y, hi[i].y, xf[c * PWR + i0 + i][n].x, xf[c * PWR + i0 + i][n].y);
                                    mma_bf16(part[i][1][n], lo[i].z, hi[i].z, lo[i].w, hi[i].w, xf[c * PWR + i0 + i][n].z, xf[c * PWR + i0 + i][n].w);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[st]));
                    ++it;
                    if (++st == a.stages) { st = 0; phase ^= 1u; }
                }
            } else {
                for (int c = 0; c < a.chunks; ++c, ++it, st = (st + 1 == a.stages ? 0 : st + 1), phase ^= (st == 0 ? 1u : 0u)) {
                    const int k0 = c * a.ck;
                    const int groups = min(groups_per_chunk, (a.K - k0) >> 5);      // K is a multiple of 64: whole groups
                    if (!mbar_wait(smem_u32(&full_bar[st]), phase)) { ok = false; break; }
                    const uint8_t* stage = smem + (size_t)st * a.stage_bytes + w_offset;
                    const uint8_t* xk = x_base + (size_t)k0 * 2;
                    for (int base = warp; base < groups; base += 4 * MMA_WARPS) {
                        uint4 lo[4], hi[4], x[4][NT];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int group = base + i * MMA_WARPS;              // the same for the whole warp
                            if (group < groups) {
                                lo[i] = *reinterpret_cast<const uint4*>(stage + group * 64);
                                hi[i] = *reinterpret_cast<const uint4*>(stage + group * 64 + w_high);
#pragma unroll
                                for (int n = 0; n < NT; ++n) x[i][n] = *reinterpret_cast<const uint4*>(xk + (size_t)n * 8 * a.x_pitch + group * 64);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (base + i * MMA_WARPS < groups) {
#pragma unroll
                                for (int n = 0; n < NT; ++n) {
                                    mma_bf16(part[i][0][n], lo[i].x, hi[i].x, lo[i].y, hi[i].y, x[i][n].x, x[i][n].y);
                                    mma_bf16(part[i][1][n], lo[i].z, hi[i].z, lo[i].w, hi[i].w, x[i][n].z, x[i][n].w);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[st]));
                }
            }
            if (!ok) break;
            const int buf = ui & 1;
            if (ui >= 2) {
                bool free_now = true;
                if (lane == 0) free_now = mbar_wait(smem_u32(&sums_empty[buf]), ((uint32_t)(ui >> 1) & 1u) ^ 1u);
                free_now = __shfl_sync(0xffffffffu, free_now, 0);
                if (!free_now) { ok = false; break; }
            }
            // c0, c1: row g of the MMA, tokens 2t, 2t+1 of the tile; c2, c3: row g + 8
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                float acc[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    acc[e] = ((part[0][0][n][e] + part[0][1][n][e]) + (part[1][0][n][e] + part[1][1][n][e])) +
                             ((part[2][0][n][e] + part[2][1][n][e]) + (part[3][0][n][e] + part[3][1][n][e]));
                sums[buf][warp][g][n * 8 + 2 * t] = acc[0];
                sums[buf][warp][g][n * 8 + 2 * t + 1] = acc[1];
                sums[buf][warp][g + 8][n * 8 + 2 * t] = acc[2];
                sums[buf][warp][g + 8][n * 8 + 2 * t + 1] = acc[3];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sums_full[buf]));
        }
        if (!ok && lane == 0 && a.error_flag) atomicExch(a.error_flag, 3);
    }
    // Nobody leaves while a copy may still be in flight into this CTA's shared memory: in a run without a
    // failed wait every stage asked for has been waited for by the MMA warps; after a failure thread 0 waits,
    // with a limit, for the stages that were asked for last.
    __syncthreads();
    if (threadIdx.x == 0 && a.error_flag && *reinterpret_cast<volatile int*>(a.error_flag) == 3) {
        int mine = 0;
        for (int block = blockIdx.x; block < a.blocks; block += grid) ++mine;
        const int total = mine * a.chunks;
        for (int it = total > a.stages ? total - a.stages : 0; it < total; ++it)
            mbar_wait(smem_u32(&full_bar[it % a.stages]), (uint32_t)(it / a.stages) & 1u);
    }
}

int x_pitch_of(int K) { return (K * 2 + 127) / 128 * 128 + PAD_BYTES; }

// How K is cut: chunks of at most CHUNK_K elements, each a multiple of 64.
void chunking(int K, int* chunks, int* ck) {
    *chunks = (K + CHUNK_K - 1) / CHUNK_K;
    *ck = ((K + *chunks - 1) / *chunks + 63) / 64 * 64;
}

int stage_bytes_of(int ck) { return (2 * HALF_ROWS * ck * 2 + PAD_BYTES + 127) / 128 * 128; }

// The register form of the kernel that takes M tokens of K elements (0, 0: none, the tokens' rows go through shared
// memory): K one chunk of 1,024 or 2,048 elements or two to four chunks of 2,048, few enough groups for a lane's
// registers (32 of them per tile of tokens; with a norm, where the 32-bit rows pass through registers, 16).
void register_form(int M, int K, bool with_norm, int* chunks, int* pw) {
    *chunks = 0; *pw = 0;
    int c, w;
    if (K == 1024) { c = 1; w = 4; }
    else if (K == 2048 || K == 4096 || K == 6144 || K == 8192) { c = K / 2048; w = 8; }
    else return;
    const int tiles = M <= 8 ? 1 : 2;
    if (c * w * tiles > (with_norm ? 16 : 32)) return;
    *chunks = c; *pw = w;
}

// Stages of the ring that fit beside the tokens' rows (0: the rows do not fit with two stages).
int stages_that_fit(int x_rows, int K, int chunks, int ck, long long blocks_per_cta) {
    const int static_bytes = 2 * MMA_WARPS * ROWS * (TOKENS + 1) * 4 + MMA_WARPS * TOKENS * 4 + (2 * MAX_STAGES + 4) * 8 + 1024;
    const int left = SMEM_LIMIT - static_bytes - x_rows * x_pitch_of(K);
    int stages = left / stage_bytes_of(ck);
    if (stages < 2) return 0;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const long long needed = (long long)chunks * blocks_per_cta;       // no more stages than the CTA ever fills
    if (needed < stages) stages = (int)(needed < 1 ? 1 : needed);
    return stages;
}

template <int MODE, int NT, int CHUNKS, int PW>
int launch(const Args& a, int ctas, cudaStream_t stream) {
    const size_t smem = (size_t)a.stages * a.stage_bytes + (CHUNKS > 0 ? 0 : (size_t)NT * 8 * a.x_pitch);
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<MODE, NT, CHUNKS, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = smem;
    }
    return lia_launch(gemm_stream_kernel<MODE, NT, CHUNKS, PW>, dim3(ctas), dim3(THREADS), smem, stream, a);
}

template <int MODE>
int launch_form(const Args& a, int chunks, int pw, int ctas, cudaStream_t stream) {
    const int form = chunks * 100 + pw;
    if (a.M <= 8) {
        switch (form) {
            case 104: return launch<MODE, 1, 1, 4>(a, ctas, stream);
            case 108: return launch<MODE, 1, 1, 8>(a, ctas, stream);
            case 208: return launch<MODE, 1, 2, 8>(a, ctas, stream);
            case 308: return launch<MODE, 1, 3, 8>(a, ctas, stream);
            case 408: return launch<MODE, 1, 4, 8>(a, ctas, stream);
            default: return launch<MODE, 1, 0, 0>(a, ctas, stream);
        }
    }
    switch (form) {
        case 104: return launch<MODE, 2, 1, 4>(a, ctas, stream);
        case 108: return launch<MODE, 2, 1, 8>(a, ctas, stream);
        case 208: return launch<MODE, 2, 2, 8>(a, ctas, stream);
        default: return launch<MODE, 2, 0, 0>(a, ctas, stream);
    }
}

// (stages, register form) for a product, stages 0 if the kernel does not take it.
void plan(int mode, int M, int N, int K, bool with_norm, int sms, int* stages, int* form_chunks, int* form_pw) {
    *stages = 0; *form_chunks = 0; *form_pw = 0;
    if (M <= 0 || M > TOKENS || K <= 0 || K % 64 || N <= 0 || sms <= 0) return;
    const long long blocks = mode == GEMM_SWIGLU ? (N + HALF_ROWS - 1) / HALF_ROWS : (N + ROWS - 1) / ROWS;
    int chunks, ck;
    chunking(K, &chunks, &ck);
    register_form(M, K, with_norm, form_chunks, form_pw);
    if (!*form_chunks && with_norm && K > 4096) return;       // the norm through shared memory: a warp holds a row of at most 4,096
    *stages = stages_that_fit(*form_chunks ? 0 : (M <= 8 ? 8 : 16), K, chunks, ck, (blocks + sms - 1) / sms);
}
}  // namespace


// Whether (and with how many stages) the kernel takes M tokens of K elements on a device of `sms` SMs for a
// product of N features: 0 when K is not a multiple of 64, when the tokens' rows leave no room for a ring of two
// stages, or with a norm when K is beyond the 4,096 elements a warp holds of a row.
LIA_EXPORT int lia_gemm_stream_stages(int mode, int M, int N, int K, int with_norm, int sms) {
    int stages, chunks, pw;
    plan(mode, M, N, K, with_norm != 0, sms, &stages, &chunks, &pw);
    return stages;
}

// X [M, K] bf16 (row stride ldx), M <= 16, or (X null) norm_src [M, K] 32-bit (row stride ld_norm) with the
// norm's weight [K] (bf16: norm_weight_dtype LIA_BF16, else LIA_F32) and eps: the rows are then RMS-normed in
// the kernel.  W [N, K] (SWIGLU: [2N, K], gate rows then up rows) bf16 (row stride ldw); out [M, N] f32 or bf16
// (row stride ldo).  Refuses K that is not a multiple of 64, ldw or ldx that are not multiples of 8 elements,
// pointers that are not 16-byte aligned (bulk copies and 16-byte loads need both), and sizes whose rows do not
// fit in shared memory beside a ring (ask lia_gemm_stream_stages first).  `stages_cap` > 0 limits the ring;
// `early_stages` > 0 sets how many stages the producer asks for before the tokens' rows have been asked for (default 2).
LIA_EXPORT int lia_gemm_stream(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                               int ldo, int M, int N, int K, float alpha, const float* norm_src, int ld_norm,
                               const void* norm_weight, int norm_weight_dtype, float eps, int sms, int stages_cap,
                               int early_stages, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (M > TOKENS || K <= 0 || K % 64 || ldw % 8 || ldw < K || ldo < N || sms <= 0) return LIA_ERR_SIZE;
    if ((uintptr_t)W & 15u) return LIA_ERR_ALIGN;
    if (norm_src) {
        if (!norm_weight || ld_norm < K || ld_norm % 4 || K > 4096) return LIA_ERR_SIZE;
        if (((uintptr_t)norm_src & 15u) || ((uintptr_t)norm_weight & 15u)) return LIA_ERR_ALIGN;
        if (norm_weight_dtype != LIA_BF16 && norm_weight_dtype != LIA_F32) return LIA_ERR_DTYPE;
    } else {
        if (!X || ldx % 8 || ldx < K) return LIA_ERR_SIZE;
        if ((uintptr_t)X & 15u) return LIA_ERR_ALIGN;
    }
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    Args a;
    a.W = (const __nv_bfloat16*)W; a.X = (const __nv_bfloat16*)X; a.out = out;
    a.norm_src = norm_src; a.norm_weight = norm_weight; a.ld_norm = ld_norm; a.eps = eps;
    a.norm = !norm_src ? 0 : (norm_weight_dtype == LIA_BF16 ? 1 : 2);
    a.out_bf16 = out_dtype == LIA_BF16;
    a.ldw = ldw; a.ldx = ldx; a.ldo = ldo; a.M = M; a.N = N; a.K = K; a.alpha = alpha; a.error_flag = error_flag;
    chunking(K, &a.chunks, &a.ck);
    const long long blocks = mode == GEMM_SWIGLU ? (N + HALF_ROWS - 1) / HALF_ROWS : (N + ROWS - 1) / ROWS;
    if (blocks > 2147483647LL) return LIA_ERR_SIZE;
    a.blocks = (int)blocks;
    a.x_pitch = x_pitch_of(K);
    a.stage_bytes = stage_bytes_of(a.ck);
    a.half_bytes = HALF_ROWS * a.ck * 2 + PAD_BYTES;
    const int ctas = blocks < sms ? (int)blocks : sms;
    int form_chunks, form_pw;
    plan(mode, M, N, K, norm_src != nullptr, sms, &a.stages, &form_chunks, &form_pw);
    if (a.stages <= 0) return LIA_ERR_SIZE;
    if (stages_cap > 0 && a.stages > stages_cap) a.stages = stages_cap;
    a.early = early_stages > 0 ? early_stages : 2;
    if (mode == GEMM_STORE) return launch_form<GEMM_STORE>(a, form_chunks, form_pw, ctas, stream);
    if (mode == GEMM_ACCUM) return launch_form<GEMM_ACCUM>(a, form_chunks, form_pw, ctas, stream);
    return launch_form<GEMM_SWIGLU>(a, form_chunks, form_pw, ctas, stream);
}
