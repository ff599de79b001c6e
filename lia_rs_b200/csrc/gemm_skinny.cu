// Matrix product for a handful of tokens (a decode batch of up to 32): out[t, f] = sum_k X[t, k] * W[f, k].
//
// With so few tokens the product is the streaming of W, once, at memory speed; everything here serves
// that.  A CTA owns 16 rows of W over the WHOLE of K, so no CTA's result has to meet another's: there
// is no scratch memory, no atomic and no second kernel.  Its rows come in as bulk asynchronous copies
// (cp.async.bulk, one per row and K chunk, completion counted on an mbarrier) that one thread issues
// as fast as it can into a ring of shared-memory stages; with K up to six chunks long the whole working
// set of the CTA is in flight at once.  The kernel is launched with programmatic dependent launch and
// asks for its weights BEFORE it waits for the kernel ahead of it, so the copies run while that kernel
// drains: weights depend on nothing.
//
// Eight warps share each chunk of K.  A warp multiplies with mma.sync m16n8k16 (bf16 in, 32-bit
// accumulate): the 16 rows of W are the MMA's M, eight tokens its N.  Operands are read 16 bytes per
// lane: lane (g, t) takes k = 8t .. 8t+7 of W rows g and g+8 from shared memory and of token g from X
// (X is tiny and lies in L2).  Feeding these to the MMA permutes k inside each group of 32, identically
// for both operands, which a sum over k does not notice.  At the end the warps' partial sums are added
// through shared memory in warp order, so the result is the same in every run.
//
// Epilogues as in the tcgen05 kernel: STORE out = alpha*acc; ACCUM out += alpha*acc;
// SWIGLU: the CTA's 16 rows are 8 gate rows and the 8 matching up rows, out = up * gate/(1+exp(-gate)).
#include "common.cuh"

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int ROWS = 16;                 // rows of W per CTA
constexpr int CHUNK_K = 1024;            // elements of K per stage
constexpr int PAD_BYTES = 64;            // row pitch = chunk bytes + 64: 16-byte reads of 8 rows hit 8 bank groups
constexpr int PITCH = CHUNK_K * 2 + PAD_BYTES;
constexpr int STAGE_BYTES = ROWS * PITCH;
constexpr int MAX_STAGES = 6;
constexpr int COMPUTE_WARPS = 8;
constexpr int THREADS = (COMPUTE_WARPS + 1) * 32;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
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

struct Args {
    const __nv_bfloat16* W;
    const __nv_bfloat16* X;
    void* out;
    int ldw, ldx, ldo, M, N, K, stages, chunks;
    float alpha;
    int* error_flag;
};

// Row of W that the CTA's row r stands for (-1: none).
template <int MODE>
__device__ __forceinline__ int weight_row(const Args& a, int block, int r) {
    if (MODE == GEMM_SWIGLU) {
        const int f = block * 8 + (r & 7);
        return f < a.N ? (r < 8 ? f : a.N + f) : -1;
    }
    const int f = block * ROWS + r;
    return f < a.N ? f : -1;
}

template <int MODE, typename TO, int NT>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(Args a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
    __shared__ float sums[COMPUTE_WARPS][ROWS][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), COMPUTE_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == COMPUTE_WARPS) {
        // ---- producer: the weights depend on no earlier kernel, so nothing is waited for ----
        if (lane == 0) {
            bool ok = true;
            for (int c = 0; c < a.chunks && ok; ++c) {
                const int st = c % a.stages;
                if (c >= a.stages && !mbar_wait(smem_u32(&empty_bar[st]), ((uint32_t)(c / a.stages) & 1u) ^ 1u)) { ok = false; break; }
                const int k0 = c * CHUNK_K;
                const uint32_t bytes = (uint32_t)min(CHUNK_K, a.K - k0) * 2u;
                int rows = 0;
                for (int r = 0; r < ROWS; ++r) rows += weight_row<MODE>(a, blockIdx.x, r) >= 0;
                const uint32_t full = smem_u32(&full_bar[st]);
                mbar_expect_tx(full, bytes * (uint32_t)rows);
                for (int r = 0; r < ROWS; ++r) {
                    const int row = weight_row<MODE>(a, blockIdx.x, r);
                    if (row >= 0)
                        bulk_copy(smem_base + (uint32_t)(st * STAGE_BYTES + r * PITCH), a.W + (size_t)row * a.ldw + k0, bytes, full);
                }
            }
            if (!ok && a.error_flag) atomicExch(a.error_flag, 3);
        }
        pdl_wait();                                   // this warp's threads take part in the epilogue below
    } else {
        // ---- eight warps: each takes every eighth group of 32 k ----
        const int g = lane >> 2, t = lane & 3;
        // one accumulator per group of 32 k that the warp takes in a chunk: the tensor-core instructions of a
        // chunk then do not wait for one another
        constexpr int CHAINS = CHUNK_K / 32 / COMPUTE_WARPS;
        float part[CHAINS][NT][4];
#pragma unroll
        for (int i = 0; i < CHAINS; ++i)
#pragma unroll
            for (int n = 0; n < NT; ++n) part[i][n][0] = part[i][n][1] = part[i][n][2] = part[i][n][3] = 0.f;
        const bool row_lo = weight_row<MODE>(a, blockIdx.x, g) >= 0, row_hi = weight_row<MODE>(a, blockIdx.x, g + 8) >= 0;
        pdl_wait();                                   // X comes from the kernel ahead
        bool ok = true;
        for (int c = 0; c < a.chunks; ++c) {
            const int st = c % a.stages;
            const int k0 = c * CHUNK_K;
            const int groups = (min(CHUNK_K, a.K - k0) + 31) / 32;
            // this warp's X fragments of the chunk: asked for before the weights are waited for
            constexpr int PER_WARP = CHUNK_K / 32 / COMPUTE_WARPS;       // 4 groups of 32 k
            uint4 xf[PER_WARP][NT];
#pragma unroll
            for (int i = 0; i < PER_WARP; ++i) {
                const int k = k0 + (warp + i * COMPUTE_WARPS) * 32 + t * 8;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const int token = n * 8 + g;
                    if (warp + i * COMPUTE_WARPS < groups && k < a.K && token < a.M)
                        xf[i][n] = __ldcg(reinterpret_cast<const uint4*>(a.X + (size_t)token * a.ldx + k));
                    else
                        xf[i][n] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (!mbar_wait(smem_u32(&full_bar[st]), (uint32_t)(c / a.stages) & 1u)) { ok = false; break; }
            const uint8_t* stage = smem + st * STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < PER_WARP; ++i) {
                const int group = warp + i * COMPUTE_WARPS;
                const int k = k0 + group * 32 + t * 8;
                if (group < groups) {
                    uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
                    if (k < a.K) {
                        const int offset = (group * 32 + t * 8) * 2;
                        if (row_lo) lo = *reinterpret_cast<const uint4*>(stage + g * PITCH + offset);
                        if (row_hi) hi = *reinterpret_cast<const uint4*>(stage + (g + 8) * PITCH + offset);
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        mma_bf16(part[i][n], lo.x, hi.x, lo.y, hi.y, xf[i][n].x, xf[i][n].y);
                        mma_bf16(part[i][n], lo.z, hi.z, lo.w, hi.w, xf[i][n].z, xf[i][n].w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && c + a.stages < a.chunks) mbar_arrive(smem_u32(&empty_bar[st]));
        }
        if (!ok && lane == 0 && a.error_flag) atomicExch(a.error_flag, 3);
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float total = part[0][n][e];
#pragma unroll
                for (int i = 1; i < CHAINS; ++i) total += part[i][n][e];
                acc[n][e] = total;
            }
        // c0, c1: row g, tokens 2t, 2t+1; c2, c3: row g+8
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            sums[warp][g][n * 8 + 2 * t] = acc[n][0];
            sums[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
            sums[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
            sums[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
        }
    }
    __syncthreads();
    TO* out = reinterpret_cast<TO*>(a.out);
    if (MODE == GEMM_SWIGLU) {
        for (int i = threadIdx.x; i < 8 * NT * 8; i += THREADS) {
            const int token = i >> 3, r = i & 7;
            const int f = blockIdx.x * 8 + r;
            if (token >= a.M || f >= a.N) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < COMPUTE_WARPS; ++w) {
                gate += sums[w][r][token];
                up += sums[w][r + 8][token];
            }
            out[(size_t)token * a.ldo + f] = from_float<TO>(up * (gate / (1.0f + __expf(-gate))));
        }
    } else {
        for (int i = threadIdx.x; i < ROWS * NT * 8; i += THREADS) {
            const int token = i >> 4, r = i & 15;
            const int f = blockIdx.x * ROWS + r;
            if (token >= a.M || f >= a.N) continue;
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < COMPUTE_WARPS; ++w) total += sums[w][r][token];
            TO* dst = out + (size_t)token * a.ldo + f;
            if (MODE == GEMM_STORE) *dst = from_float<TO>(a.alpha * total);
            else *dst = from_float<TO>(to_float(*dst) + a.alpha * total);
        }
    }
}

template <int MODE, typename TO, int NT>
int launch(const Args& a, int blocks, cudaStream_t stream) {
    const size_t smem = (size_t)a.stages * STAGE_BYTES;
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(gemm_skinny_kernel<MODE, TO, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 MAX_STAGES * STAGE_BYTES) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = (size_t)MAX_STAGES * STAGE_BYTES;
    }
    return lia_launch(gemm_skinny_kernel<MODE, TO, NT>, dim3(blocks), dim3(THREADS), smem, stream, a);
}

int sm_count() {
    static int sms = 0;
    if (!sms) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
            sms = 1;
    }
    return sms;
}

template <int MODE, typename TO>
int launch_nt(const Args& a, int blocks, cudaStream_t stream) {
    if (a.M <= 8) return launch<MODE, TO, 1>(a, blocks, stream);
    if (a.M <= 16) return launch<MODE, TO, 2>(a, blocks, stream);
    return launch<MODE, TO, 4>(a, blocks, stream);
}
}  // namespace

// Most tokens this kernel takes.
LIA_EXPORT int lia_gemm_skinny_max_tokens() { return 32; }

// X [M, K] bf16 (row stride ldx), M <= 32; W [N, K] (SWIGLU: [2N, K], gate rows then up rows) bf16 (row stride
// ldw); out [M, N] f32 or bf16 (row stride ldo).  Refuses K, ldw or ldx that are not multiples of 8 elements and
// pointers that are not 16-byte aligned (bulk copies and 16-byte loads need both).
LIA_EXPORT int lia_gemm_skinny(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                               int ldo, int M, int N, int K, float alpha, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (M > 32 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return LIA_ERR_SIZE;
    if (((uintptr_t)X & 15u) || ((uintptr_t)W & 15u)) return LIA_ERR_ALIGN;
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    Args a;
    a.W = (const __nv_bfloat16*)W; a.X = (const __nv_bfloat16*)X; a.out = out;
    a.ldw = ldw; a.ldx = ldx; a.ldo = ldo; a.M = M; a.N = N; a.K = K; a.alpha = alpha; a.error_flag = error_flag;
    a.chunks = (K + CHUNK_K - 1) / CHUNK_K;
    const long long blocks = mode == GEMM_SWIGLU ? (N + 7) / 8 : (N + ROWS - 1) / ROWS;
    if (blocks > 2147483647LL) return LIA_ERR_SIZE;
    // Stages of the ring.  A CTA that has an SM to itself anyway (no more CTAs than SMs) takes as much of K in flight
    // as fits; with more CTAs it is better that two or three of them share an SM, each with a shorter ring that it
    // uses again, than that one at a time loads, multiplies and leaves (measured at K = 4096 and 16384).
    const int most = blocks <= sm_count() ? MAX_STAGES : (blocks <= 2LL * sm_count() ? 3 : 2);
    a.stages = a.chunks < most ? a.chunks : most;
    if (mode == GEMM_STORE && out_dtype == LIA_F32) return launch_nt<GEMM_STORE, float>(a, (int)blocks, stream);
    if (mode == GEMM_STORE) return launch_nt<GEMM_STORE, __nv_bfloat16>(a, (int)blocks, stream);
    if (mode == GEMM_ACCUM) return launch_nt<GEMM_ACCUM, float>(a, (int)blocks, stream);
    if (out_dtype == LIA_F32) return launch_nt<GEMM_SWIGLU, float>(a, (int)blocks, stream);
    return launch_nt<GEMM_SWIGLU, __nv_bfloat16>(a, (int)blocks, stream);
}
