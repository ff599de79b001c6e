// Matrix product on the 5th-generation tensor cores (tcgen05), operands by TMA, accumulator in TMEM:
//     acc[t, f] = sum_k X[t, k] * W[f, k]       X [M, K] bf16 activations, W [N, K] bf16 weights
// The weight rows are the MMA's M dimension (128 per CTA) and the tokens its N dimension (16..256),
// so that one kernel serves a prompt portion of thousands of tokens and a decode batch of a few:
// a small batch costs a narrow N, not a padded M.
//
// One CTA computes one tile [128 features x n_tile tokens] over a range of K:
//   warp 0      allocates TMEM, then one lane issues the TMA loads: per 64-wide K block one box of W
//               (two for the fused gate/up product) and one box of X, 128-byte swizzled, into a ring
//               of shared-memory stages guarded by full/empty mbarriers;
//   warp 1      one lane issues tcgen05.mma (M 128, N n_tile, K 16, four per stage) into TMEM and
//               commits each stage's mbarrier when its operands have been read;
//   warps 2..5  read the accumulator with tcgen05.ld (each warp its 32 TMEM lanes = 32 features) and
//               apply the epilogue.  Lanes of a warp hold consecutive features of one token, so every
//               store is a contiguous run of the output row.
// Epilogues: STORE out = alpha*acc; ACCUM out += alpha*acc (32-bit residual stream);
// SWIGLU out = up * gate/(1+exp(-gate)) with gate and up accumulated side by side in TMEM;
// PARTIAL: the raw accumulator of one K range goes to scratch [split][M][N] and a second kernel adds
// the ranges in a fixed order and applies the epilogue.  Splitting K is how a decode batch, whose
// products have few tiles, still puts a CTA on every SM and streams the weights at memory speed.
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises the error flag,
// waits (bounded) for its TMA copies in flight, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2
#define GEMM_PARTIAL 3

namespace {
constexpr int BLOCK_K = 64;          // bf16 elements per K block: 128 bytes, one swizzle row
constexpr int TILE_F = 128;          // features per CTA: the MMA's M
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 22;      // polls of mbarrier.try_wait (each suspends up to ~1 us)
constexpr int MAX_STAGES = 8;
constexpr int SMEM_LIMIT = 200 * 1024;

// ---- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t addr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled, with
// groups of 8 rows 1024 bytes apart: start address, leading offset 1 (unused with a swizzle), stride
// offset 1024 bytes, descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: 32-bit accumulator, bf16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Shape {
    int M, N, K;              // tokens, output features (per half for SWIGLU), reduction length
    int n_tile;               // tokens per CTA: 16..256, a multiple of 16
    int stages;
    int kblocks;              // ceil(K / 64)
    int kblocks_per_split;
    int up_row_offset;        // SWIGLU: row of W where the up half starts
    int tmem_cols;
};

template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TO* __restrict__ out, int ldo, Shape s, float alpha, int* __restrict__ error_flag) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_bar;
    __shared__ uint32_t tmem_base_slot;

    constexpr int A_TILES = (MODE == GEMM_SWIGLU) ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * TILE_F, t0 = blockIdx.y * s.n_tile;
    const int kb_begin = blockIdx.z * s.kblocks_per_split;
    const int kb_end = min(s.kblocks, kb_begin + s.kblocks_per_split);
    const int iterations = kb_end - kb_begin;
    const uint32_t a_bytes = TILE_F * BLOCK_K * 2, b_bytes = (uint32_t)s.n_tile * BLOCK_K * 2;
    const uint32_t stage_bytes = A_TILES * a_bytes + b_bytes;
    // dynamic shared memory is aligned to 1024 bytes by hand (the swizzle pattern repeats every 1024)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < s.stages; ++i) {
                mbar_init(smem_u32(&full_bar[i]), 1);
                mbar_init(smem_u32(&empty_bar[i]), 1);
            }
            mbar_init(smem_u32(&acc_bar), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)s.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int issued = 0;
        bool ok = true;
        for (int it = 0; it < iterations; ++it) {
            const int st = it % s.stages;
            const uint32_t phase = (uint32_t)(it / s.stages) & 1u;
            if (!mbar_wait(smem_u32(&empty_bar[st]), phase ^ 1u)) { ok = false; break; }
            const uint32_t full = smem_u32(&full_bar[st]);
            const uint32_t dst = smem_base + (uint32_t)st * stage_bytes;
            const int k = (kb_begin + it) * BLOCK_K;
            mbar_expect_tx(full, stage_bytes);
            tma_load_2d(dst, &map_w, k, f0, full);
            if (A_TILES == 2) tma_load_2d(dst + a_bytes, &map_w, k, s.up_row_offset + f0, full);
            tma_load_2d(dst + A_TILES * a_bytes, &map_x, k, t0, full);
            issued = it + 1;
        }
        if (!ok) {
            if (error_flag) atomicExch(error_flag, 3);
            // wait, bounded, for the copies that were issued and may still be in flight
            for (int it = max(0, issued - s.stages); it < issued; ++it)
                mbar_wait(smem_u32(&full_bar[it % s.stages]), (uint32_t)(it / s.stages) & 1u);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = instr_desc(TILE_F, s.n_tile);
        bool ok = true;
        for (int it = 0; it < iterations; ++it) {
            const int st = it % s.stages;
            const uint32_t phase = (uint32_t)(it / s.stages) & 1u;
            if (!mbar_wait(smem_u32(&full_bar[st]), phase)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = smem_base + (uint32_t)st * stage_bytes;
            const uint32_t b_addr = a_addr + A_TILES * a_bytes;
#pragma unroll
            for (int k = 0; k < BLOCK_K / 16; ++k) {
                const uint64_t db = smem_desc(b_addr + k * 32);
                const uint32_t accumulate = (it > 0 || k > 0) ? 1u : 0u;
                tc_mma(tmem_base, smem_desc(a_addr + k * 32), db, idesc, accumulate);
                if (A_TILES == 2) tc_mma(tmem_base + (uint32_t)s.n_tile, smem_desc(a_addr + a_bytes + k * 32), db, idesc, accumulate);
            }
            tc_commit(smem_u32(&empty_bar[st]));      // the stage is free when these MMAs have read it
        }
        if (ok) tc_commit(smem_u32(&acc_bar));        // the accumulator is complete
        else if (error_flag) atomicExch(error_flag, 3);
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 ----
        const int group = warp & 3;
        const int f = f0 + group * 32 + lane;
        bool ok = iterations > 0 ? mbar_wait(smem_u32(&acc_bar), 0) : true;
        if (!ok && lane == 0 && error_flag) atomicExch(error_flag, 3);
        tc_fence_after();
        if (ok) {
            const uint32_t lane_addr = tmem_base + ((uint32_t)(group * 32) << 16);
            for (int c0 = 0; c0 < s.n_tile; c0 += 16) {
                if (t0 + c0 >= s.M) break;                    // uniform over the warp
                float acc[16], up[16];
                if (iterations > 0) {
                    tmem_load16(lane_addr + (uint32_t)c0, acc);
                    if (MODE == GEMM_SWIGLU) tmem_load16(lane_addr + (uint32_t)(s.n_tile + c0), up);
                } else {
#pragma unroll
                    for (int c = 0; c < 16; ++c) acc[c] = up[c] = 0.f;
                }
                if (f < s.N) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int t = t0 + c0 + c;
                        if (t >= s.M) break;
                        if (MODE == GEMM_PARTIAL) {
                            out[((size_t)blockIdx.z * s.M + t) * (size_t)ldo + f] = from_float<TO>(acc[c]);
                        } else {
                            TO* dst = out + (size_t)t * ldo + f;
                            if (MODE == GEMM_STORE) *dst = from_float<TO>(alpha * acc[c]);
                            else if (MODE == GEMM_ACCUM) *dst = from_float<TO>(to_float(*dst) + alpha * acc[c]);
                            else *dst = from_float<TO>(up[c] * (acc[c] / (1.0f + __expf(-acc[c]))));
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)s.tmem_cols) : "memory");
    }
}

// Adds the K ranges in ascending order and applies the epilogue.  partial [splits][M][n_total].
template <int MODE, typename TO>
__global__ void splitk_epilogue_kernel(const float* __restrict__ partial, int splits, int M, int n_total, int N,
                                       TO* __restrict__ out, int ldo, float alpha) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    const int t = (int)(i / N), f = (int)(i % N);
    const size_t plane = (size_t)M * n_total;
    float acc = 0.f, up = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
        const float* row = partial + sp * plane + (size_t)t * n_total;
        acc += row[f];
        if (MODE == GEMM_SWIGLU) up += row[N + f];
    }
    TO* dst = out + (size_t)t * ldo + f;
    if (MODE == GEMM_STORE) *dst = from_float<TO>(alpha * acc);
    else if (MODE == GEMM_ACCUM) *dst = from_float<TO>(to_float(*dst) + alpha * acc);
    else *dst = from_float<TO>(up * (acc / (1.0f + __expf(-acc))));
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, cols] bf16 matrix with row stride `ld` elements; boxes of [box_rows, 64], 128-byte swizzle,
// out-of-range elements read as zero.
int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return LIA_ERR_DRIVER;
    if (((uintptr_t)base & 15u) || (ld % 8)) return LIA_ERR_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LIA_OK : LIA_ERR_DRIVER;
}

int pick_n_tile(int M, bool swiglu_fused) {
    const int cap = swiglu_fused ? 128 : 256;      // two accumulators side by side must fit 512 columns and the ring
    int n = 16;
    while (n < M && n < cap) n *= 2;
    return n;
}

int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

template <int MODE, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, TO* out, int ldo, const Shape& s, float alpha, int splits,
           int* error_flag, cudaStream_t stream) {
    const int a_tiles = MODE == GEMM_SWIGLU ? 2 : 1;
    const size_t smem = (size_t)s.stages * (a_tiles * TILE_F * BLOCK_K * 2 + s.n_tile * BLOCK_K * 2) + 1024;
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT + 1024) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = SMEM_LIMIT + 1024;
    }
    dim3 grid((s.N + TILE_F - 1) / TILE_F, (s.M + s.n_tile - 1) / s.n_tile, splits);
    gemm_tc_kernel<MODE, TO><<<grid, THREADS, smem, stream>>>(mw, mx, out, ldo, s, alpha, error_flag);
    return lia_check_launch();
}
}  // namespace

// mode: GEMM_STORE | GEMM_ACCUM | GEMM_SWIGLU.  X [M, K] bf16 (row stride ldx), W [N, K] (SWIGLU: [2N, K],
// gate rows then up rows) bf16 (row stride ldw), out [M, N] f32 or bf16 (row stride ldo).
// `scratch` (32-bit, `scratch_floats` long) is used when K is split; `sm_count` is the number of SMs to fill.
// Refuses (LIA_ERR_SIZE / LIA_ERR_ALIGN) what it cannot compute: K or a row stride that is not a multiple
// of 8 elements, pointers that are not 16-byte aligned.
LIA_EXPORT int lia_gemm_tc(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                           int ldo, int M, int N, int K, float alpha, float* scratch, long long scratch_floats,
                           int sm_count, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (K <= 0 || K % 8 || ldx < K || ldw < K || ldo < N) return LIA_ERR_SIZE;
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    const bool swiglu = mode == GEMM_SWIGLU;
    const int n_total = swiglu ? 2 * N : N;
    const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;

    // How many K ranges: enough CTAs to fill the SMs when the product has few tiles.
    int n_tile = pick_n_tile(M, false);
    const long long tiles = (long long)((n_total + TILE_F - 1) / TILE_F) * ((M + n_tile - 1) / n_tile);
    int splits = 1;
    if (tiles < sm_count && M <= 256 && scratch) {
        splits = (int)min((long long)16, (2LL * sm_count + tiles - 1) / tiles);
        splits = min(splits, max(1, kblocks / 4));               // at least 4 K blocks per range
        while (splits > 1 && (long long)splits * M * n_total > scratch_floats) --splits;
    }
    Shape s;
    s.M = M; s.K = K; s.kblocks = kblocks; s.up_row_offset = N;
    CUtensorMap mw, mx;
    int rc;
    if (splits > 1) {
        s.N = n_total; s.n_tile = n_tile;
        s.kblocks_per_split = (kblocks + splits - 1) / splits;
        splits = (kblocks + s.kblocks_per_split - 1) / s.kblocks_per_split;
        s.tmem_cols = pow2_at_least(n_tile);
        const int stage_bytes = TILE_F * BLOCK_K * 2 + n_tile * BLOCK_K * 2;
        s.stages = max(2, min(MAX_STAGES, SMEM_LIMIT / stage_bytes));
        if ((rc = make_map(&mw, W, n_total, K, ldw, TILE_F)) != LIA_OK) return rc;
        if ((rc = make_map(&mx, X, M, K, ldx, n_tile)) != LIA_OK) return rc;
        rc = launch<GEMM_PARTIAL, float>(mw, mx, scratch, n_total, s, 1.0f, splits, error_flag, stream);
        if (rc != LIA_OK) return rc;
        const size_t count = (size_t)M * N;
        const int threads = 256;
        const unsigned blocks = (unsigned)((count + threads - 1) / threads);
#define LIA_EPI(MODE, TO) splitk_epilogue_kernel<MODE, TO><<<blocks, threads, 0, stream>>>(scratch, splits, M, n_total, N, (TO*)out, ldo, alpha)
        if (mode == GEMM_STORE && out_dtype == LIA_F32) LIA_EPI(GEMM_STORE, float);
        else if (mode == GEMM_STORE) LIA_EPI(GEMM_STORE, __nv_bfloat16);
        else if (mode == GEMM_ACCUM) LIA_EPI(GEMM_ACCUM, float);
        else if (out_dtype == LIA_F32) LIA_EPI(GEMM_SWIGLU, float);
        else LIA_EPI(GEMM_SWIGLU, __nv_bfloat16);
#undef LIA_EPI
        return lia_check_launch();
    }
    n_tile = pick_n_tile(M, swiglu);
    s.N = N; s.n_tile = n_tile; s.kblocks_per_split = kblocks;
    s.tmem_cols = pow2_at_least(swiglu ? 2 * n_tile : n_tile);
    const int stage_bytes = (swiglu ? 2 : 1) * TILE_F * BLOCK_K * 2 + n_tile * BLOCK_K * 2;
    s.stages = max(2, min(MAX_STAGES, SMEM_LIMIT / stage_bytes));
    if ((rc = make_map(&mw, W, n_total, K, ldw, TILE_F)) != LIA_OK) return rc;
    if ((rc = make_map(&mx, X, M, K, ldx, n_tile)) != LIA_OK) return rc;
    if (mode == GEMM_STORE && out_dtype == LIA_F32) return launch<GEMM_STORE, float>(mw, mx, (float*)out, ldo, s, alpha, 1, error_flag, stream);
    if (mode == GEMM_STORE) return launch<GEMM_STORE, __nv_bfloat16>(mw, mx, (__nv_bfloat16*)out, ldo, s, alpha, 1, error_flag, stream);
    if (mode == GEMM_ACCUM) return launch<GEMM_ACCUM, float>(mw, mx, (float*)out, ldo, s, alpha, 1, error_flag, stream);
    if (out_dtype == LIA_F32) return launch<GEMM_SWIGLU, float>(mw, mx, (float*)out, ldo, s, alpha, 1, error_flag, stream);
    return launch<GEMM_SWIGLU, __nv_bfloat16>(mw, mx, (__nv_bfloat16*)out, ldo, s, alpha, 1, error_flag, stream);
}

// ---------------------------------------------------------------------------------------------------
// The same product for callers that must not allocate: see gemm_tc_noalloc.h for who they are and for
// the contract.  The split-K scratch is a static array in the library image instead of a caller's buffer.
#include <mutex>

#include "gemm_tc_noalloc.h"

namespace {
constexpr long long NOALLOC_FLOATS = LIA_GEMM_NOALLOC_SCRATCH_BYTES / sizeof(float);
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float noalloc_scratch[NOALLOC_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
float* noalloc_address[NOALLOC_MAX_DEVICES] = {};
std::mutex noalloc_mutex;

// Device address of the static array on the current device; looked up once per device.
int noalloc_scratch_address(float** address) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NOALLOC_MAX_DEVICES) return LIA_ERR_DRIVER;
    std::lock_guard<std::mutex> lock(noalloc_mutex);
    if (!noalloc_address[device]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, noalloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return LIA_ERR_DRIVER;
        }
        noalloc_address[device] = (float*)p;
    }
    *address = noalloc_address[device];
    return LIA_OK;
}
}  // namespace

// The split plan lia_gemm_tc makes when its scratch is large enough, restated so that the need is known
// before anything is launched.
LIA_EXPORT long long lia_gemm_tc_noalloc_scratch_floats(int mode, int M, int N, int K, int sm_count) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int n_total = mode == GEMM_SWIGLU ? 2 * N : N;
    const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    const int n_tile = pick_n_tile(M, false);
    const long long tiles = (long long)((n_total + TILE_F - 1) / TILE_F) * ((M + n_tile - 1) / n_tile);
    if (!(tiles < sm_count && M <= 256)) return 0;
    int splits = (int)min((long long)16, (2LL * sm_count + tiles - 1) / tiles);
    splits = min(splits, max(1, kblocks / 4));
    if (splits <= 1) return 0;
    return (long long)splits * M * n_total;
}

LIA_EXPORT int lia_gemm_tc_noalloc(int mode, const void* X, int ldx, const void* W, int ldw, void* out,
                                   int out_dtype, int ldo, int M, int N, int K, float alpha, int sm_count,
                                   int* error_flag, cudaStream_t stream) {
    if (lia_gemm_tc_noalloc_scratch_floats(mode, M, N, K, sm_count) > NOALLOC_FLOATS) return LIA_ERR_SCRATCH;
    float* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc != LIA_OK) return rc;
    return lia_gemm_tc(mode, X, ldx, W, ldw, out, out_dtype, ldo, M, N, K, alpha, scratch, NOALLOC_FLOATS,
                       sm_count, error_flag, stream);
}
