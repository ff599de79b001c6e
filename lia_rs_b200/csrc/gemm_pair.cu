// Matrix product for many tokens on PAIRS of SMs (tcgen05 with cta_group::2):
//     acc[t, f] = sum_k X[t, k] * W[f, k]       X [M, K] bf16 activations, W [N, K] bf16 weights
//
// With one CTA per 128 x 256 tile the product is bound by what an SM can take in from L2, not by the tensor
// cores: per K block the CTA loads 16 KB of W and 32 KB of X for 4.2 MFLOP.  Here two CTAs of a cluster
// share a tile of 256 weight rows x 256 tokens: each loads ITS 128 rows of W and ITS half of the tokens
// (16 KB + 16 KB per K block), and one tcgen05.mma issued by the first CTA multiplies the whole tile, reading
// the operands from both CTAs' shared memory and writing each CTA's 128 rows of the result into that CTA's
// TMEM.  Same flops per CTA, two thirds of the bytes.  For the gated product both CTAs load gate and up rows
// (two MMAs per step against the same tokens): half the bytes per flop again.
//
// The kernel is persistent (one pair per two SMs walks the tiles round-robin) with the roles of the one-CTA
// kernel: warp 0 issues TMA loads, warp 1 allocates TMEM and (in the first CTA) issues the MMAs, warps 2..5
// read finished accumulators and store through shared memory and TMA.  What the pair adds:
//   * the "stage full" barriers live in the first CTA; the second CTA's loads complete on them too
//     (cp.async.bulk.tensor with .cta_group::2 and the barrier's address with the CTA bit cleared);
//   * "stage free" and "accumulator complete" reach both CTAs by tcgen05.commit with a multicast mask;
//   * "accumulator drained" is counted in the first CTA from the epilogue warps of both.
// Every wait on an mbarrier is bounded; a role that gives up raises the error flag and leaves its loop, and
// all threads of both CTAs still meet at the cluster barrier before TMEM is freed.
//
// Whole tiles only (no split K), outputs by TMA: the caller uses this kernel when there are many tokens and
// the output rows are 16-byte aligned, and the one-CTA kernels otherwise.
#include "tcgen05.cuh"

using namespace tc5;

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_BYTES = 226 * 1024;
constexpr int STAGING_TOKENS = 32;
constexpr int PAIR_F = 2 * TILE_F;               // weight rows per pair tile
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // clears the bit of a shared::cluster address that tells the pair's CTAs apart

struct Shape {
    int M, N, K;
    int n_tile;               // tokens per tile: 64, 128 or 256 (each CTA loads half of them)
    int stages, kblocks, f_tiles, t_tiles;
    int acc_cols, acc_buffers, tmem_cols;
    float alpha;
    int* error_flag;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load of one box whose completion is counted on the FIRST CTA's barrier, whichever CTA issues it.
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar & PEER_BIT_MASK), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive, when the MMAs issued so far are done, on the barrier at this offset in BOTH CTAs of the pair.
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// Arrive on the barrier at this offset in the FIRST CTA's shared memory.
__device__ __forceinline__ void arrive_on_first(uint32_t bar) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(bar), "r"(0));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const __grid_constant__ CUtensorMap map_o, Shape s) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;

    constexpr int A_TILES = (MODE == GEMM_SWIGLU) ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int half_tokens = s.n_tile / 2;
    const uint32_t a_bytes = TILE_F * BLOCK_K * 2, b_bytes = (uint32_t)half_tokens * BLOCK_K * 2;
    const uint32_t stage_bytes = A_TILES * a_bytes + b_bytes;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging_base = smem_base + (uint32_t)s.stages * stage_bytes;     // 2 x [32 tokens][128 features]
    const int units = s.f_tiles * s.t_tiles;
    const int first_unit = blockIdx.x >> 1, stride = gridDim.x >> 1;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < s.stages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);          // the first CTA's producer; the bytes of both CTAs
            mbar_init(smem_u32(&empty_bar[i]), 1);         // one multicast commit
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);          // one multicast commit
            mbar_init(smem_u32(&acc_empty[i]), 8);         // four epilogue warps of each CTA (counted in the first CTA)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_o) : "memory");
    }
    if (warp == 1) {
        // both CTAs of the pair allocate, with the same destination offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)s.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                    // the partner's barriers exist before anything of ours reaches them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (both CTAs): this CTA's 128 rows of W (twice for the gated product), its half of the tokens ----
        bool ok = true;
        int ahead = 0;
        {   // the first ring of W boxes goes out before the kernel ahead has finished: weights depend on nothing
            int it = 0;
            for (int index = first_unit; index < units && it < s.stages; index += stride) {
                const int f0 = (index % s.f_tiles) * PAIR_F + (int)rank * TILE_F;
                for (int kb = 0; kb < s.kblocks && it < s.stages; ++kb, ++it) {
                    const uint32_t full = smem_u32(&full_bar[it]);
                    const uint32_t dst = smem_base + (uint32_t)it * stage_bytes;
                    if (rank == 0) mbar_expect_tx(full, 2 * stage_bytes);
                    tma_load_pair(dst, &map_w, kb * BLOCK_K, f0, full);
                    if (A_TILES == 2) tma_load_pair(dst + a_bytes, &map_w, kb * BLOCK_K, s.N + f0, full);
                }
            }
            ahead = it;
        }
        pdl_wait();
        int it = 0;
        for (int index = first_unit; index < units && ok; index += stride) {
            const int f0 = (index % s.f_tiles) * PAIR_F + (int)rank * TILE_F;
            const int t0 = (index / s.f_tiles) * s.n_tile + (int)rank * half_tokens;
            for (int kb = 0; kb < s.kblocks; ++kb, ++it) {
                const int st = it % s.stages;
                const uint32_t full = smem_u32(&full_bar[st]);
                const uint32_t dst = smem_base + (uint32_t)st * stage_bytes;
                if (it >= ahead) {
                    if (!mbar_wait(smem_u32(&empty_bar[st]), ((uint32_t)(it / s.stages) & 1u) ^ 1u)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full, 2 * stage_bytes);
                    tma_load_pair(dst, &map_w, kb * BLOCK_K, f0, full);
                    if (A_TILES == 2) tma_load_pair(dst + a_bytes, &map_w, kb * BLOCK_K, s.N + f0, full);
                }
                tma_load_pair(dst + A_TILES * a_bytes, &map_x, kb * BLOCK_K, t0, full);
            }
        }
        if (!ok) {
            if (s.error_flag) atomicExch(s.error_flag, 3);
            // copies of this CTA may still be in flight (they complete on the first CTA's barriers, which the second
            // CTA cannot poll): give them a bounded time to land before the CTA goes on to leave
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer (first CTA only): 256 rows x n_tile tokens per instruction ----
        const uint32_t idesc = instr_desc(PAIR_F, s.n_tile);
        bool ok = true;
        int it = 0, n_unit = 0;
        for (int index = first_unit; index < units && ok; index += stride, ++n_unit) {
            const int buf = s.acc_buffers == 2 ? (n_unit & 1) : 0;
            const uint32_t use = s.acc_buffers == 2 ? (uint32_t)n_unit >> 1 : (uint32_t)n_unit;
            if (!mbar_wait(smem_u32(&acc_empty[buf]), (use & 1u) ^ 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)(buf * s.acc_cols);
            for (int kb = 0; kb < s.kblocks; ++kb, ++it) {
                const int st = it % s.stages;
                if (!mbar_wait(smem_u32(&full_bar[st]), (uint32_t)(it / s.stages) & 1u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_base + (uint32_t)st * stage_bytes;
                const uint32_t b_addr = a_addr + A_TILES * a_bytes;
#pragma unroll
                for (int k = 0; k < BLOCK_K / 16; ++k) {
                    const uint64_t db = smem_desc(b_addr + k * 32);
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    mma_pair(acc, smem_desc(a_addr + k * 32), db, idesc, accumulate);
                    if (A_TILES == 2) mma_pair(acc + (uint32_t)s.n_tile, smem_desc(a_addr + a_bytes + k * 32), db, idesc, accumulate);
                }
                commit_pair(smem_u32(&empty_bar[st]));        // the stage is free in both CTAs when these MMAs have read it
            }
            if (ok) commit_pair(smem_u32(&acc_full[buf]));    // the accumulator is complete, in both CTAs
        }
        if (!ok && s.error_flag) atomicExch(s.error_flag, 3);
    } else if (warp >= 2) {
        // ---- epilogue (both CTAs): warp w reads TMEM lanes 32*(w%4) .. +31 = this CTA's features ----
        const int group = warp & 3;
        const int epi_thread = threadIdx.x - 64;
        pdl_wait();
        bool ok = true;
        int n_unit = 0, chunk_count = 0;
        for (int index = first_unit; index < units && ok; index += stride, ++n_unit) {
            const int f0 = (index % s.f_tiles) * PAIR_F + (int)rank * TILE_F;
            const int t0 = (index / s.f_tiles) * s.n_tile;
            const int buf = s.acc_buffers == 2 ? (n_unit & 1) : 0;
            const uint32_t use = s.acc_buffers == 2 ? (uint32_t)n_unit >> 1 : (uint32_t)n_unit;
            if (!mbar_wait(smem_u32(&acc_full[buf]), use & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(group * 32) << 16) + (uint32_t)(buf * s.acc_cols);
            for (int c0 = 0; c0 < s.n_tile; c0 += STAGING_TOKENS) {
                if (t0 + c0 >= s.M) break;
                float acc[32], up[32];
                tmem_load32_nowait(lane_addr + (uint32_t)c0, acc);
                if (MODE == GEMM_SWIGLU) tmem_load32_nowait(lane_addr + (uint32_t)(s.n_tile + c0), up);
                tmem_load_wait();
                const int sbuf = chunk_count & 1;
                ++chunk_count;
                if (epi_thread == 0) tma_wait_read<1>();       // the store that last read this staging buffer is done with it
                epilogue_sync();
                TO* stage = reinterpret_cast<TO*>(smem_raw + (staging_base - smem_u32(smem_raw))) +
                            (size_t)sbuf * STAGING_TOKENS * TILE_F;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    float v;
                    if (MODE == GEMM_SWIGLU) v = up[c] * __fdividef(acc[c], 1.0f + __expf(-acc[c]));
                    else v = s.alpha * acc[c];
                    stage[c * TILE_F + group * 32 + lane] = from_float<TO>(v);
                }
                fence_async_smem();
                epilogue_sync();
                if (epi_thread == 0) {
                    const uint32_t src = staging_base + (uint32_t)(sbuf * STAGING_TOKENS * TILE_F * sizeof(TO));
                    if (MODE == GEMM_ACCUM) tma_reduce_add_2d(&map_o, src, f0, t0 + c0);
                    else tma_store_2d(&map_o, src, f0, t0 + c0);
                    tma_commit_group();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_on_first(smem_u32(&acc_empty[buf]));
        }
        if (!ok && lane == 0 && s.error_flag) atomicExch(s.error_flag, 3);
        if (epi_thread == 0) tma_wait_all();          // shared memory must outlive the stores that read it
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                    // neither CTA frees TMEM (or leaves) while the other may still use the pair's
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)s.tmem_cols) : "memory");
    }
}

int pow2_columns(int x) {
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

template <int MODE, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const Shape& s, int grid, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_pair_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)grid);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = (size_t)SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = lia_pdl_enabled.load(std::memory_order_relaxed) ? 2 : 1;
    lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
    if (cudaLaunchKernelEx(&config, gemm_pair_kernel<MODE, TO>, mw, mx, mo, s) != cudaSuccess) {
        cudaGetLastError();
        return LIA_ERR_LAUNCH;
    }
    return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
}

// Tokens per tile for this product, or 0 if the pair kernel should not take it.
int plan_n_tile(int mode, int M, int N, int sm_count) {
    if (M < 256 || N < PAIR_F) return 0;
    (void)mode; (void)sm_count;
    return 256;
}
}  // namespace

// 1 if lia_gemm_pair takes a product of these sizes (many tokens, at least 256 weight rows), else 0.
LIA_EXPORT int lia_gemm_pair_accepts(int mode, int M, int N, int K, int sm_count) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 || sm_count < 2) return 0;
    return plan_n_tile(mode, M, N, sm_count) > 0 ? 1 : 0;
}

// Arguments as lia_gemm_tc without the scratch.  Refuses (LIA_ERR_SIZE) what lia_gemm_pair_accepts refuses, and
// (LIA_ERR_ALIGN) operands or outputs that TMA cannot address (16-byte aligned bases and row strides).
LIA_EXPORT int lia_gemm_pair(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo,
                             int M, int N, int K, float alpha, int sm_count, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (K <= 0 || K % 8 || ldx < K || ldw < K || ldo < N || sm_count < 2) return LIA_ERR_SIZE;
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    const bool swiglu = mode == GEMM_SWIGLU;
    const int n_tile = plan_n_tile(mode, M, N, sm_count);
    if (n_tile == 0) return LIA_ERR_SIZE;
    const int esize = out_dtype == LIA_F32 ? 4 : 2;
    if (((uintptr_t)out & 15u) || ((long long)ldo * esize) % 16) return LIA_ERR_ALIGN;

    Shape s;
    s.M = M; s.N = N; s.K = K; s.n_tile = n_tile;
    s.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    s.f_tiles = (N + PAIR_F - 1) / PAIR_F;
    s.t_tiles = (M + n_tile - 1) / n_tile;
    s.acc_cols = swiglu ? 2 * n_tile : n_tile;
    s.acc_buffers = 2 * s.acc_cols <= 512 ? 2 : 1;
    s.tmem_cols = pow2_columns(s.acc_buffers * s.acc_cols);
    s.alpha = alpha; s.error_flag = error_flag;
    const int staging = 2 * STAGING_TOKENS * TILE_F * esize;
    const int stage_bytes = (swiglu ? 2 : 1) * TILE_F * BLOCK_K * 2 + (n_tile / 2) * BLOCK_K * 2;
    s.stages = max(2, min(MAX_STAGES, (SMEM_BYTES - 1024 - staging) / stage_bytes));

    CUtensorMap mw, mx, mo;
    int rc;
    if ((rc = make_map(&mw, W, swiglu ? 2 * N : N, K, ldw, TILE_F)) != LIA_OK) return rc;
    if ((rc = make_map(&mx, X, M, K, ldx, n_tile / 2)) != LIA_OK) return rc;
    if ((rc = make_out_map(&mo, out, out_dtype, M, N, ldo, STAGING_TOKENS)) != LIA_OK) return rc;
    const long long units = (long long)s.f_tiles * s.t_tiles;
    const int pairs = (int)min((long long)(sm_count / 2), units);
    const int grid = 2 * pairs;
    if (mode == GEMM_STORE && out_dtype == LIA_F32) return launch<GEMM_STORE, float>(mw, mx, mo, s, grid, stream);
    if (mode == GEMM_STORE) return launch<GEMM_STORE, __nv_bfloat16>(mw, mx, mo, s, grid, stream);
    if (mode == GEMM_ACCUM) return launch<GEMM_ACCUM, float>(mw, mx, mo, s, grid, stream);
    if (out_dtype == LIA_F32) return launch<GEMM_SWIGLU, float>(mw, mx, mo, s, grid, stream);
    return launch<GEMM_SWIGLU, __nv_bfloat16>(mw, mx, mo, s, grid, stream);
}
