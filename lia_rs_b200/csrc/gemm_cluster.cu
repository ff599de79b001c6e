// Matrix product for a middling number of tokens (a decode batch of dozens, a short prompt portion):
//     acc[t, f] = sum_k X[t, k] * W[f, k]       X [M, K] bf16 activations, W [N, K] bf16 weights
// on the 5th-generation tensor cores, with K cut over the CTAs of a thread-block cluster.
//
// With few tokens the product has few output tiles (128 weight rows x the tokens), far fewer than SMs,
// while its work is streaming W once at memory speed: every SM must take part.  So the CTAs of a cluster
// (2 to 8) share one tile and each multiplies a range of K: its W boxes and its slice of X come by TMA
// into a ring of 128-byte-swizzled stages (the whole range is usually in flight at once), one thread
// issues tcgen05.mma into a TMEM accumulator.  The partial sums then meet through DISTRIBUTED SHARED
// MEMORY: every CTA writes its accumulator to its own shared memory, the cluster synchronises, and
// CTA r adds the tokens r, r + size, ... of all CTAs in ascending rank order (so the sum is the same
// in every run and for every cutting of the batch), applies the epilogue and stores.  No scratch in
// global memory, no atomics, no second kernel.
//
// Epilogues: STORE out = alpha*acc; ACCUM out += alpha*acc (32-bit residual stream);
// SWIGLU out = up * gate/(1+exp(-gate)), gate and up accumulated side by side in TMEM.
//
// Programmatic dependent launch: W depends on no earlier kernel, so its first ring is requested before
// griddepcontrol.wait; X waits.  Every mbarrier wait is bounded; a role that gives up raises the error
// flag, and every thread still reaches both cluster barriers, so no CTA of a cluster is left waiting.
#include "tcgen05.cuh"

using namespace tc5;

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int THREADS = 224;            // warp 0: TMA, warps 1 and 6: MMA, warps 2-5: accumulator to shared memory
constexpr int MAX_STAGES = 12;
constexpr int MAX_CLUSTER = 8;
constexpr int SMEM_LIMIT = 200 * 1024;

struct Shape {
    int M, N, K;
    int n_tile;               // tokens per tile: a multiple of 16, at most 128
    int box_rows;             // rows of W per TMA box (divides 128, a multiple of 8)
    int stages, batch, kblocks, splits, f_tiles, t_tiles;   // batch: K blocks whose W boxes are issued together
    int tmem_cols;
    int chains;               // accumulators that take the K steps in turn (1, 2 or 4)
    int ldo, vector_ok;       // vector_ok: rows of out may be stored 4 elements at a time
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
// 16 bytes of the shared memory of the cluster's CTA `rank`, at the offset that `addr` has in this CTA's.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

template <int MODE, typename TO>
__device__ __forceinline__ void finish(TO* dst, float acc, float up, float alpha) {
    if (MODE == GEMM_STORE) *dst = from_float<TO>(alpha * acc);
    else if (MODE == GEMM_ACCUM) *dst = from_float<TO>(to_float(*dst) + alpha * acc);
    else *dst = from_float<TO>(up * (acc / (1.0f + __expf(-acc))));
}

template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    TO* __restrict__ out, Shape s) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full;
    __shared__ uint32_t tmem_base_slot;

    constexpr int A_TILES = (MODE == GEMM_SWIGLU) ? 2 : 1;
    constexpr int ACC_W = TILE_F * A_TILES;                 // floats per token in the exchange buffer
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t a_bytes = TILE_F * BLOCK_K * 2, b_bytes = (uint32_t)s.n_tile * BLOCK_K * 2;
    const uint32_t stage_bytes = A_TILES * a_bytes + b_bytes;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    float* exchange = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));   // [n_tile][ACC_W], reuses the ring

    const uint32_t rank = cluster_rank();
    const int tile = blockIdx.x / s.splits;
    const int f0 = (tile % s.f_tiles) * TILE_F, t0 = (tile / s.f_tiles) * s.n_tile;
    const int kb_begin = (int)((long long)rank * s.kblocks / s.splits);
    const int kb_end = (int)((long long)(rank + 1) * s.kblocks / s.splits);
    const int nkb = kb_end - kb_begin;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < s.stages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), 1);
        }
        mbar_init(smem_u32(&acc_full), s.chains >= 2 ? 2 : 1);       // one arrival per MMA issuer
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)s.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: W at once, X when the kernel ahead has finished ----
        // W comes in boxes of 8 rows x 64 k (one 1024-byte swizzle atom each), issued k-major inside a
        // batch of K blocks: consecutive requests then read consecutive 128-byte pieces of the same 8
        // rows of W, which is what DRAM pages want; a 128-row box per K block would touch 128 rows
        // before it came back to the first.
        auto issue_w = [&](int it0, int count) {
            for (int j = 0; j < count; ++j) mbar_expect_tx(smem_u32(&full_bar[(it0 + j) % s.stages]), stage_bytes);
            for (int a = 0; a < A_TILES; ++a)
                for (int g = 0; g < TILE_F / s.box_rows; ++g)
                    for (int j = 0; j < count; ++j) {
                        const int st = (it0 + j) % s.stages;
                        tma_load_2d(smem_base + (uint32_t)st * stage_bytes + (uint32_t)a * a_bytes + (uint32_t)(g * s.box_rows) * 128u, &map_w,
                                    (kb_begin + it0 + j) * BLOCK_K, a * s.N + f0 + g * s.box_rows, smem_u32(&full_bar[st]));
                    }
        };
        auto issue_x = [&](int it0, int count) {
            for (int j = 0; j < count; ++j) {
                const int st = (it0 + j) % s.stages;
                tma_load_2d(smem_base + (uint32_t)st * stage_bytes + A_TILES * a_bytes, &map_x, (kb_begin + it0 + j) * BLOCK_K, t0,
                            smem_u32(&full_bar[st]));
            }
        };
        const int ahead = min(nkb, s.stages);
        for (int it0 = 0; it0 < ahead; it0 += s.batch) issue_w(it0, min(s.batch, ahead - it0));
        pdl_wait();
        issue_x(0, ahead);
        bool ok = true;
        int issued = ahead;
        for (int it0 = ahead; it0 < nkb && ok; it0 += s.batch) {
            const int count = min(s.batch, nkb - it0);
            for (int j = 0; j < count && ok; ++j)
                ok = mbar_wait(smem_u32(&empty_bar[(it0 + j) % s.stages]), ((uint32_t)((it0 + j) / s.stages) & 1u) ^ 1u);
            if (!ok) break;
            issue_w(it0, count);
            issue_x(it0, count);
            issued = it0 + count;
        }
        if (!ok) {
            if (s.error_flag) atomicExch(s.error_flag, 3);
            for (int i = max(0, issued - s.stages); i < issued; ++i)      // copies in flight must land before the CTA may end
                mbar_wait(smem_u32(&full_bar[i % s.stages]), (uint32_t)(i / s.stages) & 1u);
        }
    } else if ((warp == 1 || warp == 6) && lane == 0) {
        // ---- MMA issuers.  Issuing one tcgen05.mma costs a thread some 130 cycles, four times what a tile this
        //      narrow computes for, so two threads issue: they take the K blocks in turn, each into accumulators of
        //      its own (an MMA that adds to the accumulator of the one before it would wait for it, too).  The
        //      epilogue adds the accumulators up in a fixed order. ----
        const int issuers = s.chains >= 2 ? 2 : 1;
        const int me = warp == 1 ? 0 : 1;
        const int own = s.chains / issuers;                   // accumulators of this issuer
        const uint32_t idesc = instr_desc(TILE_F, s.n_tile);
        bool ok = true;
        int mine = 0;                                         // K blocks this issuer has taken
        if (me < issuers) {
            // (the stage and its phase are counted along, and the descriptors are the first stage's plus an offset in
            // their lowest field, the start address in 16-byte units: what this thread does between two MMAs is
            // what a K block of a narrow tile takes)
            const uint64_t desc_a0 = smem_desc(smem_base), desc_b0 = smem_desc(smem_base + A_TILES * a_bytes);
            const uint32_t stage_step = stage_bytes >> 4, a_step = a_bytes >> 4;
            int st = me % s.stages;
            uint32_t phase = (uint32_t)(me / s.stages) & 1u;
            for (int it = me; it < nkb; it += issuers, ++mine) {
                if (!mbar_wait(smem_u32(&full_bar[st]), phase)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da0 = desc_a0 + (uint64_t)((uint32_t)st * stage_step), db0 = desc_b0 + (uint64_t)((uint32_t)st * stage_step);
#pragma unroll
                for (int k = 0; k < BLOCK_K / 16; ++k) {
                    const int chain = me * own + (k & (own - 1));
                    const uint32_t accumulate = (mine > 0 || k >= own) ? 1u : 0u;
                    const uint32_t acc_addr = tmem_base + (uint32_t)(chain * A_TILES * s.n_tile);
                    tc_mma(acc_addr, da0 + 2 * k, db0 + 2 * k, idesc, accumulate);
                    if (A_TILES == 2) tc_mma(acc_addr + (uint32_t)s.n_tile, da0 + a_step + 2 * k, db0 + 2 * k, idesc, accumulate);
                }
                tc_commit(smem_u32(&empty_bar[st]));
                st += issuers;
                while (st >= s.stages) { st -= s.stages; phase ^= 1u; }
            }
            if (ok) tc_commit(smem_u32(&acc_full));
            else if (s.error_flag) atomicExch(s.error_flag, 3);
        }
    } else if (warp >= 2 && warp <= 5) {
        // ---- accumulator to the exchange buffer: warp w holds TMEM lanes 32*(w%4) .. +31 = features ----
        const int group = warp & 3;
        const bool ok = nkb <= 0 || mbar_wait(smem_u32(&acc_full), 0u);     // all MMAs done: the ring is free to reuse
        tc_fence_after();
        if (!ok && lane == 0 && s.error_flag) atomicExch(s.error_flag, 3);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(group * 32) << 16);
        const int valid = min(s.n_tile, s.M - t0);
        for (int c0 = 0; c0 < valid; c0 += 16) {
            float acc[16], up[16];
            if (ok && nkb > 0) {
                tmem_load16(lane_addr + (uint32_t)c0, acc);
                if (MODE == GEMM_SWIGLU) tmem_load16(lane_addr + (uint32_t)(s.n_tile + c0), up);
                const int live = (s.chains >= 2 && nkb < 2) ? s.chains / 2 : s.chains;   // the second issuer's stay untouched with one K block
                for (int chain = 1; chain < live; ++chain) {              // in chain order: the same sum in every run
                    float more[16];
                    tmem_load16(lane_addr + (uint32_t)(chain * A_TILES * s.n_tile + c0), more);
#pragma unroll
                    for (int c = 0; c < 16; ++c) acc[c] += more[c];
                    if (MODE == GEMM_SWIGLU) {
                        tmem_load16(lane_addr + (uint32_t)(chain * A_TILES * s.n_tile + s.n_tile + c0), more);
#pragma unroll
                        for (int c = 0; c < 16; ++c) up[c] += more[c];
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[c] = up[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                if (c0 + c < valid) {
                    exchange[(size_t)(c0 + c) * ACC_W + group * 32 + lane] = acc[c];
                    if (MODE == GEMM_SWIGLU) exchange[(size_t)(c0 + c) * ACC_W + TILE_F + group * 32 + lane] = up[c];
                }
            }
        }
    }
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();                 // every CTA's partial sums are in its exchange buffer
    pdl_wait();                         // `out` may have been written by the kernels ahead

    {
        // ---- CTA r adds tokens r, r + splits, ... over all CTAs, in rank order, and stores ----
        const int valid = min(s.n_tile, s.M - t0);
        const int mine = valid > (int)rank ? (valid - (int)rank + s.splits - 1) / s.splits : 0;
        const uint32_t exchange_addr = smem_base;
        for (int item = threadIdx.x; item < mine * (TILE_F / 4); item += THREADS) {
            const int tl = (int)rank + (item / (TILE_F / 4)) * s.splits;
            const int q = item % (TILE_F / 4);
            const int f = f0 + q * 4;
            if (f >= s.N) continue;
            const uint32_t at = exchange_addr + (uint32_t)((tl * ACC_W + q * 4) * 4);
            float4 part[MAX_CLUSTER], part_up[MAX_CLUSTER];
#pragma unroll
            for (int c = 0; c < MAX_CLUSTER; ++c) {
                if (c < s.splits) {
                    part[c] = ld_cluster_f4(at, (uint32_t)c);
                    if (MODE == GEMM_SWIGLU) part_up[c] = ld_cluster_f4(at + TILE_F * 4, (uint32_t)c);
                }
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < MAX_CLUSTER; ++c) {
                if (c < s.splits) {
                    acc[0] += part[c].x; acc[1] += part[c].y; acc[2] += part[c].z; acc[3] += part[c].w;
                    if (MODE == GEMM_SWIGLU) { up[0] += part_up[c].x; up[1] += part_up[c].y; up[2] += part_up[c].z; up[3] += part_up[c].w; }
                }
            }
            TO* dst = out + (size_t)(t0 + tl) * s.ldo + f;
            if (s.vector_ok && f + 4 <= s.N) {
                float r[4];
                if (MODE == GEMM_ACCUM) {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    r[0] = old.x + s.alpha * acc[0]; r[1] = old.y + s.alpha * acc[1];
                    r[2] = old.z + s.alpha * acc[2]; r[3] = old.w + s.alpha * acc[3];
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        r[i] = MODE == GEMM_SWIGLU ? up[i] * (acc[i] / (1.0f + __expf(-acc[i]))) : s.alpha * acc[i];
                }
                if (sizeof(TO) == 4) {
                    *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
                    uint2 v;
                    v.x = *reinterpret_cast<uint32_t*>(&lo);
                    v.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = v;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (f + i < s.N) finish<MODE, TO>(dst + i, acc[i], up[i], s.alpha);
            }
        }
    }
    cluster_sync_all();                 // nobody leaves while a neighbour may still read its shared memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)s.tmem_cols) : "memory");
    }
}

int pow2_columns(int x) {
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

struct Plan {
    int n_tile, splits, f_tiles, t_tiles;
};

// Clusters of `size` CTAs that the device keeps resident at once (asked of the driver once per size).  A
// product with more tiles than that would run its clusters in two rounds, which costs more than a
// smaller cluster does.
int max_active_clusters(int size) {
    static int cached[MAX_CLUSTER + 1] = {};
    if (size < 1 || size > MAX_CLUSTER) return 0;
    if (cached[size] == 0) {
        auto kernel = gemm_cluster_kernel<GEMM_STORE, float>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT + 1024);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((unsigned)(size * 64));
        config.blockDim = dim3(THREADS);
        config.dynamicSmemBytes = (size_t)SMEM_LIMIT;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = (unsigned)size;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
            cudaGetLastError();
            clusters = -1;
        }
        cached[size] = clusters > 0 ? clusters : -1;
    }
    return cached[size] > 0 ? cached[size] : 0;
}

// Tokens per tile and CTAs per cluster: a function of the sizes and the SM count alone.  splits < 2
// means the product has enough tiles of its own (or too short a K) and belongs to the persistent kernel.
Plan make_plan(int M, int N, int K, int sm_count) {
    Plan p;
    p.f_tiles = (N + TILE_F - 1) / TILE_F;
    p.t_tiles = (M + 127) / 128;
    const int per_tile = (M + p.t_tiles - 1) / p.t_tiles;
    p.n_tile = (per_tile + 15) / 16 * 16;
    const long long tiles = (long long)p.f_tiles * p.t_tiles;
    const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    long long splits = tiles > 0 ? sm_count / tiles : 0;
    if (splits > MAX_CLUSTER) splits = MAX_CLUSTER;
    if (splits > kblocks) splits = kblocks;
    while (splits >= 2 && tiles > max_active_clusters((int)splits)) --splits;      // all clusters in one round
    p.splits = (int)splits;
    return p;
}

template <int MODE, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, TO* out, const Shape& s, int smem, cudaStream_t stream) {
    static int configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(gemm_cluster_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT + 1024) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = SMEM_LIMIT + 1024;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(s.f_tiles * s.t_tiles * s.splits));
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = (size_t)smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = (unsigned)s.splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = lia_pdl_enabled.load(std::memory_order_relaxed) ? 2 : 1;
    lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
    if (cudaLaunchKernelEx(&config, gemm_cluster_kernel<MODE, TO>, mw, mx, out, s) != cudaSuccess) {
        cudaGetLastError();
        return LIA_ERR_LAUNCH;
    }
    return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
}
}  // namespace

// CTAs per cluster that lia_gemm_cluster would use for these sizes (less than 2: the product is not for
// this kernel; the persistent kernel takes it).
LIA_EXPORT int lia_gemm_cluster_splits(int mode, int M, int N, int K, int sm_count) {
    if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0) return 0;
    (void)mode;
    return make_plan(M, N, K, sm_count).splits;
}

// Arguments as lia_gemm_tc without the scratch.  Refuses (LIA_ERR_SIZE) a product that
// lia_gemm_cluster_splits gives fewer than 2 CTAs per cluster, K or row strides that are not multiples of
// 8 elements, and (LIA_ERR_ALIGN) pointers that are not 16-byte aligned.
LIA_EXPORT int lia_gemm_cluster(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                                int ldo, int M, int N, int K, float alpha, int sm_count, int* error_flag,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (K <= 0 || K % 8 || ldx < K || ldw < K || ldo < N || sm_count <= 0) return LIA_ERR_SIZE;
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    const bool swiglu = mode == GEMM_SWIGLU;
    const Plan plan = make_plan(M, N, K, sm_count);
    if (plan.splits < 2) return LIA_ERR_SIZE;

    Shape s;
    s.M = M; s.N = N; s.K = K;
    s.n_tile = plan.n_tile; s.splits = plan.splits; s.f_tiles = plan.f_tiles; s.t_tiles = plan.t_tiles;
    s.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    s.chains = 4;
    while (s.chains > 1 && s.chains * (swiglu ? 2 : 1) * plan.n_tile > 512) s.chains /= 2;
    s.tmem_cols = pow2_columns(s.chains * (swiglu ? 2 : 1) * plan.n_tile);
    s.ldo = ldo; s.alpha = alpha; s.error_flag = error_flag;
    const int esize = out_dtype == LIA_F32 ? 4 : 2;
    s.vector_ok = (((uintptr_t)out % (4 * esize)) == 0 && ldo % 4 == 0) ? 1 : 0;
    const int stage_bytes = (swiglu ? 2 : 1) * TILE_F * BLOCK_K * 2 + plan.n_tile * BLOCK_K * 2;
    const int exchange_bytes = plan.n_tile * TILE_F * (swiglu ? 2 : 1) * 4;
    const int longest = (s.kblocks + plan.splits - 1) / plan.splits;
    s.stages = max(1, min(min(MAX_STAGES, longest), SMEM_LIMIT / stage_bytes));
    s.batch = s.stages;
    if (longest > s.stages && s.stages >= 2) {       // the ring is used again: two batches, one lands while the other is multiplied
        s.batch = s.stages / 2;
        s.stages = 2 * s.batch;
    }
    const int smem = max(s.stages * stage_bytes, exchange_bytes) + 1024;
    if (smem > SMEM_LIMIT + 1024) return LIA_ERR_SIZE;

    CUtensorMap mw, mx;
    int rc;
    s.box_rows = TILE_F;
    if ((rc = make_map(&mw, W, swiglu ? 2 * N : N, K, ldw, s.box_rows)) != LIA_OK) return rc;
    if ((rc = make_map(&mx, X, M, K, ldx, plan.n_tile)) != LIA_OK) return rc;
    if (mode == GEMM_STORE && out_dtype == LIA_F32) return launch<GEMM_STORE, float>(mw, mx, (float*)out, s, smem, stream);
    if (mode == GEMM_STORE) return launch<GEMM_STORE, __nv_bfloat16>(mw, mx, (__nv_bfloat16*)out, s, smem, stream);
    if (mode == GEMM_ACCUM) return launch<GEMM_ACCUM, float>(mw, mx, (float*)out, s, smem, stream);
    if (out_dtype == LIA_F32) return launch<GEMM_SWIGLU, float>(mw, mx, (float*)out, s, smem, stream);
    return launch<GEMM_SWIGLU, __nv_bfloat16>(mw, mx, (__nv_bfloat16*)out, s, smem, stream);
}
