// Matrix product on the 5th-generation tensor cores (tcgen05), operands by TMA, accumulators in TMEM:
//     acc[t, f] = sum_k X[t, k] * W[f, k]       X [M, K] bf16 activations, W [N, K] bf16 weights
// The weight rows are the MMA's M dimension (128 per tile) and the tokens its N dimension (16..256), so
// that one kernel serves a prompt portion of thousands of tokens and a decode batch of a few: a small
// batch costs a narrow N, not a padded M.
//
// The kernel is persistent: at most one CTA per SM, each walking a list of work units
// (tile, K range) round-robin.  Inside a CTA the warps have fixed roles and never wait for one another
// except through mbarriers:
//   warp 0      one lane issues the TMA loads: per 64-wide K block one box of W (two for the fused
//               gate/up product) and one box of X, 128-byte swizzled, into a ring of shared-memory
//               stages.  The ring runs on across units, so the memory pipeline never drains.
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (M 128, N n_tile, K 16, four per stage)
//               into one of TWO accumulator buffers in TMEM and commits each stage's mbarrier when its
//               operands have been read, and the buffer's mbarrier when the unit is complete.
//   warps 2..5  the epilogue: they read a finished buffer with tcgen05.ld (each warp its 32 TMEM lanes
//               = 32 features) while the MMA warp already fills the other buffer.
// Epilogues: STORE out = alpha*acc; ACCUM out += alpha*acc (32-bit residual stream);
// SWIGLU out = up * gate/(1+exp(-gate)) with gate and up accumulated side by side in TMEM.
// With many tokens the tile goes through shared memory and leaves by TMA (bulk store, or bulk
// reduce-add for ACCUM, which adds in L2 and never reads the old value into the SM); with few tokens it
// is stored directly.
//
// Few tokens mean few tiles, so K is cut into ranges to give every SM work (that is how a decode batch
// streams the weights at memory speed).  Each unit then writes its raw accumulator to scratch
// [range][M][n_total] and bumps its tile's counter; the CTA that arrives last adds the ranges in
// ascending order (so the sum does not depend on who was last), applies the epilogue and puts the
// counter back to zero.  No CTA ever waits for another one.
//
// The kernel is launched with programmatic dependent launch: it may start while the kernel before it
// in the stream is still draining.  Weights do not depend on that kernel, so the first ring of W boxes
// is requested at once; everything else waits at griddepcontrol.wait.
//
// Every wait on an mbarrier is bounded: when the bound is hit the role raises the error flag and leaves
// its loop; the CTA then waits (bounded) for its copies in flight, frees its TMEM and returns.
#include <algorithm>

#include "tcgen05.cuh"

using namespace tc5;

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 12;
constexpr int SMEM_BYTES = 226 * 1024;         // dynamic shared memory asked for (a CTA may have 227 KB; 1 KB is static)
constexpr int STAGING_TOKENS = 32;             // tokens per TMA store of the epilogue
constexpr int COUNTER_WORDS = 4096;            // tile counters at the head of the scratch

struct Shape {
    int M, N, K;              // tokens, output features (per half for SWIGLU), reduction length
    int n_total;              // rows of W: N, or 2N for SWIGLU
    int n_tile;               // tokens per tile: 16..512, a multiple of 16 (of 32 beyond 256: two MMAs, two X boxes)
    int x_box;                // tokens per TMA box of X: n_tile, or half of it beyond 256
    int stages;
    int kblocks;              // ceil(K / 64)
    int splits;               // K ranges per tile
    int f_tiles, t_tiles;
    int acc_cols;             // TMEM columns of one accumulator buffer
    int tmem_cols;            // TMEM columns allocated (all buffers, a power of two >= 32)
    int acc_buffers;          // 2: the epilogue drains one accumulator while the next unit fills the other; 1: they take turns
    int via_tma;              // 1: the epilogue leaves through shared memory and TMA
    int ldo;
    float alpha;
    float* partial;           // [splits][M][n_total]
    int* counters;            // [f_tiles * t_tiles], zero between launches
    int* error_flag;
};

// The k-th unit of this CTA: which tile, which K blocks.
struct Unit {
    int f0, t0, tile, split, kb_begin, kb_end;
};
__device__ __forceinline__ Unit unit_at(const Shape& s, int index) {
    Unit u;
    u.tile = index / s.splits;
    u.split = index - u.tile * s.splits;
    const int ft = u.tile % s.f_tiles, tt = u.tile / s.f_tiles;
    u.f0 = ft * TILE_F;
    u.t0 = tt * s.n_tile;
    u.kb_begin = (int)((long long)u.split * s.kblocks / s.splits);
    u.kb_end = (int)((long long)(u.split + 1) * s.kblocks / s.splits);
    return u;
}

template <int MODE, typename TO>
__device__ __forceinline__ void apply_epilogue(TO* dst, float acc, float up, float alpha) {
    if (MODE == GEMM_STORE) *dst = from_float<TO>(alpha * acc);
    else if (MODE == GEMM_ACCUM) *dst = from_float<TO>(to_float(*dst) + alpha * acc);
    else *dst = from_float<TO>(up * (acc / (1.0f + __expf(-acc))));
}

template <int MODE, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_o, TO* __restrict__ out, Shape s) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int last_flag;

    constexpr int A_TILES = (MODE == GEMM_SWIGLU) ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t a_bytes = TILE_F * BLOCK_K * 2, b_bytes = (uint32_t)s.n_tile * BLOCK_K * 2;
    const uint32_t stage_bytes = A_TILES * a_bytes + b_bytes;
    // dynamic shared memory is aligned to 1024 bytes by hand (the swizzle pattern repeats every 1024)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging_base = smem_base + (uint32_t)s.stages * stage_bytes;     // 2 x [32 tokens][128 features]
    const int units = s.f_tiles * s.t_tiles * s.splits;
    const int first_unit = blockIdx.x, stride = gridDim.x;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < s.stages; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 4);         // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        if (s.via_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_o) : "memory");
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
        // ---- TMA producer ----
        // The first ring of W boxes is asked for before the kernel ahead of this one has finished: the
        // weights do not depend on it.  X does, so its boxes wait.
        bool ok = true;
        int issued = 0, ahead = 0;
        {
            int it = 0;
            for (int index = first_unit; index < units && it < s.stages; index += stride) {
                const Unit u = unit_at(s, index);
                for (int kb = u.kb_begin; kb < u.kb_end && it < s.stages; ++kb, ++it) {
                    const uint32_t full = smem_u32(&full_bar[it]);
                    const uint32_t dst = smem_base + (uint32_t)it * stage_bytes;
                    mbar_expect_tx(full, stage_bytes);
                    tma_load_2d(dst, &map_w, kb * BLOCK_K, u.f0, full);
                    if (A_TILES == 2) tma_load_2d(dst + a_bytes, &map_w, kb * BLOCK_K, s.N + u.f0, full);
                }
            }
            ahead = it;
        }
        pdl_wait();
        // (the stage and its phase are counted along: a division by the number of stages per K block costs this
        // thread more than the block's loads)
        int it = 0, st = 0;
        uint32_t phase = 0;
        for (int index = first_unit; index < units && ok; index += stride) {
            const Unit u = unit_at(s, index);
            for (int kb = u.kb_begin; kb < u.kb_end; ++kb, ++it, st = (st + 1 == s.stages ? 0 : st + 1), phase ^= (st == 0 ? 1u : 0u)) {
                const uint32_t full = smem_u32(&full_bar[st]);
                const uint32_t dst = smem_base + (uint32_t)st * stage_bytes;
                if (it >= ahead) {
                    if (!mbar_wait(smem_u32(&empty_bar[st]), phase ^ 1u)) { ok = false; break; }
                    mbar_expect_tx(full, stage_bytes);
                    tma_load_2d(dst, &map_w, kb * BLOCK_K, u.f0, full);
                    if (A_TILES == 2) tma_load_2d(dst + a_bytes, &map_w, kb * BLOCK_K, s.N + u.f0, full);
                }
                tma_load_2d(dst + A_TILES * a_bytes, &map_x, kb * BLOCK_K, u.t0, full);
                if (s.x_box < s.n_tile)
                    tma_load_2d(dst + A_TILES * a_bytes + (uint32_t)s.x_box * 128u, &map_x, kb * BLOCK_K, u.t0 + s.x_box, full);
                issued = it + 1;
            }
        }
        if (!ok) {
            if (s.error_flag) atomicExch(s.error_flag, 3);
            // wait, bounded, for the copies that were issued and may still be in flight
            for (int i = max(0, issued - s.stages); i < issued; ++i)
                mbar_wait(smem_u32(&full_bar[i % s.stages]), (uint32_t)(i / s.stages) & 1u);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // a tile of more than 256 tokens takes two MMAs per K step: 256 tokens, then the rest
        const int n_first = s.n_tile > 256 ? 256 : s.n_tile, n_rest = s.n_tile - n_first;
        const uint32_t idesc = instr_desc(TILE_F, n_first), idesc_rest = instr_desc(TILE_F, n_rest > 0 ? n_rest : 16);
        bool ok = true;
        int n_unit = 0, st = 0;
        uint32_t phase = 0;
        // A narrow tile's K block is four short MMAs, and what this thread does between them sets the block's time:
        // so the stage and its phase are counted along (no division per block), and the operands' descriptors are
        // the first stage's plus an offset (the start address is their lowest field, in 16-byte units, and shared
        // memory ends below what the field holds).
        const uint64_t desc_a0 = smem_desc(smem_base), desc_b0 = smem_desc(smem_base + A_TILES * a_bytes);
        const uint64_t stage_step = stage_bytes >> 4, a_step = a_bytes >> 4, rest_step = ((uint32_t)n_first * 128u) >> 4;
        uint64_t stage_offset = 0;
        for (int index = first_unit; index < units && ok; index += stride, ++n_unit) {
            const Unit u = unit_at(s, index);
            const int buf = s.acc_buffers == 2 ? (n_unit & 1) : 0;
            const uint32_t use = s.acc_buffers == 2 ? (uint32_t)n_unit >> 1 : (uint32_t)n_unit;
            if (!mbar_wait(smem_u32(&acc_empty[buf]), (use & 1u) ^ 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)(buf * s.acc_cols);
            for (int kb = u.kb_begin; kb < u.kb_end; ++kb) {
                if (!mbar_wait(smem_u32(&full_bar[st]), phase)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da0 = desc_a0 + stage_offset, db0 = desc_b0 + stage_offset;
                const uint32_t first = kb > u.kb_begin ? 1u : 0u;
                // (the wide tile's second MMA has a loop of its own, so that the common loop carries nothing for it)
                if (n_rest == 0) {
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k) {
                        const uint32_t accumulate = k > 0 ? 1u : first;
                        tc_mma(acc, da0 + 2 * k, db0 + 2 * k, idesc, accumulate);
                        if (A_TILES == 2) tc_mma(acc + (uint32_t)s.n_tile, da0 + a_step + 2 * k, db0 + 2 * k, idesc, accumulate);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k) {
                        const uint32_t accumulate = k > 0 ? 1u : first;
                        tc_mma(acc, da0 + 2 * k, db0 + 2 * k, idesc, accumulate);
                        tc_mma(acc + (uint32_t)n_first, da0 + 2 * k, db0 + rest_step + 2 * k, idesc_rest, accumulate);
                    }
                }
                tc_commit(smem_u32(&empty_bar[st]));      // the stage is free when these MMAs have read it
                if (++st == s.stages) { st = 0; stage_offset = 0; phase ^= 1u; }
                else stage_offset += stage_step;
            }
            if (ok) tc_commit(smem_u32(&acc_full[buf]));  // the accumulator is complete
        }
        if (!ok && s.error_flag) atomicExch(s.error_flag, 3);
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 ----
        const int group = warp & 3;
        const int epi_thread = threadIdx.x - 64;          // 0..127
        pdl_wait();
        bool ok = true;
        int n_unit = 0, chunk_count = 0;
        for (int index = first_unit; index < units && ok; index += stride, ++n_unit) {
            const Unit u = unit_at(s, index);
            const int buf = s.acc_buffers == 2 ? (n_unit & 1) : 0;
            const uint32_t use = s.acc_buffers == 2 ? (uint32_t)n_unit >> 1 : (uint32_t)n_unit;
            const int f = u.f0 + group * 32 + lane;
            const bool empty_range = u.kb_end <= u.kb_begin;           // cannot happen (splits <= kblocks)
            if (!empty_range && !mbar_wait(smem_u32(&acc_full[buf]), use & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(group * 32) << 16) + (uint32_t)(buf * s.acc_cols);

            if (s.splits > 1) {
                // raw accumulator to scratch [split][t][n_total]
                float* plane = s.partial + (size_t)u.split * s.M * s.n_total;
                for (int c0 = 0; c0 < s.n_tile; c0 += 16) {
                    if (u.t0 + c0 >= s.M) break;
                    float acc[16], up[16];
                    tmem_load16(lane_addr + (uint32_t)c0, acc);
                    if (MODE == GEMM_SWIGLU) tmem_load16(lane_addr + (uint32_t)(s.n_tile + c0), up);
                    if (f < s.N) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = u.t0 + c0 + c;
                            if (t >= s.M) break;
                            plane[(size_t)t * s.n_total + f] = acc[c];
                            if (MODE == GEMM_SWIGLU) plane[(size_t)t * s.n_total + s.N + f] = up[c];
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
                // the last unit of the tile to arrive adds the ranges in ascending order
                __threadfence();
                epilogue_sync();
                if (epi_thread == 0) {
                    const int seen = atomicAdd(&s.counters[u.tile], 1);
                    last_flag = (seen == s.splits - 1);
                    if (seen == s.splits - 1) s.counters[u.tile] = 0;
                }
                epilogue_sync();
                if (last_flag) {
                    __threadfence();
                    if (f < s.N) {
                        const int rows = min(s.n_tile, s.M - u.t0);
                        for (int c0 = 0; c0 < rows; c0 += 8) {
                            float acc[8], up[8];
#pragma unroll
                            for (int c = 0; c < 8; ++c) acc[c] = up[c] = 0.f;
                            // four ranges at a time: all their loads are in flight before the first sum
                            for (int sp0 = 0; sp0 < s.splits; sp0 += 4) {
                                float v[4][8], w[4][8];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float* src = s.partial + ((size_t)(sp0 + j) * s.M + u.t0 + c0) * s.n_total + f;
#pragma unroll
                                    for (int c = 0; c < 8; ++c) {
                                        const bool there = sp0 + j < s.splits && c0 + c < rows;
                                        v[j][c] = there ? __ldcg(src + (size_t)c * s.n_total) : 0.f;
                                        if (MODE == GEMM_SWIGLU) w[j][c] = there ? __ldcg(src + (size_t)c * s.n_total + s.N) : 0.f;
                                    }
                                }
#pragma unroll
                                for (int j = 0; j < 4; ++j)
#pragma unroll
                                    for (int c = 0; c < 8; ++c) {
                                        acc[c] += v[j][c];
                                        if (MODE == GEMM_SWIGLU) up[c] += w[j][c];
                                    }
                            }
#pragma unroll
                            for (int c = 0; c < 8; ++c)
                                if (c0 + c < rows)
                                    apply_epilogue<MODE, TO>(out + (size_t)(u.t0 + c0 + c) * s.ldo + f, acc[c], up[c], s.alpha);
                        }
                    }
                }
                epilogue_sync();      // last_flag is read by all before the next unit rewrites it
            } else if (s.via_tma) {
                // through shared memory, 32 tokens at a time, out by TMA
                for (int c0 = 0; c0 < s.n_tile; c0 += STAGING_TOKENS) {
                    if (u.t0 + c0 >= s.M) break;
                    float acc[32], up[32];
                    tmem_load32_nowait(lane_addr + (uint32_t)c0, acc);
                    if (MODE == GEMM_SWIGLU) tmem_load32_nowait(lane_addr + (uint32_t)(s.n_tile + c0), up);
                    tmem_load_wait();
                    const int sbuf = chunk_count & 1;
                    ++chunk_count;
                    // the store that last read this staging buffer must be done reading it
                    if (epi_thread == 0) tma_wait_read<1>();
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
                        if (MODE == GEMM_ACCUM) tma_reduce_add_2d(&map_o, src, u.f0, u.t0 + c0);
                        else tma_store_2d(&map_o, src, u.f0, u.t0 + c0);
                        tma_commit_group();
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
            } else {
                for (int c0 = 0; c0 < s.n_tile; c0 += 16) {
                    if (u.t0 + c0 >= s.M) break;                    // uniform over the warp
                    float acc[16], up[16];
                    tmem_load16(lane_addr + (uint32_t)c0, acc);
                    if (MODE == GEMM_SWIGLU) tmem_load16(lane_addr + (uint32_t)(s.n_tile + c0), up);
                    if (f < s.N) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = u.t0 + c0 + c;
                            if (t >= s.M) break;
                            apply_epilogue<MODE, TO>(out + (size_t)t * s.ldo + f, acc[c], up[c], s.alpha);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
            }
        }
        if (!ok && lane == 0 && s.error_flag) atomicExch(s.error_flag, 3);
        if (s.via_tma && epi_thread == 0) tma_wait_all();     // shared memory must outlive the stores that read it
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)s.tmem_cols) : "memory");
    }
}

int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p *= 2;
    return p;
}

// How the product is cut: tokens per tile, K ranges per tile.  A function of the sizes and of the SM
// count alone, so the same product is always cut the same way.
struct Plan {
    int n_tile, splits, f_tiles, t_tiles;
};

Plan make_plan(int mode, int M, int N, int K, int sm_count, long long scratch_floats) {
    const bool swiglu = mode == GEMM_SWIGLU;
    const int n_total = swiglu ? 2 * N : N;
    const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    Plan p;
    p.f_tiles = (N + TILE_F - 1) / TILE_F;
    const int few = 128;                         // up to here one tile holds all tokens and K is cut into ranges
    if (M <= few) {
        p.n_tile = 16;
        while (p.n_tile < M) p.n_tile *= 2;
    } else {
        // many tokens: the tile width (a multiple of 32, the epilogue's step) that leaves the SMs least idle: rounds of
        // tiles times the time of one.  Measured on a B200: a tile takes 5.5 us plus, per K block, the longest of
        // three: its MMAs' time (0.43 us at 256 tokens at the clocks a long product runs at, in proportion below;
        // twice that for the gated product's two accumulators); the time its SM needs to take the block in (an SM
        // takes in about 108 GB/s: 16 KB of W, or 32, and 128 bytes per token; this is what a narrow tile waits
        // for, and why narrower tiles on more SMs beat wide ones on few); and what its producer thread needs to
        // issue the block's two to four TMA boxes (0.1 us each).  Ties go to the wider tile (fewer bytes through
        // shared memory per flop).  Up to 512 tokens wide (all of TMEM, so one buffer: the epilogue and the next tile
        // take turns), 256 for the gated product, where that saves a round: 2,048 tokens x 2,560 features are 140
        // tiles of 320 tokens, one round, against 260 of 160.  Down to 32 tokens where the tiles would otherwise be
        // too few for the SMs: K is NOT cut for more than 128 tokens (the CTA that arrives last would add up ranges
        // of hundreds of tokens alone, which costs more than narrow tiles do).
        const double weights = swiglu ? 2.0 : 1.0;
        const int widest = std::min(swiglu ? 256 : 512, (M + 31) / 32 * 32);
        double best = -1;
        p.n_tile = widest;
        for (int n = widest; n >= 32; n -= 32) {
            const long long tiles = (long long)p.f_tiles * ((M + n - 1) / n);
            const long long rounds = (tiles + sm_count - 1) / sm_count;
            const double mma = weights * 0.43 * n / 256.0;
            const double intake = (weights * 16384.0 + n * 128.0) / 108e3;
            const double issue = 0.1 * (weights + (n > 256 ? 2.0 : 1.0));
            const double cost = (double)rounds * (5.5 + kblocks * std::max(mma, std::max(intake, issue)));
            if (best < 0 || cost < best) { best = cost; p.n_tile = n; }
        }
    }
    p.t_tiles = (M + p.n_tile - 1) / p.n_tile;
    p.splits = 1;
    const long long tiles = (long long)p.f_tiles * p.t_tiles;
    if (M <= few && tiles < sm_count && tiles <= COUNTER_WORDS && scratch_floats > COUNTER_WORDS) {
        // cost in K-block times of the longest CTA: rounds * (blocks per range + fixed) + the last arriver's sum
        double best = 0;
        for (int sp = 1; sp <= kblocks && sp <= 32; ++sp) {
            if (sp > 1 && (long long)sp * M * n_total > scratch_floats - COUNTER_WORDS) break;
            const long long rounds = (tiles * sp + sm_count - 1) / sm_count;
            const double cost = rounds * ((kblocks + sp - 1) / sp + 2.0) + (sp > 1 ? 1.0 + 0.25 * sp : 0.0);
            if (sp == 1 || cost < best) { best = cost; p.splits = sp; }
        }
    }
    return p;
}

template <int MODE, typename TO>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, TO* out, const Shape& s, int grid,
           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    return lia_launch(gemm_tc_kernel<MODE, TO>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, stream, mw, mx, mo, out, s);
}
}  // namespace

// mode: GEMM_STORE | GEMM_ACCUM | GEMM_SWIGLU.  X [M, K] bf16 (row stride ldx), W [N, K] (SWIGLU: [2N, K],
// gate rows then up rows) bf16 (row stride ldw), out [M, N] f32 or bf16 (row stride ldo).
// `scratch` (32-bit words, `scratch_floats` long) is used when K is split: its first 4096 words are tile
// counters that must be zero before the first call and are zero again after every call; the rest holds
// partial sums.  `sm_count` is the number of SMs to fill.
// Refuses (LIA_ERR_SIZE / LIA_ERR_ALIGN) what it cannot compute: K or a row stride that is not a multiple
// of 8 elements, pointers that are not 16-byte aligned.
LIA_EXPORT int lia_gemm_tc(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                           int ldo, int M, int N, int K, float alpha, float* scratch, long long scratch_floats,
                           int sm_count, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (K <= 0 || K % 8 || ldx < K || ldw < K || ldo < N || sm_count <= 0) return LIA_ERR_SIZE;
    if (mode != GEMM_STORE && mode != GEMM_ACCUM && mode != GEMM_SWIGLU) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (out_dtype != LIA_F32 && out_dtype != LIA_BF16) return LIA_ERR_DTYPE;
    const bool swiglu = mode == GEMM_SWIGLU;
    const Plan plan = make_plan(mode, M, N, K, sm_count, scratch ? scratch_floats : 0);

    Shape s;
    s.M = M; s.N = N; s.K = K; s.n_total = swiglu ? 2 * N : N;
    s.n_tile = plan.n_tile; s.splits = plan.splits; s.f_tiles = plan.f_tiles; s.t_tiles = plan.t_tiles;
    s.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    s.x_box = plan.n_tile > 256 ? plan.n_tile / 2 : plan.n_tile;
    s.acc_cols = swiglu ? 2 * plan.n_tile : plan.n_tile;
    s.acc_buffers = 2 * s.acc_cols <= 512 ? 2 : 1;
    s.tmem_cols = pow2_at_least(s.acc_buffers * s.acc_cols);
    s.ldo = ldo; s.alpha = alpha; s.error_flag = error_flag;
    s.counters = reinterpret_cast<int*>(scratch);
    s.partial = scratch ? scratch + COUNTER_WORDS : nullptr;
    const int esize = out_dtype == LIA_F32 ? 4 : 2;
    // the epilogue leaves by TMA when there are enough tokens to make it worth it and the output can be addressed
    s.via_tma = (plan.splits == 1 && M >= 64 && ((uintptr_t)out & 15u) == 0 && ((long long)ldo * esize) % 16 == 0) ? 1 : 0;
    const int staging = s.via_tma ? 2 * STAGING_TOKENS * TILE_F * esize : 0;
    const int stage_bytes = (swiglu ? 2 : 1) * TILE_F * BLOCK_K * 2 + plan.n_tile * BLOCK_K * 2;
    s.stages = max(2, min(MAX_STAGES, (SMEM_BYTES - 1024 - staging) / stage_bytes));

    CUtensorMap mw, mx, mo;
    int rc;
    if ((rc = make_map(&mw, W, s.n_total, K, ldw, TILE_F)) != LIA_OK) return rc;
    if ((rc = make_map(&mx, X, M, K, ldx, s.x_box)) != LIA_OK) return rc;
    if (s.via_tma) {
        if ((rc = make_out_map(&mo, out, out_dtype, M, N, ldo, STAGING_TOKENS)) != LIA_OK) return rc;
    } else {
        mo = mx;
    }
    const long long units = (long long)plan.f_tiles * plan.t_tiles * plan.splits;
    const int grid = (int)min((long long)sm_count, units);
    if (mode == GEMM_STORE && out_dtype == LIA_F32) return launch<GEMM_STORE, float>(mw, mx, mo, (float*)out, s, grid, stream);
    if (mode == GEMM_STORE) return launch<GEMM_STORE, __nv_bfloat16>(mw, mx, mo, (__nv_bfloat16*)out, s, grid, stream);
    if (mode == GEMM_ACCUM) return launch<GEMM_ACCUM, float>(mw, mx, mo, (float*)out, s, grid, stream);
    if (out_dtype == LIA_F32) return launch<GEMM_SWIGLU, float>(mw, mx, mo, (float*)out, s, grid, stream);
    return launch<GEMM_SWIGLU, __nv_bfloat16>(mw, mx, mo, (__nv_bfloat16*)out, s, grid, stream);
}

// ---------------------------------------------------------------------------------------------------
// The same product for callers that must not allocate: see gemm_tc_noalloc.h for who they are and for
// the contract.  The split-K scratch is a static array in the library image instead of a caller's buffer.
#include <mutex>

#include "gemm_tc_noalloc.h"

namespace {
constexpr long long NOALLOC_FLOATS = LIA_GEMM_NOALLOC_SCRATCH_BYTES / sizeof(float);
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
// Zero when the library is loaded, which is what the tile counters at its head need.
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

// Words of scratch the product of these sizes uses when nothing limits it (0: it does not split K).
LIA_EXPORT long long lia_gemm_tc_noalloc_scratch_floats(int mode, int M, int N, int K, int sm_count) {
    if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0) return 0;
    const Plan plan = make_plan(mode, M, N, K, sm_count, 1LL << 60);
    if (plan.splits <= 1) return 0;
    return (long long)plan.splits * M * (mode == GEMM_SWIGLU ? 2 * N : N) + COUNTER_WORDS;
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

// Puts the tile counters at the head of the array back to zero, in stream order.  For use after a call whose
// kernel gave up on a wait (error flag 3): it may have left counters mid-count, and every later split-K product
// of the device would then add its ranges at the wrong moment.  Allocates nothing.
LIA_EXPORT int lia_gemm_tc_noalloc_reset(cudaStream_t stream) {
    float* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc != LIA_OK) return rc;
    if (cudaMemsetAsync(scratch, 0, COUNTER_WORDS * sizeof(int), stream) != cudaSuccess) {
        cudaGetLastError();
        return LIA_ERR_LAUNCH;
    }
    return LIA_OK;
}
