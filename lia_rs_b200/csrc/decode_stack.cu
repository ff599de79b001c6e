// A whole stack of pre-norm decoder layers for a decode step of a few tokens, as ONE persistent kernel.
//
// A decode step of a handful of tokens is the streaming of every weight once, and with one kernel per
// product (some ten per layer) most of its time goes to starting and draining them: each launch ramps
// its memory pipeline up from nothing.  Here one CTA per SM stays resident for all layers.  In each CTA
// a producer thread streams that CTA's share of EVERY weight matrix, in the fixed order in which the
// layers use them, through a ring of shared-memory stages (bulk asynchronous copies, mbarrier
// completion); it never waits for anything but a free stage, so while the CTAs meet at a grid barrier
// between two products the next product's weights are already arriving.  Eight warps consume the ring
// with mma.sync m16n8k16 (16 weight rows x 8 tokens), exactly as the few-token product does.
//
// Per layer (x: 32-bit residual stream [tokens, hidden], s: the residual scale):
//   A  qkv = rmsnorm(x) Wqkv^T                    the norm is folded in: the CTA stages bf16(x * w_norm)
//                                                 in shared memory, sums x^2 per token on the way, and
//                                                 scales the accumulator by 1/sqrt(mean + eps)
//   B  rotary positions, append k and v to their pages, attention over the paged cache split over the
//      keys, ranges merged by the CTA that finishes a token last (as in the split-key decode kernel)
//   C  x += s * attn Wo^T
//   D  act = up * gate/(1+exp(-gate)), [gate; up] = rmsnorm(x) Wgu^T      (norm folded in as in A)
//   E  x += s * act Wd^T
// with a grid barrier after each.  Every CTA takes an equal range of each matrix's rows, so all stream
// the same number of bytes.  Everything that a later phase reads and an earlier one wrote is read past
// L1 (ld.global.cg, cp.async.cg): L1 is not coherent between SMs and is not flushed inside a kernel.
//
// All sizes are parameters (hidden, heads, groups, intermediate, eps, rotary size, page size, window per
// layer); the head size is a template parameter (64 or 128), the tokens at most 16.  The caller falls
// back to the per-part kernels for anything else.
//
// The grid barrier is a counter in global memory that only grows; the launch is cooperative, so all
// CTAs are resident.  A wait that runs out (it cannot, unless a CTA died) raises the error flag and the
// kernel winds down without waiting again.
#include "attention_tc.cuh"

using namespace attn;

namespace {
constexpr int COMPUTE_WARPS = 8;
constexpr int CONSUMERS = COMPUTE_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;        // + the producer warp
constexpr int ROWS = 16;                       // weight rows per ring stage
constexpr int CHUNK_K = 1024;                  // elements of K per ring stage
constexpr int PITCH = CHUNK_K * 2 + 64;        // row pitch of a stage: 16-byte reads of 8 rows spread over the banks
constexpr int STAGE_BYTES = ROWS * PITCH;
constexpr int RING = 4;
constexpr int MAX_TOKENS = 16;
constexpr int ATTN_WARPS = 4;                  // warps 0..3 run the attention phase
constexpr int ATTN_STAGES = 2;
constexpr int SIDE_BYTES = 68 * 1024;          // staged activations (phases A, D) or attention tiles + q (phase B)
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int MAX_SPLITS = 32;
constexpr int MAX_LAYERS = 64;                 // layer records kept in shared memory (a record in global memory is a cold miss per use)

struct LayerParams {
    const void* norm1;               // [hidden] bf16 or f32
    const void* norm2;
    const __nv_bfloat16* wqkv;       // [(nq + 2 nkv) D, hidden]
    const __nv_bfloat16* wo;         // [hidden, nq D]
    const __nv_bfloat16* wgu;        // [2 intermediate, hidden]: gate rows, then up rows
    const __nv_bfloat16* wd;         // [hidden, intermediate]
    __nv_bfloat16* k_pages;          // [pages, page_size, nkv, D]
    __nv_bfloat16* v_pages;
    const int* block_table;          // [slots, table_stride]
    int table_stride, page_size, page_shift, num_pages, window, write_kv, norm_f32, pad;
};

struct StackParams {
    const LayerParams* layers;
    int n_layers, M, H, nq, nkv, I, rotary_dim, n_splits;
    float eps, residual_scale, scale_log2;
    const float* inv_freq;           // [rotary_dim / 2]
    float* h;                        // [M, H] residual stream, in and out
    float* qkv;                      // [M, (nq + 2 nkv) D] scratch
    __nv_bfloat16* attn;             // [M, nq D] scratch
    __nv_bfloat16* act;              // [M, I] scratch
    float* partial;                  // [M, nq, n_splits, D] then [M, nq, n_splits]
    int* counters;                   // [M * nkv], zero between launches
    const int* positions;            // [M]
    const int* slots;                // [M]
    unsigned long long* barrier;     // [0]: arrivals since the state was zeroed; [1]: arrivals before this launch
    int* error_flag;
    long long* timeline;             // optional [n_layers][16]: CTA 0's clock (ns) at the start of a layer, after each phase's parts and after each barrier
};

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
// The producer's wait: also ends when the consumers have given up.
__device__ __forceinline__ bool mbar_wait_or_abort(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
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
        if (*abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void attention_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float exp2_whole(float n) {       // 2^n for a whole number n <= 0 (or -infinity), exactly
    return n < -126.f ? 0.f : __int_as_float(((int)n + 127) << 23);
}
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned long long load_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// What the CTA keeps in shared memory besides the ring and the side region.
struct Control {
    uint64_t full_bar[RING], empty_bar[RING];
    unsigned long long barrier_base;
    int abort_flag, last_flag;
    float inv_rms[MAX_TOKENS];
    int positions[MAX_TOKENS], slots[MAX_TOKENS];
    float2* rotation;                                    // [tokens][rotary_dim / 2] (cos, sin) of position * inv_freq: the same in every layer       // the step's metadata, read once (a miss under load costs microseconds)
};

// One product's description, the same for the producer and the consumers.
struct Product {
    const __nv_bfloat16* W;
    int N, K, ldw, swiglu;           // N: rows of W (per half for swiglu)
};

// Rows [begin, end) of a product that this CTA owns.
__device__ __forceinline__ void my_rows(int N, int& begin, int& end) {
    begin = (int)((long long)blockIdx.x * N / gridDim.x);
    end = (int)((long long)(blockIdx.x + 1) * N / gridDim.x);
}

// ---- producer warp: the ring runs on across products and layers.  Lane 0 waits for the stage and
//      announces the bytes; then every row's copy is issued by a lane of its own (issuing a bulk copy
//      takes a thread some 80 ns, whatever its size: one thread alone would not keep up with memory) ----
__device__ void produce(const Product& g, uint8_t* ring, Control* ctl, uint32_t& it, bool& ok) {
    const int lane = threadIdx.x & 31;
    int begin, end;
    my_rows(g.N, begin, end);
    const int per_block = g.swiglu ? ROWS / 2 : ROWS;
    const int chunks = (g.K + CHUNK_K - 1) / CHUNK_K;
    for (int b0 = begin; b0 < end && ok; b0 += per_block) {
        const int rows = min(per_block, end - b0);
        for (int c = 0; c < chunks; ++c, ++it) {
            const uint32_t st = it % RING;
            const int k0 = c * CHUNK_K;
            const uint32_t bytes = (uint32_t)min(CHUNK_K, g.K - k0) * 2u;
            const uint32_t full = smem_u32(&ctl->full_bar[st]);
            const uint32_t dst = smem_u32(ring) + st * STAGE_BYTES;
            if (lane == 0) {
                if (it >= RING && !mbar_wait_or_abort(smem_u32(&ctl->empty_bar[st]), ((it / RING) & 1u) ^ 1u, &ctl->abort_flag)) ok = false;
                if (ok) mbar_expect_tx(full, bytes * (uint32_t)(g.swiglu ? 2 * rows : rows));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) return;
            // slot of the stage -> row of W: slots 0..15 are consecutive rows; for the gated product slots
            // 0..7 are gate rows and 8..15 the matching up rows
            if (lane < ROWS) {
                const int r = g.swiglu ? (lane & 7) : lane;
                const size_t w_row = g.swiglu ? (size_t)(lane < 8 ? 0 : g.N) + b0 + r : (size_t)b0 + r;
                if (r < rows)
                    bulk_copy(dst + (uint32_t)(lane * PITCH), g.W + w_row * g.ldw + k0, bytes, full);
            }
        }
    }
}

// ---- grid barrier of the consumer warps ----
__device__ bool grid_sync(const StackParams& p, Control* ctl, uint32_t& n_barrier) {
    ++n_barrier;
    consumer_sync();
    if (threadIdx.x == 0 && !ctl->abort_flag) {
        const unsigned long long target = ctl->barrier_base + (unsigned long long)n_barrier * gridDim.x;
        // release: what this CTA's threads wrote (ordered before by the barrier above) is visible to whoever
        // sees the count; acquire: what the others wrote is visible after the count is seen
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p.barrier), "l"(1ULL) : "memory");
        bool arrived = false;
        for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
            if (load_acquire(p.barrier) >= target) { arrived = true; break; }
            if ((i & 1023u) == 1023u && p.error_flag && *((volatile int*)p.error_flag) != 0) break;
        }
        if (!arrived) {
            ctl->abort_flag = 1;
            if (p.error_flag) atomicExch(p.error_flag, 3);
        }
    }
    consumer_sync();
    return ctl->abort_flag == 0;
}

enum { EPI_STORE_SCALED = 0, EPI_ACCUM = 1, EPI_SWIGLU_SCALED = 2 };

// ---- consumers: one product.  X comes from shared memory (x_smem, row pitch x_pitch bytes) or from
//      global memory (x_global, row stride ldx elements).  8 warps share each chunk of K. ----
template <int NT, int EPI>
__device__ void consume(const StackParams& p, const Product& g, const uint8_t* ring, Control* ctl, float* sums_base,
                        const uint8_t* x_smem, int x_pitch, const __nv_bfloat16* x_global, int ldx,
                        void* out, int ldo, uint32_t& it, uint32_t& n_block, bool& ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, t = lane & 3;
    int begin, end;
    my_rows(g.N, begin, end);
    const int per_block = g.swiglu ? ROWS / 2 : ROWS;
    const int chunks = (g.K + CHUNK_K - 1) / CHUNK_K;
    constexpr int SUMS_W = NT * 8 + 1;
    for (int b0 = begin; b0 < end; b0 += per_block) {
        const int rows = min(per_block, end - b0);
        const bool row_lo = g.swiglu ? gq < rows : gq < rows;
        const bool row_hi = g.swiglu ? gq < rows : gq + 8 < rows;
        // one accumulator per group of 32 k that the warp takes in a chunk: the tensor-core instructions of a
        // chunk then do not wait for one another (a chain of eight costs more than the whole chunk's copies)
        constexpr int CHAINS = CHUNK_K / 32 / COMPUTE_WARPS;
        float part[CHAINS][NT][4];
#pragma unroll
        for (int i = 0; i < CHAINS; ++i)
#pragma unroll
            for (int n = 0; n < NT; ++n) part[i][n][0] = part[i][n][1] = part[i][n][2] = part[i][n][3] = 0.f;
        for (int c = 0; c < chunks; ++c, ++it) {
            const uint32_t st = it % RING;
            const int k0 = c * CHUNK_K;
            const int groups = (min(CHUNK_K, g.K - k0) + 31) / 32;
            constexpr int PER_WARP = CHUNK_K / 32 / COMPUTE_WARPS;
            uint4 xf[PER_WARP][NT];
#pragma unroll
            for (int i = 0; i < PER_WARP; ++i) {
                const int k = k0 + (warp + i * COMPUTE_WARPS) * 32 + t * 8;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const int token = n * 8 + gq;
                    if (warp + i * COMPUTE_WARPS < groups && k < g.K && token < p.M) {
                        if (x_smem) xf[i][n] = *reinterpret_cast<const uint4*>(x_smem + (size_t)token * x_pitch + (size_t)k * 2);
                        else xf[i][n] = __ldcg(reinterpret_cast<const uint4*>(x_global + (size_t)token * ldx + k));
                    } else {
                        xf[i][n] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            if (ok && !mbar_wait(smem_u32(&ctl->full_bar[st]), (it / RING) & 1u)) ok = false;
            const uint8_t* stage = ring + st * STAGE_BYTES;
            if (ok) {
#pragma unroll
                for (int i = 0; i < PER_WARP; ++i) {
                    const int group = warp + i * COMPUTE_WARPS;
                    const int k = k0 + group * 32 + t * 8;
                    if (group < groups) {
                        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
                        if (k < g.K) {
                            const int offset = (group * 32 + t * 8) * 2;
                            if (row_lo) lo = *reinterpret_cast<const uint4*>(stage + gq * PITCH + offset);
                            if (row_hi) hi = *reinterpret_cast<const uint4*>(stage + (gq + 8) * PITCH + offset);
                        }
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            mma16816(part[i][n], lo.x, hi.x, lo.y, hi.y, xf[i][n].x, xf[i][n].y);
                            mma16816(part[i][n], lo.z, hi.z, lo.w, hi.w, xf[i][n].z, xf[i][n].w);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->empty_bar[st]));
        }
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
        // the eight warps' partial sums meet in shared memory, added in warp order; with up to 8 tokens two
        // buffers take turns, so one barrier per block is enough (the next block's barrier shields this
        // block's readers); with more tokens there is room for one buffer only, and a second barrier
        constexpr int SUMS_BUFFERS = NT == 1 ? 2 : 1;
        float* sums = sums_base + (size_t)(n_block % SUMS_BUFFERS) * COMPUTE_WARPS * ROWS * SUMS_W;
        ++n_block;
        float* mine = sums + (size_t)warp * ROWS * SUMS_W;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            mine[gq * SUMS_W + n * 8 + 2 * t] = acc[n][0];
            mine[gq * SUMS_W + n * 8 + 2 * t + 1] = acc[n][1];
            mine[(gq + 8) * SUMS_W + n * 8 + 2 * t] = acc[n][2];
            mine[(gq + 8) * SUMS_W + n * 8 + 2 * t + 1] = acc[n][3];
        }
        consumer_sync();
        if (EPI == EPI_SWIGLU_SCALED) {
            for (int i = threadIdx.x; i < 8 * NT * 8; i += CONSUMERS) {
                const int token = i >> 3, r = i & 7;
                if (token >= p.M || r >= rows) continue;
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < COMPUTE_WARPS; ++w) {
                    gate += sums[((size_t)w * ROWS + r) * SUMS_W + token];
                    up += sums[((size_t)w * ROWS + r + 8) * SUMS_W + token];
                }
                gate *= ctl->inv_rms[token];
                up *= ctl->inv_rms[token];
                reinterpret_cast<__nv_bfloat16*>(out)[(size_t)token * ldo + b0 + r] =
                    __float2bfloat16_rn(up * (gate / (1.0f + __expf(-gate))));
            }
        } else {
            for (int i = threadIdx.x; i < ROWS * NT * 8; i += CONSUMERS) {
                const int token = i >> 4, r = i & 15;
                if (token >= p.M || r >= rows) continue;
                float total = 0.f;
#pragma unroll
                for (int w = 0; w < COMPUTE_WARPS; ++w) total += sums[((size_t)w * ROWS + r) * SUMS_W + token];
                float* dst = reinterpret_cast<float*>(out) + (size_t)token * ldo + b0 + r;
                if (EPI == EPI_STORE_SCALED) *dst = total * ctl->inv_rms[token];
                else *dst = __ldcg(dst) + p.residual_scale * total;
            }
        }
        if (SUMS_BUFFERS == 1) consumer_sync();
    }
}

// Where in the side region a norm's weight is kept while the staged activations use its front (null: no room).
__device__ __forceinline__ uint8_t* norm_slot(const StackParams& p, int weight_f32, uint8_t* side, int pitch) {
    const int bytes = p.H * (weight_f32 ? 4 : 2);
    return (long long)p.M * pitch + bytes <= SIDE_BYTES ? side + SIDE_BYTES - bytes : nullptr;
}
// Ask for a norm's weight a phase before it is needed: it comes from HBM, and a miss issued while the
// weights stream waits behind them for microseconds.  All consumer threads call this; stage_normed waits.
__device__ void fetch_norm(const StackParams& p, const void* weight, int weight_f32, uint8_t* side, int pitch) {
    uint8_t* slot = norm_slot(p, weight_f32, side, pitch);
    if (slot) {
        const int bytes = p.H * (weight_f32 ? 4 : 2);
        for (int at = threadIdx.x * 16; at < bytes; at += CONSUMERS * 16)
            cp_async_16(smem_u32(slot + at), reinterpret_cast<const uint8_t*>(weight) + at, true);
    }
    cp_async_commit();
}

// ---- phases A and D: stage bf16(x * w_norm) in shared memory, 1/sqrt(mean(x^2) + eps) per token.
//      A warp owns a token: its loads are all in flight at once and the sum needs no other warp;
//      the order of the additions depends on the width alone. ----
__device__ void stage_normed(const StackParams& p, const void* weight, int weight_f32, uint8_t* side, int pitch, Control* ctl) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quads = p.H >> 2;
    const uint8_t* slot = norm_slot(p, weight_f32, side, pitch);
    cp_async_wait<0>();                                  // fetch_norm's copies
    consumer_sync();
    if (slot) weight = slot;
    for (int token = warp; token < p.M; token += COMPUTE_WARPS) {
        const float4* row = reinterpret_cast<const float4*>(p.h + (size_t)token * p.H);
        float sum = 0.f;
        for (int q0 = 0; q0 < quads; q0 += 32 * 8) {
            float4 v[8], w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {               // the norm's weight and the row: sixteen loads in flight
                const int q = q0 + j * 32 + lane;
                if (q < quads) {
                    if (weight_f32) {
                        w[j] = reinterpret_cast<const float4*>(weight)[q];
                    } else {
                        const uint2 raw = reinterpret_cast<const uint2*>(weight)[q];
                        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                        w[j] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
                    }
                    v[j] = __ldcg(row + q);
                } else {
                    v[j] = w[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int q = q0 + j * 32 + lane;
                if (q >= quads) continue;
                sum = fmaf(v[j].x, v[j].x, sum); sum = fmaf(v[j].y, v[j].y, sum);
                sum = fmaf(v[j].z, v[j].z, sum); sum = fmaf(v[j].w, v[j].w, sum);
                uint2 packed;
                packed.x = pack_bf16(v[j].x * w[j].x, v[j].y * w[j].y);
                packed.y = pack_bf16(v[j].z * w[j].z, v[j].w * w[j].w);
                *reinterpret_cast<uint2*>(side + (size_t)token * pitch + (size_t)q * 8) = packed;
            }
        }
        sum = warp_sum(sum);
        if (lane == 0) ctl->inv_rms[token] = 1.0f / sqrtf(sum / (float)p.H + p.eps);
    }
    consumer_sync();
}

// ---- phase B: one (token, kv head, range of keys), by warps 0..3 ----
template <int D>
__device__ void attend(const StackParams& p, const LayerParams& L, uint8_t* side, Control* ctl, int token, int kvh, int split) {
    using T = Tile<D>;
    constexpr int CHUNKS = T::CHUNKS;
    constexpr int ROWS_PER_PASS = ATTN_WARPS * 32 / CHUNKS;
    constexpr int PASSES = TILE_KEYS / ROWS_PER_PASS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int slot = ctl->slots[token];
    if (slot < 0) return;
    const int group = p.nq / p.nkv;                         // at most 16 (checked on the host)
    const int h0 = kvh * group;
    const int pos = ctl->positions[token];
    const int first = (L.window > 0 && pos - L.window + 1 > 0) ? pos - L.window + 1 : 0;
    const int span = pos + 1 - first;
    const int split_len = ((span + p.n_splits - 1) / p.n_splits + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS;
    const int used = min(p.n_splits, (span + split_len - 1) / split_len);
    const int key_begin = first + split * split_len;
    const int key_end = min(pos + 1, key_begin + split_len);
    if (key_begin >= key_end) return;
    const int* table = L.block_table + (size_t)slot * L.table_stride;
    const int width = (p.nq + 2 * p.nkv) * D;
    const float* row = p.qkv + (size_t)token * width;
    const int half = p.rotary_dim / 2;
    const float2* rotation = ctl->rotation + (size_t)token * half;
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(side + ATTN_STAGES * 2 * T::BYTES);      // [16][D]

    // ---- tiles of 64 keys through two stages ----
    const uint32_t smem_base = smem_u32(side);
    const int sub = lane / CHUNKS, piece = lane % CHUNKS;
    const int row_base = warp * (32 / CHUNKS) + sub;
    const uint32_t piece_offset = T::offset(row_base, piece);
    auto load_tile = [&](int stage, int key0) {
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES + piece_offset, vs = ks + T::BYTES;
        int my_row = -1;
        if (piece < PASSES) {
            const int key = key0 + row_base + piece * ROWS_PER_PASS;
            if (key < key_end) {
                const int page = L.page_shift >= 0 ? key >> L.page_shift : key / L.page_size;
                my_row = table[page] * L.page_size + (key - page * L.page_size);
            }
        }
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const int r = __shfl_sync(0xffffffffu, my_row, sub * CHUNKS + i);
            const bool valid = r >= 0;
            const size_t src = ((size_t)(valid ? r : 0) * p.nkv + kvh) * D + piece * 8;
            cp_async_16(ks + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), L.k_pages + src, valid);
            cp_async_16(vs + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), L.v_pages + src, valid);
        }
    };
    const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;
    // keys of earlier steps depend on nothing this step computes: the first tile is asked for before the
    // positions are encoded, unless it holds the key that is appended below
    const bool early = key_begin + TILE_KEYS <= pos;
    if (early) {
        load_tile(0, key_begin);
        cp_async_commit();
    }

    // ---- rotary positions for this group's queries; the CTA of the last range also appends k and v ----
    for (int w = tid; w < 16 * D; w += ATTN_WARPS * 32) q_s[w] = __float2bfloat16_rn(0.f);
    attention_sync();
    for (int w = tid; w < group * half; w += ATTN_WARPS * 32) {
        const int r = w / half, i = w % half;
        const float2 rot = rotation[i];
        const float cs = rot.x, sn = rot.y;
        const float a = __ldcg(row + (h0 + r) * D + i), b = __ldcg(row + (h0 + r) * D + i + half);
        q_s[r * D + i] = __float2bfloat16_rn(a * cs - b * sn);
        q_s[r * D + i + half] = __float2bfloat16_rn(b * cs + a * sn);
    }
    for (int w = tid; w < group * (D - p.rotary_dim); w += ATTN_WARPS * 32) {
        const int r = w / (D - p.rotary_dim), i = p.rotary_dim + w % (D - p.rotary_dim);
        q_s[r * D + i] = __float2bfloat16_rn(__ldcg(row + (h0 + r) * D + i));
    }
    if (key_end == pos + 1 && L.write_kv) {
        const int page_index = L.page_shift >= 0 ? pos >> L.page_shift : pos / L.page_size;
        const int page = table[page_index];
        if (page < 0 || page >= L.num_pages) {
            if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 2);
        } else {
            const size_t cache_row = (((size_t)page * L.page_size + (pos - page_index * L.page_size)) * p.nkv + kvh) * D;
            const float* k = row + (p.nq + kvh) * D;
            const float* v = row + (p.nq + p.nkv + kvh) * D;
            for (int i = tid; i < half; i += ATTN_WARPS * 32) {
                const float2 rot = rotation[i];
                const float cs = rot.x, sn = rot.y;
                const float a = __ldcg(k + i), b = __ldcg(k + i + half);
                L.k_pages[cache_row + i] = __float2bfloat16_rn(a * cs - b * sn);
                L.k_pages[cache_row + i + half] = __float2bfloat16_rn(b * cs + a * sn);
            }
            for (int i = p.rotary_dim + tid; i < D; i += ATTN_WARPS * 32) L.k_pages[cache_row + i] = __float2bfloat16_rn(__ldcg(k + i));
            for (int i = tid; i < D; i += ATTN_WARPS * 32) L.v_pages[cache_row + i] = __float2bfloat16_rn(__ldcg(v + i));
            __threadfence();                                  // the row is read back below, past L1
        }
    }
    attention_sync();

    if (!early) {
        load_tile(0, key_begin);
        cp_async_commit();
    }

    uint32_t qf[D / 16][4];
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int col = kk * 16 + c;
            qf[kk][0] = *reinterpret_cast<const uint32_t*>(q_s + r0 * D + col);
            qf[kk][1] = *reinterpret_cast<const uint32_t*>(q_s + (r0 + 8) * D + col);
            qf[kk][2] = *reinterpret_cast<const uint32_t*>(q_s + r0 * D + col + 8);
            qf[kk][3] = *reinterpret_cast<const uint32_t*>(q_s + (r0 + 8) * D + col + 8);
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    const int lm = lane >> 3;
    const int k_row = warp * 16 + (lm >> 1) * 8 + (lane & 7), v_row = warp * 16 + (lm & 1) * 8 + (lane & 7);

    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) load_tile((tile + 1) & 1, key_begin + (tile + 1) * TILE_KEYS);
        cp_async_commit();
        cp_async_wait<1>();
        attention_sync();
        const uint32_t ks = smem_base + (uint32_t)(tile & 1) * 2 * T::BYTES, vs = ks + T::BYTES;
        const int key0 = key_begin + tile * TILE_KEYS + warp * 16;
        if (key0 < key_end) {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(ks + T::offset(k_row, kk * 2 + (lm & 1)), b0, b1, b2, b3);
                mma_bf16(s[0], qf[kk], b0, b1);
                mma_bf16(s[1], qf[kk], b2, b3);
            }
            if (key0 + 16 > key_end) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (key0 + nt * 8 + (lane & 3) * 2 + (i & 1) >= key_end) s[nt][i] = -INFINITY;
            }
            float tile_max[2];
            tile_max[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            tile_max[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            float correction[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
                const float new_max = fmaxf(row_max[r], ceilf(tile_max[r] * p.scale_log2));      // a whole number: see the decode kernel
                correction[r] = exp2_whole(row_max[r] - new_max);
                row_max[r] = new_max;
                row_sum[r] *= correction[r];
            }
            uint32_t pf[4];
            {
                float e[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        e[nt][i] = ex2_approx(fmaf(s[nt][i], p.scale_log2, -row_max[i >> 1]));
                        row_sum[i >> 1] += e[nt][i];
                    }
                pf[0] = pack_bf16(e[0][0], e[0][1]);
                pf[1] = pack_bf16(e[0][2], e[0][3]);
                pf[2] = pack_bf16(e[1][0], e[1][1]);
                pf[3] = pack_bf16(e[1][2], e[1][3]);
            }
            if (__any_sync(0xffffffffu, correction[0] != 1.f || correction[1] != 1.f)) {
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    o[j][0] *= correction[0]; o[j][1] *= correction[0]; o[j][2] *= correction[1]; o[j][3] *= correction[1];
                }
            }
#pragma unroll
            for (int j = 0; j < D / 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vs + T::offset(v_row, j + (lm >> 1)), b0, b1, b2, b3);
                mma_bf16(o[j], pf, b0, b1);
                mma_bf16(o[j + 1], pf, b2, b3);
            }
        }
        attention_sync();          // the stage is free for the tile after next
    }
    cp_async_wait<0>();

    // ---- merge the four warps, then the ranges ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    float* merge_o = reinterpret_cast<float*>(side);                  // [4][16][D]
    float* merge_m = merge_o + ATTN_WARPS * 16 * D;
    float* merge_l = merge_m + ATTN_WARPS * 16;
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            float* dst = merge_o + ((size_t)warp * 16 + r0) * D + j * 8 + c;
            dst[0] = o[j][0]; dst[1] = o[j][1];
            dst[8 * D] = o[j][2]; dst[8 * D + 1] = o[j][3];
        }
        if ((lane & 3) == 0) {
            merge_m[warp * 16 + r0] = row_max[0]; merge_m[warp * 16 + r0 + 8] = row_max[1];
            merge_l[warp * 16 + r0] = row_sum[0]; merge_l[warp * 16 + r0 + 8] = row_sum[1];
        }
    }
    attention_sync();
    for (int idx = tid; idx < group * D; idx += ATTN_WARPS * 32) {
        const int r = idx / D, dcol = idx % D;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) top = fmaxf(top, merge_m[w * 16 + r]);
        float total = 0.f, value = 0.f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) {
            const float f = exp2_whole(merge_m[w * 16 + r] - top);
            total += f * merge_l[w * 16 + r];
            value += f * merge_o[((size_t)w * 16 + r) * D + dcol];
        }
        const float result = value / total;
        const int h = h0 + r;
        if (p.n_splits == 1) {
            p.attn[((size_t)token * p.nq + h) * D + dcol] = __float2bfloat16_rn(result);
        } else {
            const size_t at = ((size_t)token * p.nq + h) * p.n_splits + split;
            p.partial[at * D + dcol] = result;
            if (dcol == 0) p.partial[(size_t)p.M * p.nq * p.n_splits * D + at] = top + log2f(total);
        }
    }
    if (p.n_splits == 1) { attention_sync(); return; }
    int* counter = p.counters + token * p.nkv + kvh;
    __threadfence();
    attention_sync();
    if (tid == 0) {
        const int seen = atomicAdd(counter, 1);
        ctl->last_flag = seen == used - 1;
        if (seen == used - 1) *counter = 0;
    }
    attention_sync();
    const bool last = ctl->last_flag != 0;
    attention_sync();                                                 // last_flag may be rewritten by the next item
    if (!last) return;
    __threadfence();
    float* weight = reinterpret_cast<float*>(side);                   // [16][used], then [16] totals
    float* totals = weight + 16 * used;
    const float* lse = p.partial + (size_t)p.M * p.nq * p.n_splits * D;
    for (int r = warp; r < group; r += ATTN_WARPS) {
        const float* base = lse + ((size_t)token * p.nq + h0 + r) * p.n_splits;
        float top = -INFINITY;
        for (int s = lane; s < used; s += 32) top = fmaxf(top, __ldcg(base + s));
        top = warp_max(top);
        float total = 0.f;
        for (int s = lane; s < used; s += 32) {
            const float f = exp2f(__ldcg(base + s) - top);
            weight[r * used + s] = f;
            total += f;
        }
        total = warp_sum(total);
        if (lane == 0) totals[r] = total;
    }
    attention_sync();
    for (int idx = tid; idx < group * (D / 4); idx += ATTN_WARPS * 32) {
        const int r = idx / (D / 4), c4 = idx % (D / 4);
        const float4* base = reinterpret_cast<const float4*>(p.partial + ((size_t)token * p.nq + h0 + r) * p.n_splits * D) + c4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s0 = 0; s0 < used; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = s0 + j < used ? __ldcg(base + (size_t)(s0 + j) * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w = s0 + j < used ? weight[r * used + s0 + j] : 0.f;
                acc[0] += w * v[j].x; acc[1] += w * v[j].y; acc[2] += w * v[j].z; acc[3] += w * v[j].w;
            }
        }
        const float inv = 1.0f / totals[r];
        uint2 packed;
        packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
        packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(p.attn + ((size_t)token * p.nq + h0 + r) * D + c4 * 4) = packed;
    }
    attention_sync();
}

template <int D, int NT>
__global__ void __launch_bounds__(THREADS, 1)
decode_stack_kernel(StackParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint8_t* side = smem + RING * STAGE_BYTES;
    float* sums = reinterpret_cast<float*>(side + SIDE_BYTES);                       // [2 or 1][8][16][NT * 8 + 1]
    Control* ctl = reinterpret_cast<Control*>(side + SIDE_BYTES + (NT == 1 ? 2 : 1) * COMPUTE_WARPS * ROWS * (NT * 8 + 1) * 4);
    LayerParams* layers = reinterpret_cast<LayerParams*>(reinterpret_cast<uint8_t*>(ctl) + ((sizeof(Control) + 15) / 16) * 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const int words = p.n_layers * (int)(sizeof(LayerParams) / 4);
        const int* src = reinterpret_cast<const int*>(p.layers);
        int* dst = reinterpret_cast<int*>(layers);
        for (int i = threadIdx.x; i < words; i += THREADS) dst[i] = src[i];
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < RING; ++i) {
            mbar_init(smem_u32(&ctl->full_bar[i]), 1);
            mbar_init(smem_u32(&ctl->empty_bar[i]), COMPUTE_WARPS);
        }
        ctl->barrier_base = p.barrier[1];
        ctl->abort_flag = 0;
        ctl->last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < p.M) {
        ctl->positions[threadIdx.x] = p.positions[threadIdx.x];
        ctl->slots[threadIdx.x] = p.slots[threadIdx.x];
    }
    float2* rotation = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(layers) + (size_t)MAX_LAYERS * sizeof(LayerParams));
    if (threadIdx.x == 0) ctl->rotation = rotation;
    for (int w = threadIdx.x; w < p.M * (p.rotary_dim / 2); w += THREADS) {
        const int token = w / (p.rotary_dim / 2), i = w % (p.rotary_dim / 2);
        float sn, cs;
        sincosf((float)p.positions[token] * p.inv_freq[i], &sn, &cs);
        rotation[w] = make_float2(cs, sn);
    }
    __syncthreads();
    const int qkv_rows = (p.nq + 2 * p.nkv) * D;

    if (warp == COMPUTE_WARPS) {
        // ---- the producer: every weight of every layer, in the order of use ----
        {
            uint32_t it = 0;
            bool ok = true;
            const int n_products = 4 * p.n_layers;
            auto product = [&](int index) {
                const LayerParams& L = layers[index >> 2];
                switch (index & 3) {
                    case 0: return Product{L.wqkv, qkv_rows, p.H, p.H, 0};
                    case 1: return Product{L.wo, p.H, p.nq * D, p.nq * D, 0};
                    case 2: return Product{L.wgu, p.I, p.H, p.H, 1};
                    default: return Product{L.wd, p.H, p.I, p.I, 0};
                }
            };
            for (int index = 0; index < n_products && ok; ++index) produce(product(index), ring, ctl, it, ok);
            if (!ok && lane == 0) {
                // a consumer gave up (or a copy never came): wait, bounded, for the copies still in flight
                if (!ctl->abort_flag && p.error_flag) atomicExch(p.error_flag, 3);
                for (uint32_t i = it > RING ? it - RING : 0; i < it; ++i)
                    mbar_wait(smem_u32(&ctl->full_bar[i % RING]), (i / RING) & 1u);
            }
        }
        return;
    }

    uint32_t it = 0, n_barrier = 0, n_block = 0;
    bool ok = true;
    const int x_pitch = p.H * 2 + 64;
    fetch_norm(p, layers[0].norm1, layers[0].norm_f32, side, x_pitch);
    for (int l = 0; l < p.n_layers; ++l) {
        const LayerParams& L = layers[l];
        long long* mark = (p.timeline && blockIdx.x == 0 && threadIdx.x == 0) ? p.timeline + l * 16 : nullptr;
        if (mark) mark[0] = global_ns();
        // ---- A: qkv = rmsnorm(x) Wqkv^T ----
        stage_normed(p, L.norm1, L.norm_f32, side, x_pitch, ctl);
        if (mark) mark[1] = global_ns();
        {
            const Product a = {L.wqkv, qkv_rows, p.H, p.H, 0};
            consume<NT, EPI_STORE_SCALED>(p, a, ring, ctl, sums, side, x_pitch, nullptr, 0, p.qkv, qkv_rows, it, n_block, ok);
        }
        if (mark) mark[2] = global_ns();
        if (!ok || !grid_sync(p, ctl, n_barrier)) break;
        if (mark) mark[3] = global_ns();
        // ---- B: positions, cache append, attention ----
        if (warp < ATTN_WARPS) {
            const int items = p.M * p.nkv * p.n_splits;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int split = item % p.n_splits, kvh = (item / p.n_splits) % p.nkv, token = item / (p.n_splits * p.nkv);
                attend<D>(p, L, side, ctl, token, kvh, split);
            }
        }
        if (mark) mark[4] = global_ns();
        if (!grid_sync(p, ctl, n_barrier)) break;
        if (mark) mark[5] = global_ns();
        // ---- C: x += s * attn Wo^T ----
        fetch_norm(p, L.norm2, L.norm_f32, side, x_pitch);        // for phase D; the side region is free from here to there
        {
            const Product c = {L.wo, p.H, p.nq * D, p.nq * D, 0};
            consume<NT, EPI_ACCUM>(p, c, ring, ctl, sums, nullptr, 0, p.attn, p.nq * D, p.h, p.H, it, n_block, ok);
        }
        if (mark) mark[6] = global_ns();
        if (!ok || !grid_sync(p, ctl, n_barrier)) break;
        if (mark) mark[7] = global_ns();
        // ---- D: act = swiglu(rmsnorm(x) Wgu^T) ----
        stage_normed(p, L.norm2, L.norm_f32, side, x_pitch, ctl);
        if (mark) mark[8] = global_ns();
        {
            const Product d = {L.wgu, p.I, p.H, p.H, 1};
            consume<NT, EPI_SWIGLU_SCALED>(p, d, ring, ctl, sums, side, x_pitch, nullptr, 0, p.act, p.I, it, n_block, ok);
        }
        if (mark) mark[9] = global_ns();
        if (!ok || !grid_sync(p, ctl, n_barrier)) break;
        if (mark) mark[10] = global_ns();
        // ---- E: x += s * act Wd^T ----
        if (l + 1 < p.n_layers) fetch_norm(p, layers[l + 1].norm1, layers[l + 1].norm_f32, side, x_pitch);
        {
            const Product e = {L.wd, p.H, p.I, p.I, 0};
            consume<NT, EPI_ACCUM>(p, e, ring, ctl, sums, nullptr, 0, p.act, p.I, p.h, p.H, it, n_block, ok);
        }
        if (mark) mark[11] = global_ns();
        if (!ok || !grid_sync(p, ctl, n_barrier)) break;
        if (mark) mark[12] = global_ns();
    }
    if (!ok && threadIdx.x == 0) {
        ctl->abort_flag = 1;
        if (p.error_flag) atomicExch(p.error_flag, 3);
    }
    // the next launch counts its barriers from here (every CTA has read the old base long ago)
    if (blockIdx.x == 0 && threadIdx.x == 0 && ok && !ctl->abort_flag)
        p.barrier[1] = ctl->barrier_base + (unsigned long long)n_barrier * gridDim.x;
}

template <int D, int NT>
int launch_stack(const StackParams& p, int grid, cudaStream_t stream) {
    const size_t smem = (size_t)RING * STAGE_BYTES + SIDE_BYTES + (size_t)(NT == 1 ? 2 : 1) * COMPUTE_WARPS * ROWS * (NT * 8 + 1) * 4 + ((sizeof(Control) + 15) / 16) * 16 +
                        (size_t)MAX_LAYERS * sizeof(LayerParams) + (size_t)MAX_TOKENS * 64 * sizeof(float2) + 128;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(decode_stack_kernel<D, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)grid);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
    if (cudaLaunchKernelEx(&config, decode_stack_kernel<D, NT>, p) != cudaSuccess) {
        cudaGetLastError();
        return LIA_ERR_LAUNCH;
    }
    return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
}
}  // namespace

// Bytes of one LayerParams record, so that the caller can lay the array out without knowing the struct.
LIA_EXPORT int lia_decode_stack_layer_bytes() { return (int)sizeof(LayerParams); }

// Writes record `index` of the layer array that `host_layers` points to (host memory; the caller copies the
// finished array to the device once).
LIA_EXPORT int lia_decode_stack_set_layer(void* host_layers, int index, const void* norm1, const void* norm2, int norm_f32,
                                          const void* wqkv, const void* wo, const void* wgu, const void* wd, void* k_pages,
                                          void* v_pages, const int* block_table, int table_stride, int page_size,
                                          int num_pages, int window, int write_kv) {
    if (!host_layers || index < 0 || page_size <= 0) return LIA_ERR_SIZE;
    LayerParams& L = reinterpret_cast<LayerParams*>(host_layers)[index];
    L.norm1 = norm1; L.norm2 = norm2; L.norm_f32 = norm_f32;
    L.wqkv = (const __nv_bfloat16*)wqkv; L.wo = (const __nv_bfloat16*)wo;
    L.wgu = (const __nv_bfloat16*)wgu; L.wd = (const __nv_bfloat16*)wd;
    L.k_pages = (__nv_bfloat16*)k_pages; L.v_pages = (__nv_bfloat16*)v_pages;
    L.block_table = block_table; L.table_stride = table_stride; L.page_size = page_size;
    L.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if (page_size == (1 << b)) L.page_shift = b;
    L.num_pages = num_pages; L.window = window; L.write_kv = write_kv; L.pad = 0;
    return LIA_OK;
}

// Most layers one launch takes.
LIA_EXPORT int lia_decode_stack_max_layers() { return MAX_LAYERS; }

// Whether the stack kernel takes these sizes (1) or the caller must use the per-part kernels (0).
LIA_EXPORT int lia_decode_stack_accepts(int M, int H, int nq, int nkv, int d, int I, int rotary_dim, int n_splits) {
    if (M < 1 || M > MAX_TOKENS || (d != 64 && d != 128)) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv || nq / nkv > 16) return 0;
    if (H <= 0 || H % 8 || I <= 0 || I % 8 || (nq * d) % 8) return 0;                // 16-byte rows for the bulk copies
    if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1)) return 0;
    if (n_splits < 1 || n_splits > MAX_SPLITS) return 0;
    if ((long long)M * (H * 2 + 64) > SIDE_BYTES) return 0;                          // the staged activations must fit
    if (ATTN_STAGES * 2 * TILE_KEYS * d * 2 + 16 * d * 2 > SIDE_BYTES) return 0;
    return 1;
}

// Runs `n_layers` layers on M tokens (every one a decoded token: one new position per request).
// `layers`: device array of records written with lia_decode_stack_set_layer.  `barrier`: two 64-bit words,
// zero before the first launch (and again after an error).  `counters`: M * nkv int32, zero.
// `partial`: M * nq * n_splits * (d + 1) floats, 16-byte aligned.  `grid`: CTAs, at most one per SM.
// `timeline` (optional, n_layers * 16 64-bit words): CTA 0 writes its clock in ns at the start of each layer,
// after the parts of each phase and after each grid barrier (13 marks), for profiling.
LIA_EXPORT int lia_decode_stack(const void* layers, int n_layers, int M, int H, int nq, int nkv, int d, int I,
                                int rotary_dim, const float* inv_freq, float eps, float residual_scale, float attn_scale,
                                float* h, float* qkv, void* attn, void* act, float* partial, int n_splits, int* counters,
                                const int* positions, const int* slots, unsigned long long* barrier, int* error_flag,
                                long long* timeline, int grid, cudaStream_t stream) {
    if (n_layers <= 0 || M <= 0) return LIA_OK;
    if (n_layers > MAX_LAYERS) return LIA_ERR_SIZE;
    if (!lia_decode_stack_accepts(M, H, nq, nkv, d, I, rotary_dim, n_splits) || grid <= 0) return LIA_ERR_SIZE;
    if (rotary_dim > 0 && !inv_freq) return LIA_ERR_SIZE;
    if (((uintptr_t)h & 15u) || ((uintptr_t)attn & 15u) || ((uintptr_t)act & 15u) || ((uintptr_t)partial & 15u)) return LIA_ERR_ALIGN;
    StackParams p;
    p.layers = (const LayerParams*)layers; p.n_layers = n_layers; p.M = M; p.H = H; p.nq = nq; p.nkv = nkv; p.I = I;
    p.rotary_dim = rotary_dim; p.n_splits = n_splits; p.eps = eps; p.residual_scale = residual_scale;
    p.scale_log2 = attn_scale * LOG2E; p.inv_freq = inv_freq; p.h = h; p.qkv = qkv;
    p.attn = (__nv_bfloat16*)attn; p.act = (__nv_bfloat16*)act; p.partial = partial; p.counters = counters;
    p.positions = positions; p.slots = slots; p.barrier = barrier; p.error_flag = error_flag; p.timeline = timeline;
    if (d == 128) return M <= 8 ? launch_stack<128, 1>(p, grid, stream) : launch_stack<128, 2>(p, grid, stream);
    return M <= 8 ? launch_stack<64, 1>(p, grid, stream) : launch_stack<64, 2>(p, grid, stream);
}
