// Causal attention of prompt portions over the paged bfloat16 cache, on the tensor cores.
//
// The query heads of one kv head are packed along the MMA's M together with consecutive tokens:
// a CTA owns 64 rows = floor(64 / g) tokens x g heads (g = heads per kv head) of one portion and one
// kv head, 16 rows per warp.  It walks the keys from the first one any of its rows can see to the
// last, 64 at a time, through a cp.async ring in shared memory that all four warps share:
// S = Q K^T (bf16 mma.sync, 32-bit accumulate), mask by each row's own position (and window), running
// maximum and sum in 32-bit with base-2 exponentials, P in bf16 against V.  The keys of a portion's
// own tokens were appended to the cache before this kernel runs, so earlier portions and the current
// one are read the same way, and a portion may start and end anywhere.
//
// Portions are described by `segments` [n_segments][3] = (index of the portion's first token in the
// batch, its position, its token count); CTA x finds its portion and token range by walking that list.
#include "attention_tc.cuh"

using namespace attn;

namespace {
constexpr int ROWS = 64;                 // query rows per CTA
constexpr int PREFILL_STAGES = 3;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^n for a whole number n <= 0 (or -infinity), exactly.
__device__ __forceinline__ float exp2_whole(float n) {
    return n < -126.f ? 0.f : __int_as_float(((int)n + 127) << 23);
}

struct PrefillParams {
    const __nv_bfloat16* q;          // [tokens, nq, D]
    const __nv_bfloat16* k_pages;    // [pages, page_size, nkv, D]
    const __nv_bfloat16* v_pages;
    const int* segments;             // [n_segments][3]
    const int* slots;                // [tokens]
    const int* block_table;          // [slots, table_stride]
    __nv_bfloat16* out;              // [tokens, nq, D]
    int n_segments, table_stride, nq, nkv, page_size, page_shift, window, tokens_per_tile;
    float scale_log2;
    int num_pages;
    int* error_flag;                 // raised to 2 when a visible key has no page
};

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_prefill_kernel(PrefillParams p) {
    using T = Tile<D>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.nq / p.nkv;
    const int kvh = blockIdx.y;

    // ---- which portion, which tokens (later tiles first: they have the most keys) ----
    int tile = gridDim.x - 1 - blockIdx.x, seg = 0, q_offset = 0, seg_start = 0, seg_count = 0;
    for (; seg < p.n_segments; ++seg) {
        q_offset = p.segments[seg * 3];
        seg_start = p.segments[seg * 3 + 1];
        seg_count = p.segments[seg * 3 + 2];
        const int tiles = (seg_count + p.tokens_per_tile - 1) / p.tokens_per_tile;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (seg >= p.n_segments) return;
    const int tok0 = tile * p.tokens_per_tile;
    const int tok_count = min(p.tokens_per_tile, seg_count - tok0);
    pdl_launch_dependents();
    const int slot = p.slots[q_offset];
    if (slot < 0) return;
    pdl_wait();                                   // q and this step's keys come from the kernel ahead
    const int* table = p.block_table + (size_t)slot * p.table_stride;
    const int pos_first = seg_start + tok0, pos_last = pos_first + tok_count - 1;
    const int key_begin = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int key_end = pos_last + 1;

    // ---- this thread's two rows: r -> (token, head) ----
    int row_pos[2];
    const __nv_bfloat16* q_row[2];
    __nv_bfloat16* o_row[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + (lane >> 2) + i * 8;
        const int tok = r / group, head = r % group;
        row_ok[i] = tok < tok_count;
        const int token_index = q_offset + tok0 + (row_ok[i] ? tok : 0);
        row_pos[i] = row_ok[i] ? pos_first + tok : 0x3fffffff;      // a row beyond the portion sees every key and is never written
        const size_t at = ((size_t)token_index * p.nq + kvh * group + head) * D;
        q_row[i] = p.q + at;
        o_row[i] = p.out + at;
    }
    uint32_t qf[D / 16][4];
    {
        const int c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int col = kk * 16 + c;
            qf[kk][0] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q_row[0] + col) : 0u;
            qf[kk][1] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q_row[1] + col) : 0u;
            qf[kk][2] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q_row[0] + col + 8) : 0u;
            qf[kk][3] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q_row[1] + col + 8) : 0u;
        }
    }
    // the warp's rows see keys up to warp_last (tiles beyond it are skipped by the warp); a tile whose keys all
    // lie at or before warp_first, and inside every row's window, needs no mask
    int warp_last = max(row_ok[0] ? row_pos[0] : -1, row_ok[1] ? row_pos[1] : -1), warp_first = min(row_pos[0], row_pos[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        warp_last = max(warp_last, __shfl_xor_sync(0xffffffffu, warp_last, o));
        warp_first = min(warp_first, __shfl_xor_sync(0xffffffffu, warp_first, o));
    }

    // ---- loading a tile: CHUNKS lanes share a key row; lane j of them looks up the row of pass j ----
    constexpr int CHUNKS = T::CHUNKS;
    constexpr int ROWS_PER_PASS = WARPS * 32 / CHUNKS;
    constexpr int PASSES = TILE_KEYS / ROWS_PER_PASS;
    static_assert(ROWS_PER_PASS % 8 == 0 && PASSES <= CHUNKS, "the swizzle repeats every 8 rows; one lane per pass");
    const uint32_t smem_base = smem_u32(smem);
    const int sub = lane / CHUNKS, piece = lane % CHUNKS;
    const int row_base = warp * (32 / CHUNKS) + sub;
    const uint32_t piece_offset = T::offset(row_base, piece);
    auto load_tile = [&](int stage, int key0) {
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES + piece_offset, vs = ks + T::BYTES;
        int my_row = -1;
        if (piece < PASSES) {
            const int key = key0 + row_base + piece * ROWS_PER_PASS;
            if (key < key_end) my_row = cache_row_of(table, key, p.page_size, p.page_shift, p.num_pages, p.error_flag);
        }
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const int r = __shfl_sync(0xffffffffu, my_row, sub * CHUNKS + i);
            const bool valid = r >= 0;
            const size_t src = ((size_t)(valid ? r : 0) * p.nkv + kvh) * D + piece * 8;
            cp_async_16(ks + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), p.k_pages + src, valid);
            cp_async_16(vs + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), p.v_pages + src, valid);
        }
    };

    const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;
#pragma unroll
    for (int s = 0; s < PREFILL_STAGES - 1; ++s) {
        if (s < n_tiles) load_tile(s, key_begin + s * TILE_KEYS);
        cp_async_commit();
    }

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};

    for (int kt = 0; kt < n_tiles; ++kt) {
        cp_async_wait<PREFILL_STAGES - 2>();
        __syncthreads();
        {
            const int next = kt + PREFILL_STAGES - 1;
            if (next < n_tiles) load_tile(next % PREFILL_STAGES, key_begin + next * TILE_KEYS);
            cp_async_commit();
        }
        const int stage = kt % PREFILL_STAGES;
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES, vs = ks + T::BYTES;
        const int key0 = key_begin + kt * TILE_KEYS;
        if (key0 > warp_last) continue;                     // nothing in this tile is visible to the warp

        // ---- S = Q K^T: 16 rows x 64 keys = 8 n-tiles ----
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int m = lane >> 3;
#pragma unroll
            for (int np = 0; np < 4; ++np) {                 // pairs of n-tiles: 16 keys
                const int row = np * 16 + (m >> 1) * 8 + (lane & 7);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(ks + T::offset(row, kk * 2 + (m & 1)), b0, b1, b2, b3);
                mma_bf16(s[np * 2], qf[kk], b0, b1);
                mma_bf16(s[np * 2 + 1], qf[kk], b2, b3);
            }
        }
        // ---- mask by each row's own position and window, where the tile needs it ----
        if (key0 + TILE_KEYS - 1 > warp_first || (p.window > 0 && key0 <= warp_last - p.window)) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + nt * 8 + (lane & 3) * 2 + (i & 1);
                    const int pos = row_pos[i >> 1];
                    bool visible = key <= pos;
                    if (p.window > 0) visible = visible && key > pos - p.window;
                    if (!visible) s[nt][i] = -INFINITY;
                }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            tile_max[0] = fmaxf(tile_max[0], fmaxf(s[nt][0], s[nt][1]));
            tile_max[1] = fmaxf(tile_max[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float correction[2], safe_max[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
            // whole-number reference point: see attention_decode.cu
            const float new_max = fmaxf(row_max[r], ceilf(tile_max[r] * p.scale_log2));
            // a row that has seen no key yet keeps maximum -inf; exponentials are taken against 0 then
            safe_max[r] = new_max == -INFINITY ? 0.f : new_max;
            correction[r] = exp2_whole(row_max[r] - safe_max[r]);
            row_max[r] = new_max;
            row_sum[r] *= correction[r];
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s[nt][i] = ex2_approx(fmaf(s[nt][i], p.scale_log2, -safe_max[i >> 1]));
                row_sum[i >> 1] += s[nt][i];
            }
        if (__any_sync(0xffffffffu, correction[0] != 1.f || correction[1] != 1.f)) {
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                o[j][0] *= correction[0]; o[j][1] *= correction[0];
                o[j][2] *= correction[1]; o[j][3] *= correction[1];
            }
        }
        // ---- O += P V: four k-steps of 16 keys ----
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[kp * 2][0], s[kp * 2][1]);
            pf[1] = pack_bf16(s[kp * 2][2], s[kp * 2][3]);
            pf[2] = pack_bf16(s[kp * 2 + 1][0], s[kp * 2 + 1][1]);
            pf[3] = pack_bf16(s[kp * 2 + 1][2], s[kp * 2 + 1][3]);
#pragma unroll
            for (int j = 0; j < D / 8; j += 2) {
                const int m = lane >> 3;
                const int row = kp * 16 + (m & 1) * 8 + (lane & 7);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vs + T::offset(row, j + (m >> 1)), b0, b1, b2, b3);
                mma_bf16(o[j], pf, b0, b1);
                mma_bf16(o[j + 1], pf, b2, b3);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!row_ok[i]) continue;
        const float inv = 1.0f / row_sum[i];
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
            *reinterpret_cast<uint32_t*>(o_row[i] + j * 8 + c) = pack_bf16(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
    }
}

template <int D>
int launch_prefill(const PrefillParams& p, int n_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)PREFILL_STAGES * 2 * Tile<D>::BYTES;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    return lia_launch(attention_prefill_kernel<D>, dim3(n_tiles, p.nkv), dim3(WARPS * 32), smem, stream, p);
}
}  // namespace

// How many tokens of a portion one CTA takes for `group` query heads per kv head (0: not supported).
LIA_EXPORT int lia_attention_prefill_tokens_per_tile(int group) {
    return group >= 1 && group <= ROWS ? ROWS / group : 0;
}

// Prompt-portion attention, bfloat16, head_dim 32, 64 or 128, at most 64 query heads per kv head.
// `n_tiles` = sum over portions of ceil(count / tokens_per_tile).
LIA_EXPORT int lia_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* segments,
                                     int n_segments, int n_tiles, const int* slots, const int* block_table,
                                     int table_stride, void* out, int nq, int nkv, int d, int page_size, int window,
                                     float scale, int num_pages, int* error_flag, cudaStream_t stream) {
    if (n_segments <= 0 || n_tiles <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || nkv > 65535) return LIA_ERR_SIZE;
    const int per_tile = lia_attention_prefill_tokens_per_tile(nq / nkv);
    if (per_tile == 0) return LIA_ERR_SIZE;
    PrefillParams p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.segments = segments; p.slots = slots; p.block_table = block_table; p.out = (__nv_bfloat16*)out;
    p.n_segments = n_segments; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
    p.window = window; p.tokens_per_tile = per_tile; p.scale_log2 = scale * LOG2E;
    p.num_pages = num_pages; p.error_flag = error_flag;
    p.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if (page_size == (1 << b)) p.page_shift = b;
    if (d == 128) return launch_prefill<128>(p, n_tiles, stream);
    if (d == 64) return launch_prefill<64>(p, n_tiles, stream);
    if (d == 32) return launch_prefill<32>(p, n_tiles, stream);
    return LIA_ERR_SIZE;
}
