// Decode attention over the paged bfloat16 cache, split over the keys.
//
// One CTA serves one decoded token's query heads of ONE kv head (up to 16 of them, so the keys of a group are
// read once for all its query heads) over ONE range of keys.  Its four warps take 16 keys each of every 64-key
// tile.  The KEYS are the 16 rows of the MMA's M and the heads its N (8, or twice 8): S^T = K Q^T by mma.sync
// (bf16 in, 32-bit out), so a group of 8 heads wastes nothing of the instruction; running maximum and sum per
// head in 32-bit (base-2 exponentials with the scale folded in); P^T in bf16, turned into an operand with
// movmatrix, back into the tensor cores: O^T = V^T P^T.  Keys and values come from their pages through a
// three-stage cp.async ring in shared memory; ldmatrix (transposed for V) builds the fragments.  The
// four warps' partial results are merged in shared memory; the CTA then writes either the final
// output (one range) or a normalised partial output with its log-sum-exp to scratch, which the last CTA of the
// token to finish (or `attention_merge_kernel`) combines.  Ranges are `split_len` keys long, counted from the
// first visible key, so how a token's keys are cut depends on its own position, the window and split_len only.
//
// Where the ranges of a token are few enough (2, 4, 8 or 16) and all clusters fit on the device at once, the CTAs of
// a token's ranges form a thread-block cluster and the ranges meet in DISTRIBUTED SHARED MEMORY instead: every CTA
// leaves its normalised partial output and log-sum-exp in its own shared memory, the cluster synchronises, and
// CTA r combines every S-th piece of the output over all ranges in ascending order and writes it.  That replaces
// three dependent trips (partials to global memory, an atomic, the last CTA reading all partials back: 4-5 us
// of a 13 us kernel at batch 8) by one cluster barrier.
//
// The work of this kernel is streaming the cache: 2 * kv_heads * head_dim * 2 bytes per key and token.
#include "attention_tc.cuh"

using namespace attn;

namespace {
struct Params {
    const __nv_bfloat16* q;          // [tokens, nq, D]
    const __nv_bfloat16* k_pages;    // [pages, page_size, nkv, D]
    const __nv_bfloat16* v_pages;
    const int* rows;                 // [n_rows] batch index of each decoded token (negative: skip)
    const int* positions;            // [tokens]
    const int* slots;                // [tokens]
    const int* block_table;          // [slots, table_stride]
    __nv_bfloat16* out;              // [tokens, nq, D]
    float* partial;                  // [tokens, nq, n_splits, D] normalised outputs, then [tokens, nq, n_splits] log2-sum-exps
    int* counters;                   // [n_rows, gridDim.y], zero between launches; null: ranges are merged by a second kernel
    int n_tokens, table_stride, nq, nkv, page_size, page_shift, window, split_len, n_splits;
    float scale_log2;                // softmax scale * log2(e)
    // position encoding and cache append in the same kernel (qkv non-null): q is taken from qkv, rotated here;
    // the CTA of a token's last range also rotates its new key and appends key and value to their page
    const float* qkv;                // [tokens, (nq + 2 nkv) D] 32-bit
    const float* inv_freq;           // [rotary_dim / 2]
    __nv_bfloat16* k_write;          // the pages again, writable
    __nv_bfloat16* v_write;
    int rotary_dim, write_kv, num_pages;
    int cluster;                     // the CTAs of a token's ranges are one cluster (gridDim.z of them) and merge in shared memory
    int all_new;                     // any of a row's keys may have been written by this step's kernels (rows of prompt portions), not only its own
    int* error_flag;
};

constexpr int MAX_FUSED_SPLITS = 128;     // ranges that the last CTA of a token can merge (its weights lie in shared memory)

// Keys per range for a token that sees `span` keys: the given length, or (split_len 0) the span cut into
// n_splits ranges of a multiple of 64 keys.  The second rule depends on the token's own span and on
// n_splits alone, so a launch captured in a CUDA graph serves every context length.
__device__ __forceinline__ int range_length(const Params& p, int span) {
    if (p.split_len > 0) return p.split_len;
    const int per = (span + p.n_splits - 1) / p.n_splits;
    return (per + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^n for a whole number n <= 0 (or -infinity), exactly.
__device__ __forceinline__ float exp2_whole(float n) {
    return n < -126.f ? 0.f : __int_as_float(((int)n + 127) << 23);
}

__device__ __forceinline__ uint32_t transpose_8x8(uint32_t pair) {       // movmatrix: the 8 x 8 matrix of 16-bit elements a warp holds, transposed
    uint32_t out;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(out) : "r"(pair));
    return out;
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 / 4 bytes of the shared memory of the cluster's CTA `rank`, at the offset that `addr` has in this CTA's.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float ld_cluster_f(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

constexpr int MAX_CLUSTER = 16;
// Where a CTA leaves its range's result for the cluster: [16 heads][D] normalised outputs, then [16] log2-sum-exps
// (minus infinity: the range has no keys), behind the buffers of the four warps' merge.
template <int D> __device__ __forceinline__ float* exchange_of(uint8_t* smem) {
    return reinterpret_cast<float*>(smem) + WARPS * 16 * (D + 4 + 3);
}

// The cluster's CTAs combine their ranges: piece i (four elements of a head) is written by CTA i mod S, which adds
// the ranges in ascending order, so the result does not depend on which CTA finishes when.  Every thread of every
// CTA of the cluster calls this once.
template <int D>
__device__ __forceinline__ void cluster_merge(const Params& p, uint8_t* smem, int t, int h0, int heads) {
    cluster_sync_all();                               // every CTA's result is in its exchange buffer
    const uint32_t rank = cluster_rank();
    const int S = gridDim.z;
    const uint32_t base = smem_u32(exchange_of<D>(smem));
    for (int item = (int)rank + (int)threadIdx.x * S; item < heads * (D / 4); item += S * WARPS * 32) {
        const int r = item / (D / 4), c4 = item % (D / 4);
        float l[MAX_CLUSTER];
        float4 v[MAX_CLUSTER];
#pragma unroll
        for (int c = 0; c < MAX_CLUSTER; ++c) {
            if (c < S) {
                l[c] = ld_cluster_f(base + (uint32_t)((16 * D + r) * 4), (uint32_t)c);
                v[c] = ld_cluster_f4(base + (uint32_t)((r * D + c4 * 4) * 4), (uint32_t)c);
            }
        }
        float top = -INFINITY;
#pragma unroll
        for (int c = 0; c < MAX_CLUSTER; ++c)
            if (c < S) top = fmaxf(top, l[c]);
        float total = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < MAX_CLUSTER; ++c) {
            if (c < S && l[c] > -INFINITY) {            // a range without keys left nothing to read
                const float w = exp2f(l[c] - top);
                total += w;
                acc[0] += w * v[c].x; acc[1] += w * v[c].y; acc[2] += w * v[c].z; acc[3] += w * v[c].w;
            }
        }
        const float inv = total > 0.f ? 1.0f / total : 0.f;
        uint2 packed;
        packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
        packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(p.out + ((size_t)t * p.nq + h0 + r) * D + c4 * 4) = packed;
    }
    cluster_sync_all();                               // nobody leaves while a neighbour may still read its shared memory
}

// NH: groups of 8 query heads per kv head that the CTA serves (1 or 2)
template <int D, int NH>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(Params p) {
    using T = Tile<D>;
    constexpr int CHUNKS = T::CHUNKS;                 // 16-byte pieces per key row = lanes that share a row
    constexpr int ROWS_PER_PASS = WARPS * 32 / CHUNKS; // rows that one cp.async of every thread covers
    constexpr int PASSES = TILE_KEYS / ROWS_PER_PASS;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int last_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    pdl_launch_dependents();
    // The step's metadata and the keys of earlier steps depend on no kernel of this step; only q and the
    // newest key do, so everything up to pdl_wait() below overlaps the kernel ahead.  (Rows that are the last tokens of
    // prompt portions, `all_new`, have keys that this step's kernels wrote anywhere before them: no tile is asked
    // for before the wait.)
    const int t = p.rows[blockIdx.x];
    if (t < 0) return;
    const int slot = p.slots[t];
    if (slot < 0) return;
    const int group = p.nq / p.nkv;
    const int groups16 = (group + 15) / 16;
    const int kvh = blockIdx.y / groups16;
    const int h0 = kvh * group + (blockIdx.y % groups16) * 16;        // first query head of this CTA
    const int heads = min(16, kvh * group + group - h0);
    const int pos = p.positions[t];
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int split_len = range_length(p, pos + 1 - first);
    const int key_begin = first + blockIdx.z * split_len;
    const int key_end = min(pos + 1, key_begin + split_len);
    if (key_begin >= key_end) {
        if (!p.cluster) return;
        float* exchange = exchange_of<D>(smem);       // a range without keys: it says so and stays for the cluster's merge
        if (tid < 16) exchange[16 * D + tid] = -INFINITY;
        cluster_merge<D>(p, smem, t, h0, heads);
        return;
    }
    const int* table = p.block_table + (size_t)slot * p.table_stride;

    // ---- loading a tile: CHUNKS lanes share a key row; lane j of them looks up the row of pass j ----
    const uint32_t smem_base = smem_u32(smem);
    const int sub = lane / CHUNKS, piece = lane % CHUNKS;
    const int row_base = warp * (32 / CHUNKS) + sub;                 // this thread's row in pass 0
    const uint32_t piece_offset = T::offset(row_base, piece);        // later passes: + ROWS_PER_PASS rows, same swizzle
    static_assert(ROWS_PER_PASS % 8 == 0 && PASSES <= CHUNKS, "the swizzle repeats every 8 rows; one lane per pass");
    // `left_out`: a key whose row of the tile no copy touches (this CTA writes it into the tile itself)
    auto load_tile = [&](int stage, int key0, int left_out) {
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES + piece_offset, vs = ks + T::BYTES;
        constexpr int LEFT_OUT = -2147483647 - 1;         // no row of the cache: cache_row_of gives -1 or a row >= 0
        int my_row = -1;
        if (piece < PASSES) {
            const int key = key0 + row_base + piece * ROWS_PER_PASS;
            if (key == left_out) my_row = LEFT_OUT;
            else if (key < key_end) my_row = cache_row_of(table, key, p.page_size, p.page_shift, p.num_pages, p.error_flag);
        }
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const int row = __shfl_sync(0xffffffffu, my_row, sub * CHUNKS + i);
            if (row == LEFT_OUT) continue;
            const bool valid = row >= 0;
            const size_t src = ((size_t)(valid ? row : 0) * p.nkv + kvh) * D + piece * 8;
            cp_async_16(ks + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), p.k_pages + src, valid);
            cp_async_16(vs + (uint32_t)(i * ROWS_PER_PASS * CHUNKS * 16), p.v_pages + src, valid);
        }
    };

    const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;
    // With the append in this kernel, the range that ends at the token's own position holds a key that does not
    // exist yet.  Where its tile (the range's last) is among the first STAGES, the copies leave that row
    // out and this CTA writes the rotated key and the value into the tile itself, beside the cache (`direct`);
    // otherwise the tile is asked for only after the append (and a fence).  A layer that reads another layer's
    // cache (write_kv 0) waits for the step's earlier kernels before it asks for that tile (`deferred`).
    const bool appends = p.qkv != nullptr && key_end == pos + 1;
    const bool writes = appends && p.write_kv && blockIdx.y % groups16 == 0;
    const bool direct = writes && n_tiles <= STAGES;
    int deferred = -1;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {       // the first STAGES tiles are asked for at once: tile i is copy group i
        if (s < n_tiles) {
            const bool holds_new = p.all_new || key_begin + (s + 1) * TILE_KEYS > pos;
            if (holds_new && appends && !direct) {
                deferred = s;
            } else {
                if (holds_new && !appends) pdl_wait();                   // the tile holds the key this step wrote
                load_tile(s, key_begin + s * TILE_KEYS, direct ? pos : -1);
            }
        }
        if (deferred < 0) cp_async_commit();
    }

    // ---- Q fragments: rows = heads (row r -> head h0 + r), zero beyond `heads` ----
    uint32_t qb[D / 16][NH][2];          // Q^T as the MMA's second operand: lane (g, t) holds head g (+ 8), d = 2t, 2t + 1 (+ 8)
    if (p.qkv) {
        __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * 2 * T::BYTES);       // [16][D]
        const int width = (p.nq + 2 * p.nkv) * D;
        const float* row = p.qkv + (size_t)t * width;
        const int half = p.rotary_dim / 2;
        float2* rotation = reinterpret_cast<float2*>(q_s + 16 * D);      // [half] (cos, sin) of the token's angles
        float* raw = reinterpret_cast<float*>(rotation + D / 2);        // [16 + 2][D] the step's 32-bit q, k and v rows
        // the angles and the padding depend on the position alone: before the wait
        for (int i = tid; i < half; i += WARPS * 32) {
            float sn, cs;
            sincosf((float)pos * p.inv_freq[i], &sn, &cs);
            rotation[i] = make_float2(cs, sn);
        }
        for (int w = tid; w < (16 - heads) * D; w += WARPS * 32) q_s[heads * D + w] = __float2bfloat16_rn(0.f);
        const int page_index = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
        const int page = writes ? table[page_index] : 0;
        pdl_wait();
        // The step's rows come in with ONE trip to memory: every thread has all its 16-byte loads in flight
        // before it stores the first.  (Heads of 16 k elements: rows and widths are multiples of 16 bytes.)
        {
            constexpr int PER_THREAD = (18 * D / 4 + WARPS * 32 - 1) / (WARPS * 32);
            const int q4 = heads * (D / 4), all4 = q4 + (writes ? 2 * (D / 4) : 0);
            const float4* q_src = reinterpret_cast<const float4*>(row + (size_t)h0 * D);
            const float4* k_src = reinterpret_cast<const float4*>(row + (size_t)(p.nq + kvh) * D);
            const float4* v_src = reinterpret_cast<const float4*>(row + (size_t)(p.nq + p.nkv + kvh) * D);
            float4 got[PER_THREAD] = {};
#pragma unroll
            for (int j = 0; j < PER_THREAD; ++j) {
                const int w = tid + j * WARPS * 32;
                if (w < q4) got[j] = __ldcg(q_src + w);
                else if (w < q4 + D / 4 && w < all4) got[j] = __ldcg(k_src + (w - q4));
                else if (w < all4) got[j] = __ldcg(v_src + (w - q4 - D / 4));
            }
#pragma unroll
            for (int j = 0; j < PER_THREAD; ++j) {
                const int w = tid + j * WARPS * 32;
                if (w < q4) reinterpret_cast<float4*>(raw)[w] = got[j];
                else if (w < all4) reinterpret_cast<float4*>(raw + 16 * D)[w - q4] = got[j];
            }
        }
        __syncthreads();
        if (p.rotary_dim == D) {
            // the whole head rotates (the usual case): a thread keeps its column, so its angle, and walks the heads
            constexpr int HALF = D / 2, STEP = WARPS * 32 / HALF > 0 ? WARPS * 32 / HALF : 1;
            const int i = tid % HALF;
            const float cs = rotation[i].x, sn = rotation[i].y;
#pragma unroll 4
            for (int r = tid / HALF; r < heads; r += STEP) {
                const float a = raw[r * D + i], b = raw[r * D + i + HALF];
                q_s[r * D + i] = __float2bfloat16_rn(a * cs - b * sn);
                q_s[r * D + i + HALF] = __float2bfloat16_rn(b * cs + a * sn);
            }
        } else {
#pragma unroll 4
            for (int w = tid; w < heads * half; w += WARPS * 32) {
                const int r = w / half, i = w % half;
                const float cs = rotation[i].x, sn = rotation[i].y;
                const float a = raw[r * D + i], b = raw[r * D + i + half];
                q_s[r * D + i] = __float2bfloat16_rn(a * cs - b * sn);
                q_s[r * D + i + half] = __float2bfloat16_rn(b * cs + a * sn);
            }
        }
        for (int w = tid; w < heads * (D - p.rotary_dim); w += WARPS * 32) {
            const int r = w / (D - p.rotary_dim), i = p.rotary_dim + w % (D - p.rotary_dim);
            q_s[r * D + i] = __float2bfloat16_rn(raw[r * D + i]);
        }
        if (writes) {
            if (page < 0 || page >= p.num_pages) {
                if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 2);
                // (a `direct` tile then keeps whatever the row held: the step's results are discarded anyway)
            } else {
                const size_t cache_row = (((size_t)page * p.page_size + (pos - page_index * p.page_size)) * p.nkv + kvh) * D;
                const float* k = raw + 16 * D;
                const float* v = raw + 17 * D;
                // the row of the tile that the copies left out, if this CTA fills it itself
                const int tile_row = pos - key_begin - (n_tiles - 1) * TILE_KEYS;
                uint8_t* k_tile = smem + (size_t)(n_tiles - 1) * 2 * T::BYTES;
                uint8_t* v_tile = k_tile + T::BYTES;
                auto put = [&](__nv_bfloat16* cache, uint8_t* tile, int i, float value) {
                    const __nv_bfloat16 x = __float2bfloat16_rn(value);
                    cache[cache_row + i] = x;
                    if (direct) *reinterpret_cast<__nv_bfloat16*>(tile + T::offset(tile_row, i >> 3) + (i & 7) * 2) = x;
                };
                for (int i = tid; i < half; i += WARPS * 32) {
                    const float cs = rotation[i].x, sn = rotation[i].y;
                    const float a = k[i], b = k[i + half];
                    put(p.k_write, k_tile, i, a * cs - b * sn);
                    put(p.k_write, k_tile, i + half, b * cs + a * sn);
                }
                for (int i = p.rotary_dim + tid; i < D; i += WARPS * 32) put(p.k_write, k_tile, i, k[i]);
                for (int i = tid; i < D; i += WARPS * 32) put(p.v_write, v_tile, i, v[i]);
            }
            if (!direct) __threadfence();                                 // the row is read back below, past L1
        }
        __syncthreads();
        if (deferred >= 0) {
            load_tile(deferred, key_begin + deferred * TILE_KEYS, -1);
            for (int s = deferred; s < STAGES; ++s) cp_async_commit();
        }
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                const __nv_bfloat16* src = q_s + (h * 8 + r0) * D + kk * 16 + c;
                qb[kk][h][0] = *reinterpret_cast<const uint32_t*>(src);
                qb[kk][h][1] = *reinterpret_cast<const uint32_t*>(src + 8);
            }
    } else {
        pdl_wait();
        const int r0 = lane >> 2, c = (lane & 3) * 2;
        const __nv_bfloat16* base = p.q + ((size_t)t * p.nq + h0) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                const bool there = h * 8 + r0 < heads;
                const __nv_bfloat16* src = base + (size_t)(h * 8 + r0) * D + kk * 16 + c;
                qb[kk][h][0] = there ? *reinterpret_cast<const uint32_t*>(src) : 0u;
                qb[kk][h][1] = there ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
            }
    }

    // O^T: d = 16 mt + g (+ 8) down the rows, head 8 h + 2 t (+ 1) across; lane (g, t) holds [mt][h][0..3]
    float o[D / 16][NH][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt)
#pragma unroll
        for (int h = 0; h < NH; ++h) o[mt][h][0] = o[mt][h][1] = o[mt][h][2] = o[mt][h][3] = 0.f;
    // per head 8 h + 2 t + j: the running maximum (the same in the 8 lanes that share t) and THIS lane's part of the sum
    float head_max[NH][2], head_sum[NH][2];
#pragma unroll
    for (int h = 0; h < NH; ++h) { head_max[h][0] = head_max[h][1] = -INFINITY; head_sum[h][0] = head_sum[h][1] = 0.f; }
    // shared-memory offsets of this lane's ldmatrix rows inside a tile (the tile's base is added per stage):
    // keys as the first operand want the matrices in the order (keys 0-7, k low), (keys 8-15, k low), (.., k high)
    const int lm = lane >> 3;
    const int k_row = warp * 16 + (lm & 1) * 8 + (lane & 7), v_row = warp * 16 + (lm >> 1) * 8 + (lane & 7);

    for (int tile = 0; tile < n_tiles; ++tile) {
        // groups asked for so far: STAGES, and one per earlier iteration but the first; tile i is group i
        if (tile == 0) cp_async_wait<STAGES - 1>(); else cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (tile > 0) {   // refill the stage that was consumed in the previous iteration
            const int next = tile - 1 + STAGES;
            if (next < n_tiles) load_tile(next % STAGES, key_begin + next * TILE_KEYS, -1);
            cp_async_commit();
        }
        const int stage = tile % STAGES;
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES, vs = ks + T::BYTES;
        const int key0 = key_begin + tile * TILE_KEYS + warp * 16;       // this warp's 16 keys
        if (key0 < key_end) {
            // ---- S^T = K Q^T for 16 keys.  All fragments are asked for before the first product (one warp per
            //      scheduler: nothing else hides the shared-memory latency); the sums run in two chains per
            //      group of heads that meet at the end ----
            uint32_t kf[D / 16][4];
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ldmatrix_x4(ks + T::offset(k_row, kk * 2 + (lm >> 1)), kf[kk][0], kf[kk][1], kf[kk][2], kf[kk][3]);
            float st[NH][4], st_odd[NH][4];
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int i = 0; i < 4; ++i) st[h][i] = st_odd[h][i] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
                for (int h = 0; h < NH; ++h) mma_bf16(kk & 1 ? st_odd[h] : st[h], kf[kk], qb[kk][h][0], qb[kk][h][1]);
            // the values' fragments travel while the probabilities are made: V^T as the first operand
            uint32_t vf[D / 16][4];
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt)
                ldmatrix_x4_trans(vs + T::offset(v_row, mt * 2 + (lm & 1)), vf[mt][0], vf[mt][1], vf[mt][2], vf[mt][3]);
            // st[h][0], [1]: key g, heads 2t, 2t + 1; [2], [3]: key g + 8
            const bool low_hidden = key0 + (lane >> 2) >= key_end, high_hidden = key0 + (lane >> 2) + 8 >= key_end;
            uint32_t pb[NH][2];
#pragma unroll
            for (int h = 0; h < NH; ++h) {
#pragma unroll
                for (int i = 0; i < 4; ++i) st[h][i] += st_odd[h][i];
                if (low_hidden) st[h][0] = st[h][1] = -INFINITY;       // (only the range's last keys can be)
                if (high_hidden) st[h][2] = st[h][3] = -INFINITY;
                float correction[2], e[4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float top = fmaxf(st[h][j], st[h][j + 2]);
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 4));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 8));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 16));
                    // The reference point of the exponentials is a whole number (in base-2 logarithms), so the
                    // 16-bit probabilities have the same mantissas whatever tile, warp or range a key falls
                    // in, and rescaling by `correction` (a power of two) is exact.
                    const float new_max = fmaxf(head_max[h][j], ceilf(top * p.scale_log2));   // finite: key0 < key_end
                    correction[j] = exp2_whole(head_max[h][j] - new_max);
                    head_max[h][j] = new_max;
                    e[j] = ex2_approx(fmaf(st[h][j], p.scale_log2, -new_max));
                    e[j + 2] = ex2_approx(fmaf(st[h][j + 2], p.scale_log2, -new_max));
                    head_sum[h][j] = head_sum[h][j] * correction[j] + (e[j] + e[j + 2]);
                }
                // P^T as the second operand: what lane (g, t) holds of P (key g, heads 2t, 2t+1) it must hold of P^T
                pb[h][0] = transpose_8x8(pack_bf16(e[0], e[1]));
                pb[h][1] = transpose_8x8(pack_bf16(e[2], e[3]));
                // ---- O^T = O^T * correction + V^T P^T (the maximum is a whole number and seldom moves) ----
                if (__any_sync(0xffffffffu, correction[0] != 1.f || correction[1] != 1.f)) {
#pragma unroll
                    for (int mt = 0; mt < D / 16; ++mt) {
                        o[mt][h][0] *= correction[0]; o[mt][h][1] *= correction[1];
                        o[mt][h][2] *= correction[0]; o[mt][h][3] *= correction[1];
                    }
                }
            }
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt)
#pragma unroll
                for (int h = 0; h < NH; ++h) mma_bf16(o[mt][h], vf[mt], pb[h][0], pb[h][1]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a quarter of the keys) ----
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int j = 0; j < 2; ++j) {                                 // the eight lanes that share t hold parts of a head's sum
            head_sum[h][j] += __shfl_xor_sync(0xffffffffu, head_sum[h][j], 4);
            head_sum[h][j] += __shfl_xor_sync(0xffffffffu, head_sum[h][j], 8);
            head_sum[h][j] += __shfl_xor_sync(0xffffffffu, head_sum[h][j], 16);
        }
    constexpr int MERGE_STRIDE = D + 4;                               // heads 4 words apart: a warp's 32 stores meet 32 banks
    float* merge_o = reinterpret_cast<float*>(smem);                  // [WARPS][16][MERGE_STRIDE]
    float* merge_m = merge_o + WARPS * 16 * MERGE_STRIDE;             // [WARPS][16]
    float* merge_l = merge_m + WARPS * 16;
    float* merge_f = merge_l + WARPS * 16;                            // [WARPS][16] each warp's share of a row
    {
        const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt)
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                float* dst = merge_o + ((size_t)warp * 16 + h * 8 + t2) * MERGE_STRIDE + mt * 16 + g;
                dst[0] = o[mt][h][0];
                dst[MERGE_STRIDE] = o[mt][h][1];
                dst[8] = o[mt][h][2];
                dst[MERGE_STRIDE + 8] = o[mt][h][3];
            }
        if (g == 0) {
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    merge_m[warp * 16 + h * 8 + t2 + j] = head_max[h][j];
                    merge_l[warp * 16 + h * 8 + t2 + j] = head_sum[h][j];
                }
        }
    }
    __syncthreads();
    if (tid < heads) {                                                // one thread per row: the warps' shares
        const int r = tid;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) top = fmaxf(top, merge_m[w * 16 + r]);
        float f[WARPS], total = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            f[w] = exp2_whole(merge_m[w * 16 + r] - top);             // both are whole numbers (or -infinity)
            total += f[w] * merge_l[w * 16 + r];
        }
        const float inv = 1.0f / total;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) merge_f[w * 16 + r] = f[w] * inv;
        if (p.cluster) exchange_of<D>(smem)[16 * D + r] = top + log2f(total);
        else if (p.n_splits > 1)
            p.partial[(size_t)p.n_tokens * p.nq * p.n_splits * D + ((size_t)t * p.nq + h0 + r) * p.n_splits + blockIdx.z] =
                top + log2f(total);
    }
    __syncthreads();
    {
        constexpr int PER_THREAD = (16 * (D / 4) + WARPS * 32 - 1) / (WARPS * 32);
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int idx = tid + j * WARPS * 32;
            if (idx >= heads * (D / 4)) break;
            const int r = idx / (D / 4), c4 = idx % (D / 4);
            float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float share = merge_f[w * 16 + r];
                const float4 part = *reinterpret_cast<const float4*>(merge_o + ((size_t)w * 16 + r) * MERGE_STRIDE + c4 * 4);
                value.x += share * part.x; value.y += share * part.y; value.z += share * part.z; value.w += share * part.w;
            }
            const int h = h0 + r;
            if (p.cluster) {
                *reinterpret_cast<float4*>(exchange_of<D>(smem) + r * D + c4 * 4) = value;
            } else if (p.n_splits == 1) {
                uint2 packed;
                packed.x = pack_bf16(value.x, value.y);
                packed.y = pack_bf16(value.z, value.w);
                *reinterpret_cast<uint2*>(p.out + ((size_t)t * p.nq + h) * D + c4 * 4) = packed;
            } else {
                const size_t at = ((size_t)t * p.nq + h) * p.n_splits + blockIdx.z;
                *reinterpret_cast<float4*>(p.partial + at * D + c4 * 4) = value;
            }
        }
    }
    if (p.cluster) {
        cluster_merge<D>(p, smem, t, h0, heads);
        return;
    }
    if (p.n_splits == 1 || !p.counters) return;

    // ---- the CTA of this token and head group that finishes last combines the ranges, in ascending
    //      order, so the result does not depend on which CTA that is ----
    const int used = min(p.n_splits, (pos + 1 - first + split_len - 1) / split_len);
    int* counter = p.counters + blockIdx.x * gridDim.y + blockIdx.y;
    // The CTA's partial results are published by ONE release: the barrier orders every thread's stores before
    // thread 0's atomic, whose release carries them along (and its acquire, with the barrier after it, orders the
    // last CTA's loads behind the other CTAs' releases): one trip instead of a fence in each thread and an atomic.
    __syncthreads();
    if (tid == 0) {
        int seen;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counter) : "memory");
        last_flag = seen == used - 1;
        if (seen == used - 1) *counter = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    const float* lse = p.partial + (size_t)p.n_tokens * p.nq * p.n_splits * D;
    if (used <= 16) {
        // Few ranges: a thread owns eight elements of a head and has every load it needs (the ranges'
        // log-sum-exps and their eight elements) in flight at once, so the token's tail is one trip to L2.
        for (int idx = tid; idx < heads * (D / 8); idx += WARPS * 32) {
            const int r = idx / (D / 8), c8 = idx % (D / 8);
            const float* lrow = lse + ((size_t)t * p.nq + h0 + r) * p.n_splits;
            const float4* base = reinterpret_cast<const float4*>(p.partial + ((size_t)t * p.nq + h0 + r) * p.n_splits * D) + c8 * 2;
            float l[16];
            float4 v[16][2];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const bool there = j < used;
                l[j] = there ? __ldcg(lrow + j) : -INFINITY;
                v[j][0] = there ? __ldcg(base + (size_t)j * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[j][1] = there ? __ldcg(base + (size_t)j * (D / 4) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float top = l[0];
#pragma unroll
            for (int j = 1; j < 16; ++j) top = fmaxf(top, l[j]);
            float total = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 16; ++j) {                        // ascending ranges: the order depends on nothing else
                const float w = exp2f(l[j] - top);
                total += w;
                acc[0] += w * v[j][0].x; acc[1] += w * v[j][0].y; acc[2] += w * v[j][0].z; acc[3] += w * v[j][0].w;
                acc[4] += w * v[j][1].x; acc[5] += w * v[j][1].y; acc[6] += w * v[j][1].z; acc[7] += w * v[j][1].w;
            }
            const float inv = 1.0f / total;
            uint4 packed;
            packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
            packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
            packed.z = pack_bf16(acc[4] * inv, acc[5] * inv);
            packed.w = pack_bf16(acc[6] * inv, acc[7] * inv);
            *reinterpret_cast<uint4*>(p.out + ((size_t)t * p.nq + h0 + r) * D + c8 * 8) = packed;
        }
        return;
    }
    float* weight = reinterpret_cast<float*>(smem);                   // [16][used], then [16] totals
    float* totals = weight + 16 * used;
    for (int r = warp; r < heads; r += WARPS) {
        const float* base = lse + ((size_t)t * p.nq + h0 + r) * p.n_splits;
        float top = -INFINITY;
        for (int s = lane; s < used; s += 32) top = fmaxf(top, __ldcg(base + s));
        top = warp_max(top);
        float total = 0.f;
        for (int s = lane; s < used; s += 32) {
            const float f = exp2f(__ldcg(base + s) - top);
            weight[r * used + s] = f;
            total += f;
        }
        total = warp_sum(total);                  // the order of this sum depends on `used` alone
        if (lane == 0) totals[r] = total;
    }
    __syncthreads();
    // 16 bytes per load, eight ranges in flight per thread: the last CTA's reads are the tail of the step
    for (int idx = tid; idx < heads * (D / 4); idx += WARPS * 32) {
        const int r = idx / (D / 4), c4 = idx % (D / 4);
        const float4* base = reinterpret_cast<const float4*>(p.partial + ((size_t)t * p.nq + h0 + r) * p.n_splits * D) + c4;
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
        *reinterpret_cast<uint2*>(p.out + ((size_t)t * p.nq + h0 + r) * D + c4 * 4) = packed;
    }
}

// Combine the ranges of one (token, head): out = sum_s 2^(lse_s - L) o_s / sum_s 2^(lse_s - L).
template <int D>
__global__ void attention_merge_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = p.rows[blockIdx.x];
    if (t < 0) return;
    if (p.slots[t] < 0) return;
    const int h = blockIdx.y;
    const int pos = p.positions[t];
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int split_len = range_length(p, pos + 1 - first);
    const int used = min(p.n_splits, (pos + 1 - first + split_len - 1) / split_len);
    const size_t at = ((size_t)t * p.nq + h) * p.n_splits;
    const float* lse = p.partial + (size_t)p.n_tokens * p.nq * p.n_splits * D + at;
    float top = -INFINITY;
    for (int s = 0; s < used; ++s) top = fmaxf(top, lse[s]);
    for (int dcol = threadIdx.x; dcol < D; dcol += blockDim.x) {
        float total = 0.f, value = 0.f;
        for (int s = 0; s < used; ++s) {
            const float f = exp2f(lse[s] - top);
            total += f;
            value += f * p.partial[(at + s) * D + dcol];
        }
        p.out[((size_t)t * p.nq + h) * D + dcol] = __float2bfloat16_rn(value / total);
    }
}

template <int D>
size_t decode_smem_bytes() {
    const size_t ring = (size_t)STAGES * 2 * Tile<D>::BYTES + 16 * D * 2 + D * 4 + 18 * D * 4;   // the tiles, the rotated queries, the angles' cosines and sines, the step's 32-bit rows
    const size_t merge = (size_t)WARPS * 16 * (D + 4 + 3) * sizeof(float) + (size_t)(16 * D + 16) * sizeof(float);   // the warps' merge, then the cluster's exchange
    const size_t weights = (size_t)16 * (MAX_FUSED_SPLITS + 1) * sizeof(float);
    return ring > merge ? (ring > weights ? ring : weights) : (merge > weights ? merge : weights);
}

template <int D, int NH>
int configure_decode() {
    static int state = 0;                  // 1: done, -1: failed
    if (state == 0) {
        state = 1;
        if (cudaFuncSetAttribute(attention_decode_kernel<D, NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem_bytes<D>()) != cudaSuccess ||
            cudaFuncSetAttribute(attention_decode_kernel<D, NH>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
            cudaGetLastError();
            state = -1;
        }
    }
    return state == 1 ? LIA_OK : LIA_ERR_LAUNCH;
}

// Clusters of `size` CTAs of the kernel that the device holds at once (asked of the driver once per size; 0: none).
template <int D, int NH>
int max_active_clusters(int size) {
    static int cached[MAX_CLUSTER + 1] = {};
    if (size < 2 || size > MAX_CLUSTER) return 0;
    if (cached[size] == 0) {
        cached[size] = -1;
        if (configure_decode<D, NH>() == LIA_OK) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(1, 1, (unsigned)size);
            config.blockDim = dim3(WARPS * 32);
            config.dynamicSmemBytes = decode_smem_bytes<D>();
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeClusterDimension;
            attribute[0].val.clusterDim.x = 1;
            attribute[0].val.clusterDim.y = 1;
            attribute[0].val.clusterDim.z = (unsigned)size;
            config.attrs = attribute;
            config.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel<D, NH>, &config) == cudaSuccess && clusters > 0)
                cached[size] = clusters;
            else
                cudaGetLastError();
        }
    }
    return cached[size] > 0 ? cached[size] : 0;
}

template <int D, int NH>
int launch_decode(const Params& p, int n_rows, cudaStream_t stream) {
    int rc = configure_decode<D, NH>();
    if (rc != LIA_OK) return rc;
    const size_t smem = decode_smem_bytes<D>();
    const int group = p.nq / p.nkv;
    dim3 grid(n_rows, p.nkv * ((group + 15) / 16), p.n_splits);
    if (p.cluster) {
        cudaLaunchConfig_t config = {};
        config.gridDim = grid;
        config.blockDim = dim3(WARPS * 32);
        config.dynamicSmemBytes = smem;
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = 1;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = (unsigned)p.n_splits;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes;
        config.numAttrs = lia_pdl_enabled.load(std::memory_order_relaxed) ? 2 : 1;
        lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
        if (cudaLaunchKernelEx(&config, attention_decode_kernel<D, NH>, p) != cudaSuccess) {
            cudaGetLastError();
            return LIA_ERR_LAUNCH;
        }
        return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
    }
    rc = lia_launch(attention_decode_kernel<D, NH>, grid, dim3(WARPS * 32), smem, stream, p);
    if (rc != LIA_OK) return rc;
    if (p.n_splits > 1 && !p.counters)
        rc = lia_launch(attention_merge_kernel<D>, dim3(n_rows, p.nq), dim3(D < 128 ? D : 128), 0, stream, p);
    return rc;
}

// CTAs of the kernel that one SM holds at once (asked of the driver once; 0: unknown).
template <int D, int NH>
int ctas_per_sm() {
    static int cached = 0;
    if (cached == 0) {
        cached = -1;
        int blocks = 0;
        if (configure_decode<D, NH>() == LIA_OK &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_decode_kernel<D, NH>, WARPS * 32, decode_smem_bytes<D>()) == cudaSuccess &&
            blocks > 0)
            cached = blocks;
        else
            cudaGetLastError();
    }
    return cached > 0 ? cached : 0;
}

template <int D>
int cluster_splits_for(bool wide, int clusters, int wanted) {
    for (int size = MAX_CLUSTER; size >= 2; size /= 2) {
        if (size > wanted) continue;
        const int fit = wide ? max_active_clusters<D, 2>(size) : max_active_clusters<D, 1>(size);
        if (clusters <= fit) return size;
    }
    return 1;
}
}  // namespace

// Into how many ranges (2, 4, 8 or 16, at most `wanted`) the kernel can cut the keys of `clusters` (token, head group)
// pairs with the ranges of a pair as one thread-block cluster, all clusters on the device at once; 1: none, the
// ranges then meet through scratch memory (or there is one range).
LIA_EXPORT int lia_attention_decode_cluster_splits(int d, int heads_per_kv_head, int clusters, int wanted) {
    if (clusters <= 0 || wanted < 2) return 1;
    const bool wide = heads_per_kv_head > 8;
    if (d == 128) return cluster_splits_for<128>(wide, clusters, wanted);
    if (d == 64) return cluster_splits_for<64>(wide, clusters, wanted);
    if (d == 32) return cluster_splits_for<32>(wide, clusters, wanted);
    return 1;
}

// CTAs of the kernel that an SM holds at once for this head size (registers and shared memory decide: 2 at head
// size 128, more below); 0: the kernel does not take the head size, or the driver did not say.
LIA_EXPORT int lia_attention_decode_ctas_per_sm(int d, int heads_per_kv_head) {
    const bool wide = heads_per_kv_head > 8;
    if (d == 128) return wide ? ctas_per_sm<128, 2>() : ctas_per_sm<128, 1>();
    if (d == 64) return wide ? ctas_per_sm<64, 2>() : ctas_per_sm<64, 1>();
    if (d == 32) return wide ? ctas_per_sm<32, 2>() : ctas_per_sm<32, 1>();
    return 0;
}

// Floats of scratch that n_rows tokens with n_splits ranges need.
LIA_EXPORT long long lia_attention_decode_scratch_floats(int n_tokens, int nq, int d, int n_splits) {
    return n_splits > 1 ? (long long)n_tokens * nq * n_splits * (d + 1) : 0;
}

// `qkv` non-null: q is ignored; the kernel takes the queries from the 32-bit q|k|v rows, applies the rotary
// encoding (rotary_dim leading elements of each head; 0: none) and, when `write_kv`, the CTA of each token's last
// range rotates the token's key and appends key and value to the page of its position before reading them.
// Decode attention for the tokens listed in `rows` (indices into the step's batch), bfloat16 only,
// head_dim 32, 64 or 128 (other sizes: LIA_ERR_SIZE; the caller falls back to the generic kernel).
// `cluster` non-zero: `n_splits` is what lia_attention_decode_cluster_splits gave; `partial` and `counters` are not used.
// `all_new` non-zero: the rows may be tokens of prompt portions of this step, whose earlier keys the kernels ahead
// have written too; zero: only a row's own key is of this step (decoded tokens), and older tiles are fetched early.
// `n_splits` ranges of `split_len` keys each must cover the longest visible span among the rows;
// split_len 0 lets every row cut its own span into n_splits ranges (see range_length).
LIA_EXPORT int lia_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* rows,
                                    int n_rows, const int* positions, const int* slots, const int* block_table,
                                    int table_stride, void* out, float* partial, long long partial_floats,
                                    int* counters, int n_tokens, int nq, int nkv, int d, int page_size, int window, float scale,
                                    int split_len, int n_splits, const float* qkv, const float* inv_freq, int rotary_dim,
                                    int write_kv, int num_pages, int cluster, int all_new, int* error_flag, cudaStream_t stream) {
    if (n_rows <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || split_len < 0 || split_len % TILE_KEYS || n_splits <= 0 ||
        n_splits > 65535)
        return LIA_ERR_SIZE;
    if (cluster && (n_splits < 2 || n_splits > MAX_CLUSTER || (n_splits & (n_splits - 1)))) return LIA_ERR_SIZE;
    if (!cluster && n_splits > 1 && (!partial || partial_floats < lia_attention_decode_scratch_floats(n_tokens, nq, d, n_splits)))
        return LIA_ERR_SIZE;
    if (!cluster && n_splits > 1 && ((uintptr_t)partial & 15u)) return LIA_ERR_ALIGN;
    Params p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.rows = rows; p.positions = positions; p.slots = slots; p.block_table = block_table;
    p.out = (__nv_bfloat16*)out; p.partial = partial;
    p.counters = n_splits <= MAX_FUSED_SPLITS ? counters : nullptr;
    if (qkv && (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim > 0 && !inv_freq) || nq / nkv > 16))
        return LIA_ERR_SIZE;             // with more than 16 heads per kv head two CTAs would share the appended key
    p.qkv = qkv; p.inv_freq = inv_freq; p.rotary_dim = rotary_dim; p.write_kv = write_kv; p.num_pages = num_pages;
    p.k_write = (__nv_bfloat16*)const_cast<void*>(k_pages); p.v_write = (__nv_bfloat16*)const_cast<void*>(v_pages);
    p.error_flag = error_flag;
    p.cluster = cluster ? 1 : 0;
    p.all_new = all_new ? 1 : 0;
    p.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if (page_size == (1 << b)) p.page_shift = b;
    p.n_tokens = n_tokens; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window;
    p.split_len = split_len; p.n_splits = n_splits; p.scale_log2 = scale * LOG2E;
    const bool wide = nq / nkv > 8;             // more than 8 query heads per kv head: two groups of 8 per CTA
    if (d == 128) return wide ? launch_decode<128, 2>(p, n_rows, stream) : launch_decode<128, 1>(p, n_rows, stream);
    if (d == 64) return wide ? launch_decode<64, 2>(p, n_rows, stream) : launch_decode<64, 1>(p, n_rows, stream);
    if (d == 32) return wide ? launch_decode<32, 2>(p, n_rows, stream) : launch_decode<32, 1>(p, n_rows, stream);
    return LIA_ERR_SIZE;
}
