// Decode attention over the paged bfloat16 cache, split over the keys.
//
// One CTA serves one decoded token's query heads of ONE kv head (up to 16 of them: they are the 16
// rows of the MMA's M, so the keys of a group are read once for all its query heads) over ONE range of
// keys.  Its four warps take 16 keys each of every 64-key tile: S = Q K^T by mma.sync (bf16 in, 32-bit
// out), running maximum and sum per row in 32-bit (base-2 exponentials with the scale folded in),
// P in bf16 back into the tensor cores against V.  Keys and values come from their pages through a
// three-stage cp.async ring in shared memory; ldmatrix (transposed for V) builds the fragments.  The
// four warps' partial results are merged in shared memory; the CTA then writes either the final
// output (one range) or a normalised partial output with its log-sum-exp to scratch, which
// `attention_merge_kernel` combines.  Ranges are `split_len` keys long, counted from the first visible
// key, so how a token's keys are cut depends on its own position, the window and split_len only.
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
    float* partial;                  // [tokens, nq, n_splits, D + 1]: normalised output, then log2-sum-exp
    int table_stride, nq, nkv, page_size, window, split_len, n_splits;
    float scale_log2;                // softmax scale * log2(e)
};

// Keys per range for a token that sees `span` keys: the given length, or (split_len 0) the span cut into
// n_splits ranges of a multiple of 64 keys.  The second rule depends on the token's own span and on
// n_splits alone, so a launch captured in a CUDA graph serves every context length.
__device__ __forceinline__ int range_length(const Params& p, int span) {
    if (p.split_len > 0) return p.split_len;
    const int per = (span + p.n_splits - 1) / p.n_splits;
    return (per + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS;
}

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(Params p) {
    using T = Tile<D>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
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
    if (key_begin >= key_end) return;
    const int* table = p.block_table + (size_t)slot * p.table_stride;

    // ---- Q fragments: rows = heads (row r -> head h0 + r), zero beyond `heads` ----
    uint32_t qf[D / 16][4];
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
        const __nv_bfloat16* base = p.q + ((size_t)t * p.nq + h0) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int col = kk * 16 + c;
            qf[kk][0] = r0 < heads ? *reinterpret_cast<const uint32_t*>(base + (size_t)r0 * D + col) : 0u;
            qf[kk][1] = r0 + 8 < heads ? *reinterpret_cast<const uint32_t*>(base + (size_t)(r0 + 8) * D + col) : 0u;
            qf[kk][2] = r0 < heads ? *reinterpret_cast<const uint32_t*>(base + (size_t)r0 * D + col + 8) : 0u;
            qf[kk][3] = r0 + 8 < heads ? *reinterpret_cast<const uint32_t*>(base + (size_t)(r0 + 8) * D + col + 8) : 0u;
        }
    }

    const uint32_t smem_base = smem_u32(smem);
    auto load_tile = [&](int stage, int key0) {
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES, vs = ks + T::BYTES;
        for (int id = tid; id < TILE_KEYS * T::CHUNKS; id += WARPS * 32) {
            const int r = id / T::CHUNKS, c = id % T::CHUNKS;
            const int key = key0 + r;
            const bool valid = key < key_end;
            size_t row = 0;
            if (valid) row = (size_t)table[key / p.page_size] * p.page_size + key % p.page_size;
            const size_t src = (row * p.nkv + kvh) * D + c * 8;
            cp_async_16(ks + T::offset(r, c), p.k_pages + src, valid);
            cp_async_16(vs + T::offset(r, c), p.v_pages + src, valid);
        }
    };

    const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_tiles) load_tile(s, key_begin + s * TILE_KEYS);
        cp_async_commit();
    }

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};

    for (int tile = 0; tile < n_tiles; ++tile) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {   // refill the stage that was consumed in the previous iteration
            const int next = tile + STAGES - 1;
            if (next < n_tiles) load_tile(next % STAGES, key_begin + next * TILE_KEYS);
            cp_async_commit();
        }
        const int stage = tile % STAGES;
        const uint32_t ks = smem_base + (uint32_t)stage * 2 * T::BYTES, vs = ks + T::BYTES;
        const int key0 = key_begin + tile * TILE_KEYS + warp * 16;       // this warp's 16 keys
        if (key0 < key_end) {
            // ---- S = Q K^T for 16 keys: two n-tiles of 8 ----
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int m = lane >> 3;
                const int row = warp * 16 + (m >> 1) * 8 + (lane & 7);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(ks + T::offset(row, kk * 2 + (m & 1)), b0, b1, b2, b3);
                mma_bf16(s[0], qf[kk], b0, b1);
                mma_bf16(s[1], qf[kk], b2, b3);
            }
            // ---- scale, mask, running maximum and sum ----
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + nt * 8 + (lane & 3) * 2 + (i & 1);
                    const float v = key < key_end ? s[nt][i] * p.scale_log2 : -INFINITY;
                    s[nt][i] = v;
                    tile_max[i >> 1] = fmaxf(tile_max[i >> 1], v);
                }
            float correction[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
                // The reference point of the exponentials is a whole number (in base-2 logarithms), so the
                // 16-bit probabilities have the same mantissas whatever tile, warp or range a key falls
                // in, and rescaling by `correction` is exact.
                const float new_max = fmaxf(row_max[r], ceilf(tile_max[r]));     // finite: key0 < key_end
                correction[r] = exp2f(row_max[r] - new_max);
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
                        e[nt][i] = exp2f(s[nt][i] - row_max[i >> 1]);
                        row_sum[i >> 1] += e[nt][i];
                    }
                pf[0] = pack_bf16(e[0][0], e[0][1]);
                pf[1] = pack_bf16(e[0][2], e[0][3]);
                pf[2] = pack_bf16(e[1][0], e[1][1]);
                pf[3] = pack_bf16(e[1][2], e[1][3]);
            }
            // ---- O = O * correction + P V ----
#pragma unroll
            for (int j = 0; j < D / 8; j += 2) {
                o[j][0] *= correction[0]; o[j][1] *= correction[0]; o[j][2] *= correction[1]; o[j][3] *= correction[1];
                o[j + 1][0] *= correction[0]; o[j + 1][1] *= correction[0]; o[j + 1][2] *= correction[1]; o[j + 1][3] *= correction[1];
                const int m = lane >> 3;
                const int row = warp * 16 + (m & 1) * 8 + (lane & 7);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vs + T::offset(row, j + (m >> 1)), b0, b1, b2, b3);
                mma_bf16(o[j], pf, b0, b1);
                mma_bf16(o[j + 1], pf, b2, b3);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a quarter of the keys) ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    float* merge_o = reinterpret_cast<float*>(smem);                  // [WARPS][16][D]
    float* merge_m = merge_o + WARPS * 16 * D;                        // [WARPS][16]
    float* merge_l = merge_m + WARPS * 16;
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
    __syncthreads();
    for (int idx = tid; idx < heads * D; idx += WARPS * 32) {
        const int r = idx / D, dcol = idx % D;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) top = fmaxf(top, merge_m[w * 16 + r]);
        float total = 0.f, value = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = merge_m[w * 16 + r];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - top);
            total += f * merge_l[w * 16 + r];
            value += f * merge_o[((size_t)w * 16 + r) * D + dcol];
        }
        const float result = value / total;
        const int h = h0 + r;
        if (p.n_splits == 1) {
            p.out[((size_t)t * p.nq + h) * D + dcol] = __float2bfloat16_rn(result);
        } else {
            float* dst = p.partial + (((size_t)t * p.nq + h) * p.n_splits + blockIdx.z) * (D + 1);
            dst[dcol] = result;
            if (dcol == 0) dst[D] = top + log2f(total);
        }
    }
}

// Combine the ranges of one (token, head): out = sum_s 2^(lse_s - L) o_s / sum_s 2^(lse_s - L).
template <int D>
__global__ void attention_merge_kernel(Params p) {
    const int t = p.rows[blockIdx.x];
    if (t < 0) return;
    if (p.slots[t] < 0) return;
    const int h = blockIdx.y;
    const int pos = p.positions[t];
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int split_len = range_length(p, pos + 1 - first);
    const int used = min(p.n_splits, (pos + 1 - first + split_len - 1) / split_len);
    const float* base = p.partial + ((size_t)t * p.nq + h) * p.n_splits * (D + 1);
    float top = -INFINITY;
    for (int s = 0; s < used; ++s) top = fmaxf(top, base[(size_t)s * (D + 1) + D]);
    for (int dcol = threadIdx.x; dcol < D; dcol += blockDim.x) {
        float total = 0.f, value = 0.f;
        for (int s = 0; s < used; ++s) {
            const float f = exp2f(base[(size_t)s * (D + 1) + D] - top);
            total += f;
            value += f * base[(size_t)s * (D + 1) + dcol];
        }
        p.out[((size_t)t * p.nq + h) * D + dcol] = __float2bfloat16_rn(value / total);
    }
}

template <int D>
int launch_decode(const Params& p, int n_rows, cudaStream_t stream) {
    const size_t ring = (size_t)STAGES * 2 * Tile<D>::BYTES;
    const size_t merge = (size_t)WARPS * 16 * (D + 2) * sizeof(float);
    const size_t smem = ring > merge ? ring : merge;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    const int group = p.nq / p.nkv;
    dim3 grid(n_rows, p.nkv * ((group + 15) / 16), p.n_splits);
    attention_decode_kernel<D><<<grid, WARPS * 32, smem, stream>>>(p);
    if (lia_check_launch() != LIA_OK) return LIA_ERR_LAUNCH;
    if (p.n_splits > 1) {
        attention_merge_kernel<D><<<dim3(n_rows, p.nq), D < 128 ? D : 128, 0, stream>>>(p);
        if (lia_check_launch() != LIA_OK) return LIA_ERR_LAUNCH;
    }
    return LIA_OK;
}
}  // namespace

// Floats of scratch that n_rows tokens with n_splits ranges need.
LIA_EXPORT long long lia_attention_decode_scratch_floats(int n_tokens, int nq, int d, int n_splits) {
    return n_splits > 1 ? (long long)n_tokens * nq * n_splits * (d + 1) : 0;
}

// Decode attention for the tokens listed in `rows` (indices into the step's batch), bfloat16 only,
// head_dim 32, 64 or 128 (other sizes: LIA_ERR_SIZE; the caller falls back to the generic kernel).
// `n_splits` ranges of `split_len` keys each must cover the longest visible span among the rows;
// split_len 0 lets every row cut its own span into n_splits ranges (see range_length).
LIA_EXPORT int lia_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* rows,
                                    int n_rows, const int* positions, const int* slots, const int* block_table,
                                    int table_stride, void* out, float* partial, long long partial_floats,
                                    int n_tokens, int nq, int nkv, int d, int page_size, int window, float scale,
                                    int split_len, int n_splits, cudaStream_t stream) {
    if (n_rows <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || split_len < 0 || split_len % TILE_KEYS || n_splits <= 0 ||
        n_splits > 65535)
        return LIA_ERR_SIZE;
    if (n_splits > 1 && (!partial || partial_floats < lia_attention_decode_scratch_floats(n_tokens, nq, d, n_splits)))
        return LIA_ERR_SIZE;
    Params p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.rows = rows; p.positions = positions; p.slots = slots; p.block_table = block_table;
    p.out = (__nv_bfloat16*)out; p.partial = partial;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window;
    p.split_len = split_len; p.n_splits = n_splits; p.scale_log2 = scale * LOG2E;
    if (d == 128) return launch_decode<128>(p, n_rows, stream);
    if (d == 64) return launch_decode<64>(p, n_rows, stream);
    if (d == 32) return launch_decode<32>(p, n_rows, stream);
    return LIA_ERR_SIZE;
}
