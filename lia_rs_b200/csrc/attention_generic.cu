// Causal grouped-query attention over the paged cache, for every head size that is a multiple of
// 16 (up to 256), any number of heads and groups, any page size, prompt portions and single decoded
// tokens alike.  One warp owns one (token, query head): it walks the visible keys 32 at a time,
// each lane scoring one key, keeps the running maximum and sum of the softmax in 32-bit, and
// accumulates the output with each lane owning head elements lane, lane+32, ...
//
// A token at position p of request slot s sees keys j with max(0, p - window + 1) <= j <= p
// (window <= 0: all keys), read from that slot's pages.  The order of the work depends on p and the
// window alone, so a token's result does not depend on the batch it is in.
// This is the attention of the true 32-bit path and the fallback of the bfloat16 path.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ positions,
                         const int* __restrict__ slots, const int* __restrict__ block_table,
                         int table_stride, const int* __restrict__ rows, T* __restrict__ out, int n_tokens,
                         int nq, int nkv, int d,
                         int page_size, int window, float scale, int num_pages, int* __restrict__ error_flag) {
    __shared__ float q_shared[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * nq) return;
    const int t = rows ? rows[item / nq] : (int)(item / nq);
    const int h = (int)(item % nq);
    if (t < 0) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int kvh = h / (nq / nkv);
    const T* qrow = q + ((size_t)t * nq + h) * d;
    for (int i = lane; i < d; i += 32) q_shared[warp][i] = to_float(qrow[i]);
    __syncwarp();
    const int* table = block_table + (size_t)slot * table_stride;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int chunks = (d + 31) / 32;
    float acc[MAX_D / 32];
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] = 0.f;
    float running_max = -INFINITY, running_sum = 0.f;

    for (int base = first; base <= pos; base += 32) {
        const int j = base + lane;
        bool valid = j <= pos;
        int row = 0;
        float score = -INFINITY;
        if (valid) {
            row = cache_row_of(table, j, page_size, -1, num_pages, error_flag);
            valid = row >= 0;                       // a key without a page counts for nothing (and the flag is up)
            row = valid ? row : 0;
        }
        if (valid) {
            const T* krow = k_pages + ((size_t)row * nkv + kvh) * d;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot = fmaf(q_shared[warp][i], to_float(krow[i]), dot);
            score = dot * scale;
        }
        const float chunk_max = warp_max(score);
        const float new_max = fmaxf(running_max, chunk_max);
        const float correction = expf(running_max - new_max);   // exp(-inf) = 0 on the first chunk
        const float p = valid ? expf(score - new_max) : 0.f;
        running_sum = running_sum * correction + warp_sum(p);
        running_max = new_max;
#pragma unroll
        for (int c = 0; c < MAX_D / 32; ++c) acc[c] *= correction;
        const int count = min(32, pos - base + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vrow = v_pages + ((size_t)rj * nkv + kvh) * d;
#pragma unroll
            for (int c = 0; c < MAX_D / 32; ++c) {
                const int i = c * 32 + lane;
                if (c < chunks && i < d) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
            }
        }
    }
    T* orow = out + ((size_t)t * nq + h) * d;
    const float inv = 1.0f / running_sum;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = c * 32 + lane;
        if (c < chunks && i < d) orow[i] = from_float<T>(acc[c] * inv);
    }
}
}  // namespace

// q, out [tokens, nq, d]; k_pages, v_pages [num_pages, page_size, nkv, d]; all of `dtype`.
// `rows` (optional) lists the n_tokens batch indices to compute; without it tokens 0..n_tokens-1.
LIA_EXPORT int lia_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                     const int* positions, const int* slots, const int* block_table,
                                     int table_stride, const int* rows, void* out, int n_tokens, int nq,
                                     int nkv, int d,
                                     int page_size, int window, float scale, int num_pages, int* error_flag,
                                     cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || d <= 0 || d > MAX_D || d % 16 || page_size <= 0)
        return LIA_ERR_SIZE;
    const long long items = (long long)n_tokens * nq;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return LIA_ERR_SIZE;
    if (dtype == LIA_F32)
        attention_generic_kernel<float><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const float*)q, (const float*)k_pages, (const float*)v_pages, positions, slots, block_table,
            table_stride, rows, (float*)out, n_tokens, nq, nkv, d, page_size, window, scale, num_pages, error_flag);
    else if (dtype == LIA_BF16)
        attention_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, positions,
            slots, block_table, table_stride, rows, (__nv_bfloat16*)out, n_tokens, nq, nkv, d, page_size, window,
            scale, num_pages, error_flag);
    else
        return LIA_ERR_DTYPE;
    return lia_check_launch();
}
