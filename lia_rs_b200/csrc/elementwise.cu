// Embedding gather, RMSNorm, and the rotary encoding fused with the key/value append.
// Every kernel takes all sizes as arguments; the residual stream is always 32-bit.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// Embedding: h[t, :] = table[token_t, :] * scale, written in 32-bit.
// A token id outside [0, vocab) writes zeros and raises the error flag (no read out of range).
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                 float* __restrict__ out, int n_tokens, int hidden, int vocab,
                                 float scale, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int token = tokens[t];
    const bool ok = token >= 0 && token < vocab;
    if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    const TW* row = table + (size_t)(ok ? token : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = ok ? to_float(row[i]) * scale : 0.f;
}

LIA_EXPORT int lia_embedding(const int* tokens, const void* table, int table_dtype, float* out,
                             int n_tokens, int hidden, int vocab, float scale, int* error_flag,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (hidden <= 0 || vocab <= 0) return LIA_ERR_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LIA_BF16)
        return lia_launch(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                          (const __nv_bfloat16*)table, out, n_tokens, hidden, vocab, scale, error_flag);
    if (table_dtype == LIA_F32)
        return lia_launch(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table,
                          out, n_tokens, hidden, vocab, scale, error_flag);
    return LIA_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// RMSNorm of 32-bit rows: y = x * rsqrt(mean(x^2) + eps) * w * out_scale.
// Sum of squares, mean, eps and the reciprocal root are 32-bit; the order of the additions
// depends on `hidden` alone, not on the number of rows.  `rows_index` (optional) gathers:
// output row r is computed from input row rows_index[r] (negative index -> zeros).
//
// One warp owns one row and keeps it in registers between the sum and the scaling (rows of up to
// 4096 elements whose width is a multiple of 4): 16-byte loads, all in flight at once, no block
// barrier.  Other widths take the block-per-row kernel below.
template <typename TO> __device__ __forceinline__ void store4(TO* dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}
template <typename TW> __device__ __forceinline__ float4 load4(const TW* src);
template <> __device__ __forceinline__ float4 load4<float>(const float* src) { return *reinterpret_cast<const float4*>(src); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* src) {
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

template <typename TW, typename TO, int VPL>      // VPL: float4 per lane; the row has at most 128 * VPL elements
__global__ void rmsnorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ rows_index,
                                    const TW* __restrict__ weight, TO* __restrict__ out, int rows,
                                    int hidden, float eps, float out_scale) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int quads = hidden >> 2;
    float4 w[VPL];                                   // the weights wait for no one
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = lane + i * 32;
        w[i] = q < quads ? load4<TW>(weight + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const int src = rows_index ? rows_index[r] : r;
    TO* dst = out + (size_t)r * hidden;
    if (src < 0) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int q = lane + i * 32;
            if (q < quads) store4<TO>(dst + 4 * q, 0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    const float* row = x + (size_t)src * hidden;
    float4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = lane + i * 32;
        v[i] = q < quads ? *reinterpret_cast<const float4*>(row + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        sum = fmaf(v[i].x, v[i].x, sum);
        sum = fmaf(v[i].y, v[i].y, sum);
        sum = fmaf(v[i].z, v[i].z, sum);
        sum = fmaf(v[i].w, v[i].w, sum);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int q = lane + i * 32;
        if (q < quads)
            store4<TO>(dst + 4 * q, v[i].x * inv * w[i].x * out_scale, v[i].y * inv * w[i].y * out_scale,
                       v[i].z * inv * w[i].z * out_scale, v[i].w * inv * w[i].w * out_scale);
    }
}

template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows_index,
                               const TW* __restrict__ weight, TO* __restrict__ out, int rows,
                               int hidden, float eps, float out_scale) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int src = rows_index ? rows_index[r] : r;
    TO* dst = out + (size_t)r * hidden;
    if (src < 0) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<TO>(0.f);
        return;
    }
    const float* row = x + (size_t)src * hidden;
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = row[i];
        sum = fmaf(v, v, sum);
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = from_float<TO>(row[i] * inv * to_float(weight[i]) * out_scale);
}

template <typename TW, typename TO>
int launch_rmsnorm(const float* x, const int* rows_index, const void* weight, void* out, int rows, int hidden,
                   float eps, float out_scale, cudaStream_t stream) {
    const bool vector = hidden % 4 == 0 && hidden <= 4096 && ((uintptr_t)x & 15u) == 0 && ((uintptr_t)weight & 15u) == 0 &&
                        ((uintptr_t)out & 15u) == 0;
    if (!vector)
        return lia_launch(rmsnorm_kernel<TW, TO>, dim3(rows), dim3(hidden >= 1024 ? 256 : 128), 0, stream, x, rows_index,
                          (const TW*)weight, (TO*)out, rows, hidden, eps, out_scale);
    const int warps = rows >= 256 ? 4 : 1;             // few rows: one warp per CTA, spread over the SMs
    const dim3 grid((rows + warps - 1) / warps), block(warps * 32);
#define LIA_NORM_WARP(VPL)                                                                                          \
    return lia_launch(rmsnorm_warp_kernel<TW, TO, VPL>, grid, block, 0, stream, x, rows_index, (const TW*)weight, \
                      (TO*)out, rows, hidden, eps, out_scale)
    if (hidden <= 512) LIA_NORM_WARP(4);
    if (hidden <= 1024) LIA_NORM_WARP(8);
    if (hidden <= 2048) LIA_NORM_WARP(16);
    LIA_NORM_WARP(32);
#undef LIA_NORM_WARP
}

LIA_EXPORT int lia_rmsnorm(const float* x, const int* rows_index, const void* weight, int weight_dtype,
                           void* out, int out_dtype, int rows, int hidden, float eps, float out_scale,
                           cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (hidden <= 0) return LIA_ERR_SIZE;
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_BF16)
        return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, rows_index, weight, out, rows, hidden, eps, out_scale, stream);
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_F32)
        return launch_rmsnorm<__nv_bfloat16, float>(x, rows_index, weight, out, rows, hidden, eps, out_scale, stream);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_BF16)
        return launch_rmsnorm<float, __nv_bfloat16>(x, rows_index, weight, out, rows, hidden, eps, out_scale, stream);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_F32)
        return launch_rmsnorm<float, float>(x, rows_index, weight, out, rows, hidden, eps, out_scale, stream);
    return LIA_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// Rotary encoding (rotate-half over the first `rotary_dim` elements of each head; 0 = none)
// of q and k, fused with the append of k and v to the paged cache.
//   qkv      [n_tokens, (nq + 2 nkv) d] 32-bit: q heads, then k heads, then v heads
//   q_out    [n_tokens, nq d]
//   k_pages, v_pages [num_pages, page_size, nkv, d]
//   block_table [slots, table_stride]: page of (slot, position / page_size)
//   inv_freq [rotary_dim / 2] 32-bit: theta^(-2i/rotary_dim), rounded once from 64-bit on the host
// The angle pos * inv_freq[i] and its sine and cosine are 32-bit (the reference likewise casts
// the position to f32 and multiplies: src/gpu/kernels/llama_position.rs:35-46).
// A token whose slot is negative is padding and is skipped.  `write_kv` = 0 leaves the cache
// alone (a layer that reads another layer's cache).
template <typename TQ, typename TC>
__global__ void rope_kv_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                               const int* __restrict__ slots, const int* __restrict__ block_table,
                               int table_stride, TQ* __restrict__ q_out, TC* __restrict__ k_pages,
                               TC* __restrict__ v_pages, int n_tokens, int nq, int nkv, int d,
                               int rotary_dim, const float* __restrict__ inv_freq, int page_size,
                               int num_pages, int write_kv, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int width = (nq + 2 * nkv) * d;
    const float* row = qkv + (size_t)t * width;
    const int half = rotary_dim / 2;
    size_t cache_row = 0;
    bool cache_ok = false;
    if (write_kv) {
        const int page = block_table[(size_t)slot * table_stride + pos / page_size];
        cache_ok = page >= 0 && page < num_pages;
        if (!cache_ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
        cache_row = ((size_t)(cache_ok ? page : 0) * page_size + pos % page_size) * nkv * d;
    }
    const int rot_heads = nq + nkv;
    // sine and cosine of the token's angles, once for all heads
    extern __shared__ float rotation[];                  // [half] cosines, then [half] sines
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &rotation[half + i], &rotation[i]);
    __syncthreads();
    if (rotary_dim == d && d % 8 == 0) {
        // The usual case, four elements at a time: 16-byte loads of the 32-bit row, 8-byte (or 16-byte) stores.
        // (Rows of qkv, q_out and the pages are multiples of 4 elements long from 16-byte-aligned bases.)
        const int quads = half / 4;
        for (int w = threadIdx.x; w < rot_heads * quads; w += blockDim.x) {
            const int head = w / quads, i = (w % quads) * 4;
            const float4 a = *reinterpret_cast<const float4*>(row + head * d + i);
            const float4 b = *reinterpret_cast<const float4*>(row + head * d + i + half);
            const float4 c = *reinterpret_cast<const float4*>(rotation + i), sn = *reinterpret_cast<const float4*>(rotation + half + i);
            const float lo[4] = {a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w};
            const float hi[4] = {b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y, b.z * c.z + a.z * sn.z, b.w * c.w + a.w * sn.w};
            if (head < nq) {
                TQ* dst = q_out + (size_t)t * nq * d + head * d + i;
                store4<TQ>(dst, lo[0], lo[1], lo[2], lo[3]);
                store4<TQ>(dst + half, hi[0], hi[1], hi[2], hi[3]);
            } else if (cache_ok) {
                TC* dst = k_pages + cache_row + (head - nq) * d + i;
                store4<TC>(dst, lo[0], lo[1], lo[2], lo[3]);
                store4<TC>(dst + half, hi[0], hi[1], hi[2], hi[3]);
            }
        }
        if (cache_ok) {
            const float* v = row + (nq + nkv) * d;
            for (int w = threadIdx.x * 4; w < nkv * d; w += blockDim.x * 4) {
                const float4 x = *reinterpret_cast<const float4*>(v + w);
                store4<TC>(v_pages + cache_row + w, x.x, x.y, x.z, x.w);
            }
        }
        return;
    }
    // rotated part: one work item per (head, i < half)
    for (int w = threadIdx.x; w < rot_heads * half; w += blockDim.x) {
        const int head = w / half, i = w % half;
        const float c = rotation[i], s = rotation[half + i];
        const float a = row[head * d + i], b = row[head * d + i + half];
        const float ra = a * c - b * s, rb = b * c + a * s;
        if (head < nq) {
            TQ* dst = q_out + (size_t)t * nq * d + head * d;
            dst[i] = from_float<TQ>(ra);
            dst[i + half] = from_float<TQ>(rb);
        } else if (cache_ok) {
            TC* dst = k_pages + cache_row + (head - nq) * d;
            dst[i] = from_float<TC>(ra);
            dst[i + half] = from_float<TC>(rb);
        }
    }
    // pass-through part of q and k (elements beyond rotary_dim)
    const int rest = d - rotary_dim;
    if (rest > 0) {
        for (int w = threadIdx.x; w < rot_heads * rest; w += blockDim.x) {
            const int head = w / rest, i = rotary_dim + w % rest;
            const float a = row[head * d + i];
            if (head < nq) q_out[(size_t)t * nq * d + head * d + i] = from_float<TQ>(a);
            else if (cache_ok) k_pages[cache_row + (head - nq) * d + i] = from_float<TC>(a);
        }
    }
    if (cache_ok) {
        const float* v = row + (nq + nkv) * d;
        for (int w = threadIdx.x; w < nkv * d; w += blockDim.x)
            v_pages[cache_row + w] = from_float<TC>(v[w]);
    }
}

LIA_EXPORT int lia_rope_kv_write(const float* qkv, const int* positions, const int* slots,
                                 const int* block_table, int table_stride, void* q_out, void* k_pages,
                                 void* v_pages, int dtype, int n_tokens, int nq, int nkv, int d,
                                 int rotary_dim, const float* inv_freq, int page_size, int num_pages,
                                 int write_kv, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || rotary_dim < 0 || rotary_dim > d ||
        (rotary_dim & 1) || (rotary_dim > 0 && !inv_freq))
        return LIA_ERR_SIZE;
    const int threads = 256;
#define LIA_ROPE(T)                                                                                          \
    return lia_launch(rope_kv_kernel<T, T>, dim3(n_tokens), dim3(threads), (size_t)rotary_dim * sizeof(float), stream, qkv, positions, slots, \
                      block_table, table_stride, (T*)q_out, (T*)k_pages, (T*)v_pages, n_tokens, nq, nkv, d,  \
                      rotary_dim, inv_freq, page_size, num_pages, write_kv, error_flag)
    if (dtype == LIA_BF16) LIA_ROPE(__nv_bfloat16);
    if (dtype == LIA_F32) LIA_ROPE(float);
#undef LIA_ROPE
    return LIA_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// Gather of rows: dst[r, :] = src[index[r], :], rows of `row_bytes` bytes copied as they are (any element
// type); a negative index gives a row of zeros.  The reference gathers the rows whose logits are wanted
// before the last layer's feed-forward (src/gpu/kernels/llama.rs:185-198).
template <typename V>
__global__ void gather_rows_kernel(const V* __restrict__ src, const int* __restrict__ index, V* __restrict__ dst,
                                   int rows, int src_rows, long long src_stride, long long dst_stride, int words) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int from = index[r];
    V* out = dst + (size_t)r * dst_stride;
    if (from < 0 || from >= src_rows) {
        V zero;
        memset(&zero, 0, sizeof(V));
        for (int i = threadIdx.x; i < words; i += blockDim.x) out[i] = zero;
        return;
    }
    const V* in = src + (size_t)from * src_stride;
    for (int i = threadIdx.x; i < words; i += blockDim.x) out[i] = in[i];
}

// src [src_rows, src_stride_bytes a row], dst [rows, dst_stride_bytes a row], row_bytes copied per row.
LIA_EXPORT int lia_gather_rows(const void* src, const int* index, void* dst, int rows, int src_rows,
                               long long src_stride_bytes, long long dst_stride_bytes, long long row_bytes,
                               cudaStream_t stream) {
    if (rows <= 0 || row_bytes <= 0) return LIA_OK;
    if (src_rows <= 0 || src_stride_bytes < row_bytes || dst_stride_bytes < row_bytes || row_bytes > (1LL << 30))
        return LIA_ERR_SIZE;
    const uintptr_t together = (uintptr_t)src | (uintptr_t)dst | (uintptr_t)src_stride_bytes |
                               (uintptr_t)dst_stride_bytes | (uintptr_t)row_bytes;
    const int threads = row_bytes >= 4096 ? 256 : 128;
    if ((together & 15u) == 0)
        return lia_launch(gather_rows_kernel<uint4>, dim3(rows), dim3(threads), 0, stream, (const uint4*)src, index,
                          (uint4*)dst, rows, src_rows, src_stride_bytes / 16, dst_stride_bytes / 16, (int)(row_bytes / 16));
    if ((together & 3u) == 0)
        return lia_launch(gather_rows_kernel<uint32_t>, dim3(rows), dim3(threads), 0, stream, (const uint32_t*)src, index,
                          (uint32_t*)dst, rows, src_rows, src_stride_bytes / 4, dst_stride_bytes / 4, (int)(row_bytes / 4));
    if ((together & 1u) == 0)
        return lia_launch(gather_rows_kernel<uint16_t>, dim3(rows), dim3(threads), 0, stream, (const uint16_t*)src, index,
                          (uint16_t*)dst, rows, src_rows, src_stride_bytes / 2, dst_stride_bytes / 2, (int)(row_bytes / 2));
    return LIA_ERR_ALIGN;
}
