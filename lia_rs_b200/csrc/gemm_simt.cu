// Matrix product on the 32-bit pipes, for every size and element type:
//     acc[m, n] = sum_k A[m, k] * W[n, k]        (W is [out, in] row-major, as in the checkpoint)
// It is the product of the true 32-bit path (plain FMA, no tensor-core mode that would round the
// operands) and the fallback of the bfloat16 path for shapes the tcgen05 kernel refuses.
// The sum over k runs in ascending order for each output element, whatever M and N are, so a
// row's result does not depend on which other rows are in the batch.
//
// Epilogues:
//   STORE   out[m, n]  = alpha * acc
//   ACCUM   out[m, n] += alpha * acc                       (32-bit out: the residual stream)
//   SWIGLU  out[m, n]  = up * gate / (1 + exp(-gate)),  gate = acc over W rows [0, N),
//                                                        up   = acc over W rows [N, 2N)
#include "common.cuh"

#define GEMM_STORE 0
#define GEMM_ACCUM 1
#define GEMM_SWIGLU 2

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                 TO* __restrict__ out, int ldo, int M, int N, int K, float alpha) {
    constexpr int NW = (MODE == GEMM_SWIGLU) ? 2 : 1;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[NW][BK][BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[NW][4][4];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[w][i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, k = e % BK;
            const int gm = m0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
        }
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int e = tid; e < BN * BK; e += 256) {
                const int r = e / BK, k = e % BK;
                const int gn = n0 + r, gk = k0 + k;
                Ws[w][k][r] = (gn < N && gk < K) ? to_float(W[((size_t)w * N + gn) * ldw + gk]) : 0.f;
            }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Ws[w][k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[w][i][j] = fmaf(a[i], b[j], acc[w][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            TO* dst = out + (size_t)gm * ldo + gn;
            if (MODE == GEMM_STORE) {
                *dst = from_float<TO>(alpha * acc[0][i][j]);
            } else if (MODE == GEMM_ACCUM) {
                *dst = from_float<TO>(to_float(*dst) + alpha * acc[0][i][j]);
            } else {
                const float gate = acc[0][i][j], up = acc[NW - 1][i][j];
                *dst = from_float<TO>(up * (gate / (1.0f + expf(-gate))));
            }
        }
    }
}

template <typename TA, typename TW, typename TO>
int launch_modes(int mode, const void* A, int lda, const void* W, int ldw, void* out, int ldo, int M,
                 int N, int K, float alpha, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return LIA_ERR_SIZE;
#define LIA_GEMM(MODE)                                                                          \
    gemm_simt_kernel<TA, TW, TO, MODE><<<grid, 256, 0, stream>>>((const TA*)A, lda, (const TW*)W, \
                                                                 ldw, (TO*)out, ldo, M, N, K, alpha)
    if (mode == GEMM_STORE) LIA_GEMM(GEMM_STORE);
    else if (mode == GEMM_ACCUM) LIA_GEMM(GEMM_ACCUM);
    else if (mode == GEMM_SWIGLU) LIA_GEMM(GEMM_SWIGLU);
    else return LIA_ERR_SIZE;
#undef LIA_GEMM
    return lia_check_launch();
}
}  // namespace

// A [M, K] (a_dtype), W [N, K] or, for SWIGLU, [2N, K] (w_dtype), out [M, N] (out_dtype).
// ACCUM needs a 32-bit out.  Supported element types: (f32, f32 -> f32) and
// (bf16, bf16 -> f32 | bf16).
LIA_EXPORT int lia_gemm_simt(int mode, const void* A, int a_dtype, int lda, const void* W, int w_dtype,
                             int ldw, void* out, int out_dtype, int ldo, int M, int N, int K,
                             float alpha, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return LIA_OK;
    if (K <= 0 || lda < K || ldw < K || ldo < N) return LIA_ERR_SIZE;
    if (mode == GEMM_ACCUM && out_dtype != LIA_F32) return LIA_ERR_DTYPE;
    if (a_dtype == LIA_F32 && w_dtype == LIA_F32 && out_dtype == LIA_F32)
        return launch_modes<float, float, float>(mode, A, lda, W, ldw, out, ldo, M, N, K, alpha, stream);
    if (a_dtype == LIA_BF16 && w_dtype == LIA_BF16 && out_dtype == LIA_F32)
        return launch_modes<__nv_bfloat16, __nv_bfloat16, float>(mode, A, lda, W, ldw, out, ldo, M, N, K,
                                                                 alpha, stream);
    if (a_dtype == LIA_BF16 && w_dtype == LIA_BF16 && out_dtype == LIA_BF16)
        return launch_modes<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(mode, A, lda, W, ldw, out, ldo, M,
                                                                         N, K, alpha, stream);
    return LIA_ERR_DTYPE;
}
