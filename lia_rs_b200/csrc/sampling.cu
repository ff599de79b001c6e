// Token selection on the device: greedy argmax, and temperature sampling by the Gumbel-max
// rule with noise keyed by (seed, position, token), so that a request's draw at a position does
// not depend on the batch it is drawn in.
//
// Greedy: the largest logit; among equal logits the LARGEST token id wins, as the reference's
// `max_by(total_cmp)` keeps the last maximum (src/server/paged/request.rs:117-124,
// src/gpu/kernels/selection.rs:29-35).
// Gumbel: score = (logit - max) / T + g(u(hash(seed, position, token))); hash, u and g follow
// src/sampling/gumbel.rs:4-52 (MurmurHash3 mixer over four words; 32 bits to a uniform in (0,1);
// -log(-log(1-u)) with a series below u = 1/4).  Among equal scores the SMALLEST id wins.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }

__device__ __forceinline__ uint32_t murmur_hash(uint64_t seed, uint64_t position, uint32_t token) {
    uint32_t h = 0;
    const uint32_t words[4] = {(uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)position, token};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t k = rotl32(words[i] * 0xcc9e2d51u, 15) * 0x1b873593u;
        h = rotl32(h ^ k, 13) * 5u + 0xe6546b64u;
    }
    h ^= 16u;
    h ^= h >> 16;
    h *= 0x85ebca6bu;
    h ^= h >> 13;
    h *= 0xc2b2ae35u;
    return h ^ (h >> 16);
}

__device__ __forceinline__ float gumbel_noise(uint32_t word) {
    const float u = (float)(word >> 16) * (1.0f / 65536.0f) +
                    ((float)(word & 65535u) + 0.5f) * (1.0f / 4294967296.0f);
    float negative_log;
    if (u < 0.25f) {
        float poly = 1.0f / 8.0f;
#pragma unroll
        for (int den = 7; den >= 1; --den) poly = fmaf(u, poly, 1.0f / (float)den);
        negative_log = u * poly;
    } else {
        negative_log = -logf(fmaxf(1.0f - u, 1.0f / 16777216.0f));
    }
    return -logf(negative_log);
}

struct Best {
    float value;
    int index;
};

template <bool LARGEST_ID>
__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.index < 0) return a;
    if (a.index < 0) return b;
    if (b.value > a.value) return b;
    if (b.value < a.value) return a;
    if (LARGEST_ID) return b.index > a.index ? b : a;
    return b.index < a.index ? b : a;
}

template <bool LARGEST_ID>
__device__ Best block_best(Best mine, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, mine.value, o), __shfl_xor_sync(0xffffffffu, mine.index, o)};
        mine = better<LARGEST_ID>(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    Best total = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : Best{0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, total.value, o), __shfl_xor_sync(0xffffffffu, total.index, o)};
        total = better<LARGEST_ID>(total, other);
    }
    return total;
}

// One block per row.  temperature[r] <= 0 selects greedy for that row.
__global__ void __launch_bounds__(THREADS)
select_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ seeds, const long long* __restrict__ positions,
              int* __restrict__ out, int rows) {
    __shared__ Best scratch[32];
    const int r = blockIdx.x;
    if (r >= rows) return;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature ? temperature[r] : 0.f;
    Best mine{0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (x != x) continue;   // a NaN never wins
        mine = better<true>(mine, Best{x, i});
    }
    Best top = block_best<true>(mine, scratch);
    if (!(T > 0.f)) {
        if (threadIdx.x == 0) out[r] = top.index;
        return;
    }
    const unsigned long long seed = seeds[r];
    const unsigned long long position = (unsigned long long)positions[r];
    mine = Best{0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (x != x || x == -INFINITY) continue;
        const float score = (x - top.value) / T + gumbel_noise(murmur_hash(seed, position, (uint32_t)i));
        mine = better<false>(mine, Best{score, i});
    }
    Best pick = block_best<false>(mine, scratch);
    if (threadIdx.x == 0) out[r] = pick.index;
}
}  // namespace

// logits [rows, ld >= vocab] 32-bit; temperature [rows] (may be null: all greedy);
// seeds [rows] u64, positions [rows] i64 (used only where temperature > 0); out [rows] i32.
LIA_EXPORT int lia_select_tokens(const float* logits, int ld, int vocab, const float* temperature,
                                 const unsigned long long* seeds, const long long* positions, int* out,
                                 int rows, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (vocab <= 0 || ld < vocab) return LIA_ERR_SIZE;
    select_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, vocab, temperature, seeds, positions, out, rows);
    return lia_check_launch();
}
