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
constexpr int PART_THREADS = 256;
constexpr int MAX_ROWS = 65535;          // rows of one call (the grid's second dimension)

// Ranges a row is cut into: about 2,048 tokens each, at most 64.
inline int select_parts(int vocab) {
    const int parts = (vocab + 2047) / 2048;
    return parts < 1 ? 1 : (parts > 64 ? 64 : parts);
}

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

// The sum of a value over the CTA, in a fixed tree (every thread calls it; every thread gets the sum).
__device__ double block_sum(double mine, double* warp_sums) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    __syncthreads();
    if (lane == 0) warp_sums[warp] = mine;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_sums[w];
    return total;
}

// A row is cut into `parts` ranges of `chunk` tokens, a CTA each, so that a handful of rows still keeps many SMs
// busy; the CTA that finishes a row last (a counter that it leaves at zero again) picks among the ranges' bests.
// `better` is a total order (value, then id), so the pick does not depend on which CTA that is.
// PICK false: the row's largest logit: the greedy choice, written to out, and the reference point of the
// Gumbel scores, written to tops.  PICK true (rows with temperature > 0 only): the best Gumbel score.
template <bool PICK>
__global__ void __launch_bounds__(PART_THREADS)
select_part_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
                   const unsigned long long* __restrict__ seeds, const long long* __restrict__ positions,
                   int* __restrict__ out, int parts, int chunk, int* __restrict__ counters, float* __restrict__ tops,
                   float* __restrict__ part_value, int* __restrict__ part_index) {
    __shared__ Best scratch[32];
    __shared__ int last;
    pdl_launch_dependents();
    const int r = blockIdx.y, part = blockIdx.x;
    const float T = temperature ? temperature[r] : 0.f;
    if (PICK && !(T > 0.f)) return;
    pdl_wait();                                        // the logits come from the kernel ahead
    const float* row = logits + (size_t)r * ld;
    const int begin = part * chunk, end = min(vocab, begin + chunk);
    Best mine{0.f, -1};
    if (!PICK) {
#pragma unroll 4
        for (int i = begin + threadIdx.x; i < end; i += PART_THREADS) {
            const float x = row[i];
            if (x == x) mine = better<true>(mine, Best{x, i});       // a NaN never wins
        }
    } else {
        const float top = tops[r];
        const unsigned long long seed = seeds[r];
        const unsigned long long position = (unsigned long long)positions[r];
#pragma unroll 4
        for (int i = begin + threadIdx.x; i < end; i += PART_THREADS) {
            const float x = row[i];
            if (x != x || x == -INFINITY) continue;
            const float score = (x - top) / T + gumbel_noise(murmur_hash(seed, position, (uint32_t)i));
            mine = better<false>(mine, Best{score, i});
        }
    }
    const Best best = block_best<!PICK>(mine, scratch);
    if (threadIdx.x == 0) {
        part_value[(size_t)r * parts + part] = best.value;
        part_index[(size_t)r * parts + part] = best.index;
        __threadfence();
        const int seen = atomicAdd(&counters[r], 1);
        last = seen == parts - 1;
        if (last) counters[r] = 0;
    }
    __syncthreads();
    if (!last || threadIdx.x >= 32) return;
    __threadfence();
    Best pick{0.f, -1};
    for (int i = threadIdx.x; i < parts; i += 32)
        pick = better<!PICK>(pick, Best{__ldcg(part_value + (size_t)r * parts + i), __ldcg(part_index + (size_t)r * parts + i)});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, pick.value, o), __shfl_xor_sync(0xffffffffu, pick.index, o)};
        pick = better<!PICK>(pick, other);
    }
    if (threadIdx.x == 0) {
        out[r] = pick.index;
        if (!PICK) tops[r] = pick.value;
    }
}

// The best `k` logits of every row with their token ids, best first: larger logit, among equal logits the
// larger id (the order in which the host's sampling rule takes its top_k candidates); minus infinity is no
// candidate, a row with fewer than k others ends in ids of -1.  `nonfinite` counts NaN and infinities of either
// sign over all rows (the host refuses such logits).  A row is cut into ranges as above: every CTA keeps its
// range in shared memory and takes its best k out of it one by one; the last CTA of a row to finish does the
// same with the ranges' candidates.
__global__ void __launch_bounds__(PART_THREADS)
candidates_kernel(const float* __restrict__ logits, int ld, int vocab, int k, float* __restrict__ out_value,
                  int* __restrict__ out_index, int* __restrict__ nonfinite, int parts, int chunk,
                  int* __restrict__ counters, float* __restrict__ part_value, int* __restrict__ part_index,
                  const double* __restrict__ temperature, double* __restrict__ mass, double* __restrict__ part_mass) {
    extern __shared__ float held[];                     // the range's logits; later the row's parts * k candidates
    __shared__ Best scratch[32];
    __shared__ double sums[PART_THREADS / 32];
    __shared__ int last;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, part = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int begin = part * chunk, count = max(0, min(vocab, begin + chunk) - begin);
    int odd = 0;
    for (int i = threadIdx.x; i < count; i += PART_THREADS) {
        const float x = row[begin + i];
        odd += !(fabsf(x) <= 3.402823466e38f);          // NaN or an infinity
        held[i] = x == x ? x : -INFINITY;
    }
    if (odd) atomicAdd(nonfinite, odd);
    __syncthreads();
    if (mass) {
        // the range's share of the row's softmax mass at the row's temperature, in 64-bit: its largest logit and
        // the sum of exp((x - largest) / T) over it, added up in an order that depends on nothing but the sizes
        Best mine{0.f, -1};
        for (int i = threadIdx.x; i < count; i += PART_THREADS)
            if (held[i] != -INFINITY) mine = better<true>(mine, Best{held[i], begin + i});
        const Best top = block_best<true>(mine, scratch);
        const double t = temperature[r];
        double sum = 0.0;
        if (top.index >= 0 && t > 0.0)
            for (int i = threadIdx.x; i < count; i += PART_THREADS)
                if (held[i] != -INFINITY) sum += exp(((double)held[i] - (double)top.value) / t);
        sum = block_sum(sum, sums);
        if (threadIdx.x == 0) {
            part_mass[((size_t)r * parts + part) * 2] = top.index >= 0 ? (double)top.value : -INFINITY;
            part_mass[((size_t)r * parts + part) * 2 + 1] = sum;
        }
    }
    for (int n = 0; n < k; ++n) {
        Best mine{0.f, -1};
        for (int i = threadIdx.x; i < count; i += PART_THREADS)
            if (held[i] != -INFINITY) mine = better<true>(mine, Best{held[i], begin + i});
        const Best best = block_best<true>(mine, scratch);
        if (threadIdx.x == 0) {
            part_value[((size_t)r * parts + part) * k + n] = best.index >= 0 ? best.value : -INFINITY;
            part_index[((size_t)r * parts + part) * k + n] = best.index;
            if (best.index >= 0) held[best.index - begin] = -INFINITY;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        __threadfence();
        const int seen = atomicAdd(&counters[r], 1);
        last = seen == parts - 1;
        if (last) counters[r] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (mass) {
        // the ranges' shares brought to the row's largest logit: total = sum_p sum_p * exp((largest_p - largest) / T)
        const double t = temperature[r];
        double largest = -INFINITY;
        for (int p = 0; p < parts; ++p) largest = fmax(largest, __ldcg(part_mass + ((size_t)r * parts + p) * 2));
        double term = 0.0;
        for (int p = threadIdx.x; p < parts; p += PART_THREADS) {
            const double share = __ldcg(part_mass + ((size_t)r * parts + p) * 2 + 1);
            if (share > 0.0 || share != share)
                term += share * exp((__ldcg(part_mass + ((size_t)r * parts + p) * 2) - largest) / t);
        }
        term = block_sum(term, sums);
        if (threadIdx.x == 0) {
            mass[(size_t)r * 2] = largest;
            mass[(size_t)r * 2 + 1] = term;
        }
    }
    const int all = parts * k;                            // at most 64 * 32 candidates: they fit where the range lay (see the launch)
    int* held_index = reinterpret_cast<int*>(held + all);
    for (int i = threadIdx.x; i < all; i += PART_THREADS) {
        held[i] = __ldcg(part_value + (size_t)r * all + i);
        held_index[i] = __ldcg(part_index + (size_t)r * all + i);
    }
    __syncthreads();
    for (int n = 0; n < k; ++n) {
        Best mine{0.f, -1};
        int where = -1;
        for (int i = threadIdx.x; i < all; i += PART_THREADS) {
            if (held_index[i] < 0) continue;
            const Best here{held[i], held_index[i]};
            const Best top = better<true>(mine, here);
            if (top.index == here.index) { mine = here; where = i; }
        }
        const Best best = block_best<true>(mine, scratch);
        if (best.index >= 0 && mine.index == best.index && where >= 0) held_index[where] = -1;    // token ids are unique: one thread owns it
        if (threadIdx.x == 0) {
            out_value[(size_t)r * k + n] = best.index >= 0 ? best.value : -INFINITY;
            out_index[(size_t)r * k + n] = best.index;
        }
        __syncthreads();
    }
}
}  // namespace

// Floats of scratch that `rows` rows of `vocab` logits need (zero before the first call).  Its first MAX_ROWS words
// are the rows' counters, whatever the number of rows, and every call leaves them zero; the rest is rewritten by
// every call.
LIA_EXPORT long long lia_select_tokens_scratch_floats(int rows, int vocab) {
    const int parts = select_parts(vocab);
    return (long long)MAX_ROWS + (long long)rows * (1 + 2 * parts);
}

// logits [rows, ld >= vocab] 32-bit; temperature [rows] (may be null: all greedy);
// seeds [rows] u64, positions [rows] i64 (used only where temperature > 0); out [rows] i32;
// scratch: lia_select_tokens_scratch_floats(rows, vocab) 32-bit words.
LIA_EXPORT int lia_select_tokens(const float* logits, int ld, int vocab, const float* temperature,
                                 const unsigned long long* seeds, const long long* positions, int* out,
                                 int rows, float* scratch, long long scratch_floats, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (vocab <= 0 || ld < vocab || rows > MAX_ROWS) return LIA_ERR_SIZE;
    if (!scratch || scratch_floats < lia_select_tokens_scratch_floats(rows, vocab)) return LIA_ERR_SIZE;
    const int parts = select_parts(vocab);
    const int chunk = (vocab + parts - 1) / parts;
    int* counters = reinterpret_cast<int*>(scratch);
    float* tops = scratch + MAX_ROWS;
    float* part_value = tops + rows;
    int* part_index = reinterpret_cast<int*>(part_value + (size_t)rows * parts);
    int rc = lia_launch(select_part_kernel<false>, dim3(parts, rows), dim3(PART_THREADS), 0, stream, logits, ld, vocab,
                        temperature, seeds, positions, out, parts, chunk, counters, tops, part_value, part_index);
    if (rc != LIA_OK || !temperature) return rc;
    return lia_launch(select_part_kernel<true>, dim3(parts, rows), dim3(PART_THREADS), 0, stream, logits, ld, vocab,
                      temperature, seeds, positions, out, parts, chunk, counters, tops, part_value, part_index);
}

// Most candidates a row can be asked for.
LIA_EXPORT int lia_select_candidates_max() { return 32; }

// Floats of scratch for lia_select_candidates (zero before the first call; the counters at its head stay zero).
LIA_EXPORT long long lia_select_candidates_scratch_floats(int rows, int vocab, int k) {
    return (long long)MAX_ROWS + 1 + 2LL * rows * select_parts(vocab) * k + 4LL * rows * select_parts(vocab);
}

// logits [rows, ld >= vocab] 32-bit; out_value, out_index [rows, k], 1 <= k <= 32; nonfinite: one int32 that the
// kernel adds to.  With `temperature` [rows] and `mass` [rows, 2] (64-bit, both or neither): mass[r] = (the row's
// largest logit, the sum over the row of exp((x - largest) / temperature[r])), 0 where the temperature is 0.
LIA_EXPORT int lia_select_candidates(const float* logits, int ld, int vocab, int rows, int k, float* out_value,
                                     int* out_index, int* nonfinite, const double* temperature, double* mass,
                                     float* scratch, long long scratch_floats, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (vocab <= 0 || ld < vocab || rows > MAX_ROWS || k < 1 || k > 32 || !nonfinite) return LIA_ERR_SIZE;
    if ((temperature == nullptr) != (mass == nullptr)) return LIA_ERR_SIZE;
    if (reinterpret_cast<uintptr_t>(scratch) % 8) return LIA_ERR_SIZE;
    if (!scratch || scratch_floats < lia_select_candidates_scratch_floats(rows, vocab, k)) return LIA_ERR_SIZE;
    const int parts = select_parts(vocab);
    const int chunk = (vocab + parts - 1) / parts;
    const size_t range = (size_t)chunk * sizeof(float), merged = (size_t)parts * k * 2 * sizeof(float);
    const size_t smem = range > merged ? range : merged;
    if (smem > 200 * 1024) return LIA_ERR_SIZE;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        if (cudaFuncSetAttribute(candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = smem;
    }
    int* counters = reinterpret_cast<int*>(scratch);
    float* part_value = scratch + MAX_ROWS;
    int* part_index = reinterpret_cast<int*>(part_value + (size_t)rows * parts * k);
    const size_t words = (size_t)MAX_ROWS + 2 * (size_t)rows * parts * k;
    double* part_mass = reinterpret_cast<double*>(scratch + words + (words & 1));      // on an 8-byte boundary
    return lia_launch(candidates_kernel, dim3(parts, rows), dim3(PART_THREADS), smem, stream, logits, ld, vocab, k, out_value,
                      out_index, nonfinite, parts, chunk, counters, part_value, part_index, temperature, mass, part_mass);
}
