// Causal attention of prompt portions over the paged bfloat16 cache on the 5th-generation tensor cores.
//
// A CTA owns 128 query rows = (128 / g) consecutive tokens x the g query heads of one kv head, and walks
// the keys its rows can see, 128 at a time:
//     S = Q K^T     tcgen05.mma, M 128 (rows), N 128 (keys), K head_dim, accumulator in TMEM
//     softmax       two threads per row, each with 64 of its 128 scores from tcgen05.ld (no shuffles: a row lives in
//                   one TMEM lane, which the warps w and w + 4 can both read); the two meet through shared memory
//                   for the row's maximum (a whole number of base-2 logarithms, so rescaling is exact and rare);
//                   each makes the exponentials of its 64 keys and keeps their sum, in 32-bit; probabilities back
//                   to TMEM as bf16 pairs (tcgen05.st)
//     O += P V      tcgen05.mma with P as the operand from TMEM, M 128, N head_dim, K 128 keys, V taken as it lies
//                   in its pages ([key][dim], an MN-major operand), accumulator in TMEM for the whole walk
// Roles: warps 0..7 softmax, warp 8 allocates TMEM and one of its lanes issues the MMAs, warps
// 9..12 bring Q once and then K and V tiles from their pages with cp.async into 128-byte-swizzled shared
// memory (three stages: Q and three tiles of K and V fill it).  The roles meet only through mbarriers, every wait
// on one is bounded.  The first product of tile j + 1 is issued before the softmax of tile j is awaited (two score
// buffers in TMEM), and the softmax of tile j + 1 runs while the second product of tile j does (two buffers of
// probabilities in TMEM, so the softmax never waits for the product that reads the other): the tensor cores and
// the exponentials overlap.  TMEM holds all of it: 2 x 128 columns of scores, 128 of output, 2 x 64 of
// probabilities.
// What bounds a tile (~2,650 cycles, counted per role): the softmax warps work for ~2,100 of them (TMEM load 120,
// the maximum and its exchange 600, the exponentials 1,270, of which the special-function pipe alone needs 1,024 for
// a tile's 16,384 ex2).  It is the number of instructions the softmax warps issue that counts: arguments and sums
// two at a time (fma.f32x2, add.f32x2) and the conversion instruction for a bf16 pair took a tile from 2,650 to
// 2,500 cycles, while exponentials by polynomial on the FMA pipes (ten instructions for one) made it slower.  The one thread that issues the MMAs is held at the tensor pipe's pace for ~1,250 (a
// 128 x 128 x 16 MMA takes 64 cycles alone and 70-100 here, where tcgen05.ld and .st of the softmax share the
// tensor memory's ports) and waits for the probabilities for the rest; the loaders' cp.async of a 64 KB tile keep the
// load/store unit busy for ~1,700.  Two warps per scheduler hide the special-function pipe's latency where one
// thread with 128 scores in registers could keep only two exponentials in flight.
//
// A portion that gives fewer CTAs than the device has SMs (few tokens late in a long prompt) has its keys cut into
// ranges of whole tiles (grid z): each range is a CTA of its own that leaves its unnormalised output, its reference
// point and its sum in scratch memory, and attention_prefill_merge_kernel puts a row's ranges together.
//
// Rows are (token, head) pairs: row r is token r / g, head r % g of the CTA's tokens, so the keys of a kv
// head are read once for all its query heads.  Head sizes 64 and 128, g a divisor of 128; the caller uses
// the mma.sync kernel (attention_prefill.cu) for everything else.
#include "tcgen05.cuh"

using namespace tc5;

namespace {
constexpr int ROWS = 128;                // query rows per CTA: the MMA's M
constexpr int KT = 128;                  // keys per tile: N of the first product, K of the second
constexpr int SOFTMAX_WARPS = 8, LOAD_WARPS = 4;
constexpr int THREADS = (SOFTMAX_WARPS + 1 + LOAD_WARPS) * 32;
constexpr int LOADERS = LOAD_WARPS * 32;
constexpr int STAGES = 3;                // K and V tiles in flight (the probabilities live in tensor memory, so three fit)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LAZY = 8.f;              // see the softmax

struct Params {
    const __nv_bfloat16* q;          // [tokens, nq, D]
    const __nv_bfloat16* k_pages;    // [pages, page_size, nkv, D]
    const __nv_bfloat16* v_pages;
    const int* segments;             // [n_segments][3]: first token's batch index, its position, count
    const int* slots;                // [tokens]
    const int* block_table;          // [slots, table_stride]
    __nv_bfloat16* out;              // [tokens, nq, D]
    int n_segments, table_stride, nq, nkv, page_size, page_shift, window, tokens_per_tile;
    float scale_log2;
    int num_pages;
    int* error_flag;
    // With `splits` > 1 the keys of every CTA's rows are cut into that many ranges (blockIdx.z; whole tiles): each
    // range leaves its output unnormalised and the row's reference point and sum, and the merge kernel puts them together.
    int splits;
    float* partial_o;                // [splits][tokens * nq][D]
    float* partial_ms;               // [splits][tokens * nq][2]: reference point (a whole number, or -infinity), sum
    long long n_rows_total;          // tokens * nq
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two 32-bit floats in one 64-bit register, and the instructions that work on both at once.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float exp2_whole(float n) {       // 2^n for a whole number n <= 0 (or -infinity), exactly
    return n < -126.f ? 0.f : __int_as_float(((int)n + 127) << 23);
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// 16 consecutive columns of this warp's 32 TMEM lanes, written from registers.
__device__ __forceinline__ void tmem_store16(uint32_t addr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}
// 64 consecutive columns of this warp's 32 TMEM lanes into registers; the caller waits (tc5::tmem_load_wait) before use.
__device__ __forceinline__ void tmem_load64_nowait(uint32_t addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(addr));
}
// 32 consecutive columns of this warp's 32 TMEM lanes, written from registers.
__device__ __forceinline__ void tmem_store32(uint32_t addr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// D (+)= A B with A from tensor memory (rows = lanes, two 16-bit elements of K per 32-bit column, the lower index in
// the lower half) and B from shared memory.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A tile of `rows` rows x D elements as the tensor cores want a K-major operand (and, read with the other
// descriptor, an MN-major one): blocks of 64 elements (128 bytes) per row, 128-byte swizzle, 8 rows per 1024
// bytes, the blocks of one row `rows` * 128 bytes apart.  Byte offset of the 16-byte piece `piece` of row `row`.
template <int TILE_ROWS>
__device__ __forceinline__ uint32_t tile_offset(int row, int piece) {
    return (uint32_t)((piece >> 3) * (TILE_ROWS * 128) + (row >> 3) * 1024 + (row & 7) * 128 + (((piece & 7) ^ (row & 7)) << 4));
}
// K-major operand: see smem_desc in tcgen05.cuh.  MN-major operand with 128-byte swizzle: leading offset = the
// distance between two 64-element blocks of the MN dimension, stride offset = the distance between two groups
// of 8 rows of K.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor as instr_desc(), with B taken MN-major.
__device__ __forceinline__ uint32_t instr_desc_b_mn(int m, int n) { return instr_desc(m, n) | (1u << 16); }

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[STAGES], v_full[STAGES], k_empty[STAGES], v_empty[STAGES], s_full[2], p_ready, p_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ short pair_ref[2][2][ROWS];         // what the two threads of a row tell each other (16 bits: shared memory is full to the last KB)
    constexpr int PIECES = D / 8;                      // 16-byte pieces per row
    constexpr uint32_t Q_BYTES = ROWS * D * 2, KV_BYTES = KT * D * 2;
    // tensor memory: two score buffers of 128 columns, the output's head_dim columns (128 kept), and two buffers of
    // probabilities of 64 columns (128 keys as bf16 pairs)
    constexpr int TMEM_COLS = 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = smem_base, kv_s = q_s + Q_BYTES;   // kv_s: [stage][K, V]
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

    // ---- which portion, which tokens, which kv head (later tiles first: they have the most keys) ----
    const int group = p.nq / p.nkv;
    const int kvh = blockIdx.y;
    int tile = gridDim.x - 1 - blockIdx.x, seg = 0, q_offset = 0, seg_start = 0, seg_count = 0;
    for (; seg < p.n_segments; ++seg) {
        q_offset = p.segments[seg * 3];
        seg_start = p.segments[seg * 3 + 1];
        seg_count = p.segments[seg * 3 + 2];
        const int tiles = (seg_count + p.tokens_per_tile - 1) / p.tokens_per_tile;
        if (tile < tiles) break;
        tile -= tiles;
    }
    const bool active = seg < p.n_segments && p.slots[q_offset] >= 0;
    const int tok0 = tile * p.tokens_per_tile;
    const int tok_count = active ? min(p.tokens_per_tile, seg_count - tok0) : 0;
    const int pos_first = seg_start + tok0, pos_last = pos_first + tok_count - 1;
    const int key_end = pos_last + 1;
    int key_begin = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    int n_tiles = active ? (key_end - key_begin + KT - 1) / KT : 0;
    if (p.splits > 1) {                             // this CTA's range of the tiles
        const int per = (n_tiles + p.splits - 1) / p.splits;
        const int first = min(n_tiles, (int)blockIdx.z * per);
        n_tiles = min(n_tiles, first + per) - first;
        key_begin += first * KT;
    }

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), LOADERS);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&k_full[i]), LOADERS);
            mbar_init(smem_u32(&v_full[i]), LOADERS);
            mbar_init(smem_u32(&k_empty[i]), 1);
            mbar_init(smem_u32(&v_empty[i]), 1);
        }
        mbar_init(smem_u32(&s_full[0]), 1);
        mbar_init(smem_u32(&s_full[1]), 1);
        mbar_init(smem_u32(&p_ready), SOFTMAX_WARPS * 32);
        mbar_init(smem_u32(&p_free[0]), 1);
        mbar_init(smem_u32(&p_free[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == SOFTMAX_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 2 * KT, tmem_p = tmem_o + 128;   // score buffer b at tmem_s + b * KT, probabilities b at tmem_p + b * KT / 2
    pdl_launch_dependents();
    pdl_wait();                                   // q and this step's keys come from the kernel ahead

    if (warp > SOFTMAX_WARPS && n_tiles > 0) {
        // ---- loaders: Q once, then the K and V tiles, each thread whole 16-byte pieces ----
        const int lt = threadIdx.x - (SOFTMAX_WARPS + 1) * 32;            // 0..127
        const int* table = p.block_table + (size_t)p.slots[q_offset] * p.table_stride;
        for (int id = lt; id < ROWS * PIECES; id += LOADERS) {
            const int r = id / PIECES, piece = id % PIECES;
            const int tok = r / group, head = r % group;
            const bool valid = tok < tok_count;
            const size_t src = ((size_t)(q_offset + tok0 + (valid ? tok : 0)) * p.nq + kvh * group + head) * D + piece * 8;
            cp_async_16(q_s + tile_offset<ROWS>(r, piece), p.q + src, valid);
        }
        cp_async_commit();                        // (Q is awaited below, with the first tile's copies already on their way)
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % STAGES;
            // the keys' stage is free as soon as the first product of three tiles ago has read it, the values' stage
            // only after the second
            if (j >= STAGES && !mbar_wait(smem_u32(&k_empty[st]), ((uint32_t)(j / STAGES) & 1u) ^ 1u)) { ok = false; break; }
            const uint32_t ks = kv_s + (uint32_t)st * 2 * KV_BYTES, vs = ks + KV_BYTES;
            const int key0 = key_begin + j * KT;
            // PIECES lanes share a key row (their 16-byte pieces make one coalesced request); lane j of them looks
            // up the row of pass j
            {
                constexpr int ROWS_PER_PASS = LOADERS / PIECES, PASSES = KT / ROWS_PER_PASS;
                static_assert(PASSES <= PIECES, "one lane per pass");
                const int sub = lt / PIECES, piece = lt % PIECES, lane_group = (lane / PIECES) * PIECES;
                int my_row = -1, rows[PASSES];
                if (piece < PASSES) {
                    const int key = key0 + sub + piece * ROWS_PER_PASS;
                    if (key < key_end) my_row = cache_row_of(table, key, p.page_size, p.page_shift, p.num_pages, p.error_flag);
                }
#pragma unroll
                for (int i = 0; i < PASSES; ++i) {
                    const int row = __shfl_sync(0xffffffffu, my_row, lane_group + i);
                    const bool valid = row >= 0;
                    const size_t src = ((size_t)(valid ? row : 0) * p.nkv + kvh) * D + piece * 8;
                    const uint32_t at = tile_offset<KT>(sub + i * ROWS_PER_PASS, piece);
                    cp_async_16(ks + at, p.k_pages + src, valid);
                    rows[i] = row;
                }
                cp_async_commit();
                if (j >= STAGES && !mbar_wait(smem_u32(&v_empty[st]), ((uint32_t)(j / STAGES) & 1u) ^ 1u)) { ok = false; break; }
#pragma unroll
                for (int i = 0; i < PASSES; ++i) {
                    const bool valid = rows[i] >= 0;
                    const size_t src = ((size_t)(valid ? rows[i] : 0) * p.nkv + kvh) * D + piece * 8;
                    cp_async_16(vs + tile_offset<KT>(sub + i * ROWS_PER_PASS, piece), p.v_pages + src, valid);
                }
                cp_async_commit();
            }
            if (j == 0) {
                asm volatile("cp.async.wait_group 2;" ::: "memory");    // Q has landed (groups complete in the order they were made)
                fence_async_smem();
                mbar_arrive(smem_u32(&q_full));
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");        // the keys have landed
            fence_async_smem();
            mbar_arrive(smem_u32(&k_full[st]));
            cp_async_wait_all();
            fence_async_smem();
            mbar_arrive(smem_u32(&v_full[st]));
        }
        if (!ok && p.error_flag) atomicExch(p.error_flag, 3);
    } else if (warp == SOFTMAX_WARPS && lane == 0 && n_tiles > 0) {
        // ---- MMA issuer ----
        const uint32_t idesc_s = instr_desc(ROWS, KT), idesc_o = instr_desc_b_mn(ROWS, D);
        bool ok = mbar_wait(smem_u32(&q_full), 0u);
        // the operands' descriptors: the tile's first plus an offset in their lowest field (the start address in 16-byte
        // units; shared memory ends below what the field holds), so that an MMA costs this thread an addition
        static_assert(ROWS == KT, "Q and K tiles share their offsets");
        const uint64_t desc_q0 = smem_desc(q_s), desc_kv0 = smem_desc(kv_s), desc_v0 = smem_desc_mn(kv_s + KV_BYTES, KT * 128, 1024);
        // S_j = Q K_j^T into score buffer j & 1: issued one tile ahead, so that it runs while the softmax of the
        // tile before is at work (that buffer's last reader arrived on p_ready two tiles ago)
        auto first_product = [&](int j) {
            const int st = j % STAGES;
            if (!mbar_wait(smem_u32(&k_full[st]), (uint32_t)(j / STAGES) & 1u)) { ok = false; return; }
            tc_fence_after();
            const uint64_t desc_k = desc_kv0 + (uint64_t)((uint32_t)st * (2 * KV_BYTES >> 4));
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t offset = (uint64_t)(((kk >> 2) * (ROWS * 128) + (kk & 3) * 32) >> 4);      // Q and K tiles are laid out alike
                tc_mma(tmem_s + (uint32_t)((j & 1) * KT), desc_q0 + offset, desc_k + offset, idesc_s, kk > 0 ? 1u : 0u);
            }
            tc_commit(smem_u32(&s_full[j & 1]));
            tc_commit(smem_u32(&k_empty[st]));
        };
        if (ok) first_product(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % STAGES;
            const uint64_t desc_v = desc_v0 + (uint64_t)((uint32_t)st * (2 * KV_BYTES >> 4));
            if (j + 1 < n_tiles) first_product(j + 1);
            if (!ok) break;
            // O += P V once the values lie in shared memory and the probabilities in TMEM (and O has been rescaled if it had to be)
            if (!mbar_wait(smem_u32(&v_full[st]), (uint32_t)(j / STAGES) & 1u)) { ok = false; break; }
            if (!mbar_wait(smem_u32(&p_ready), (uint32_t)j & 1u)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int ks16 = 0; ks16 < KT / 16; ++ks16) {
                // (16 keys = two groups of 8 rows = 2,048 bytes further in the tile)
                tc_mma_ts(tmem_o, tmem_p + (uint32_t)((j & 1) * (KT / 2) + ks16 * 8), desc_v + (uint64_t)(ks16 * (2048 >> 4)), idesc_o, (j > 0 || ks16 > 0) ? 1u : 0u);
            }
            tc_commit(smem_u32(&v_empty[st]));
            tc_commit(smem_u32(&p_free[j & 1]));       // this tile's buffer of probabilities is free again, and O holds the tile
        }
        if (!ok && p.error_flag) atomicExch(p.error_flag, 3);
    } else if (warp < SOFTMAX_WARPS && n_tiles > 0) {
        // ---- softmax: warp w and warp w + 4 share the rows of TMEM lanes 32 (w % 4) ..; each takes half the keys of
        //      a tile and half the output's columns ----
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;                                  // 0..127
        const int tok = r / group, head = r % group;
        const bool row_ok = tok < tok_count;
        const int pos = row_ok ? pos_first + tok : 0x3fffffff;              // a row beyond the portion sees every key and is never written
        const uint32_t lane_base = ((uint32_t)(quarter * 32) << 16);
        constexpr int HALF = KT / 2;
        float row_max = -INFINITY, row_sum = 0.f;                           // the sum: of this thread's keys only
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int key0 = key_begin + j * KT + half * HALF;              // this thread's first key of the tile
            if (!mbar_wait(smem_u32(&s_full[j & 1]), ((uint32_t)j >> 1) & 1u)) { ok = false; break; }
            tc_fence_after();
            const bool masked = key_begin + j * KT + KT - 1 > pos_first || (p.window > 0 && key_begin + j * KT <= pos_last - p.window);
            uint32_t raw[HALF];
            tmem_load64_nowait(tmem_s + (uint32_t)((j & 1) * KT + half * HALF) + lane_base, raw);
            tmem_load_wait();
            if (masked) {
#pragma unroll
                for (int c = 0; c < HALF; ++c) {
                    const int key = key0 + c;
                    bool visible = key <= pos;
                    if (p.window > 0) visible = visible && key > pos - p.window;
                    if (!visible) raw[c] = 0xff800000u;                         // -infinity
                }
            }
            float tile_max;
            {   // four chains: a single one would be 64 instructions that wait for one another
                float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < HALF; ++c) part[c & 3] = fmaxf(part[c & 3], __uint_as_float(raw[c]));
                tile_max = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
            }
            // the row's maximum: the two threads tell each other theirs (two buffers: the partner may still read
            // the tile before's while this thread writes; the barrier of a tile orders the tile before's reads)
            // Whole-number reference point: see attention_decode.cu.  What the two threads exchange is that whole number
            // (the ceiling of the larger maximum is the larger ceiling), as 16 bits: beyond +-126 a 32-bit exponential
            // is 0 or infinite anyway, so the clamp to +-30,000 changes nothing; -32,768 stands for minus infinity.
            const float own_ref = ceilf(tile_max * p.scale_log2);
            pair_ref[j & 1][half][r] = own_ref == -INFINITY ? (short)-32768 : (short)fminf(fmaxf(own_ref, -30000.f), 30000.f);
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            const short both = max(pair_ref[j & 1][0][r], pair_ref[j & 1][1][r]);
            // ... and it moves only when the tile's maximum lies more than LAZY whole numbers above it: the
            // probabilities then reach 2^LAZY at most, which bf16 and the 32-bit sums hold, and O is rescaled once
            // or twice in a row's walk instead of at most of its first tiles (686 cycles each time)
            const float tile_ref = both == -32768 ? -INFINITY : (float)both;
            const float new_max = (row_max == -INFINITY || tile_ref > row_max + LAZY) ? fmaxf(row_max, tile_ref) : row_max;
            const float safe_max = new_max == -INFINITY ? 0.f : new_max;        // a row that has seen no key yet
            const float correction = exp2_whole(row_max - safe_max);
            row_max = new_max;
            row_sum *= correction;
            // probabilities, as bf16 pairs (the scores' registers are reused)
            // (two scores at a time where the instruction set has it: one fused multiply-add for a pair's arguments,
            // one addition for a pair's contributions to the sums; the softmax warps are bound by how many
            // instructions they issue, not by the pipes)
            uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};             // four chains of pairs again, met in a fixed order
            const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), shift2 = pack_f32x2(-safe_max, -safe_max);
#pragma unroll
            for (int c = 0; c < HALF; c += 2) {
                float x0, x1;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(raw[c]), __uint_as_float(raw[c + 1])), scale2, shift2), x0, x1);
                const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                sums[(c >> 1) & 3] = add_f32x2(sums[(c >> 1) & 3], pack_f32x2(e0, e1));
                // to a bf16 pair with the conversion instruction: it shares the exponentials' pipe (4 cycles a warp
                // beside their 2 x 8), which has room, and is one instruction where rounding with integer adds and a
                // byte permute is three (measured: 340 -> 331 us at 8,192 tokens)
                const __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
                raw[c >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
            }
            {
                float lo, hi;
                unpack_f32x2(add_f32x2(add_f32x2(sums[0], sums[1]), add_f32x2(sums[2], sums[3])), lo, hi);
                row_sum += lo + hi;
            }
            // This tile's buffer of probabilities (one of two) is free once the second product of two tiles ago is done:
            // it is, since this tile's scores are there: the commit that announced them stands for every MMA the
            // issuing thread had issued before, and the second product of two tiles ago is one of them.  O may be
            // rescaled only when the second product of the tile before is done, which is awaited where it happens
            // (that barrier has then completed all its earlier phases and at most this one: the parity tells).
            const bool rescale = __any_sync(0xffffffffu, correction != 1.f) && j > 0;
            if (rescale) {
                if (!mbar_wait(smem_u32(&p_free[(j - 1) & 1]), (uint32_t)((j - 1) >> 1) & 1u)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 16) {
                    float o[16];
                    tmem_load16(tmem_o + lane_base + (uint32_t)c0, o);
#pragma unroll
                    for (int c = 0; c < 16; ++c) o[c] *= correction;
                    tmem_store16(tmem_o + lane_base + (uint32_t)c0, o);
                }
                tmem_store_wait();
            }
            tmem_store32(tmem_p + lane_base + (uint32_t)((j & 1) * (KT / 2) + half * (HALF / 2)), raw);
            tmem_store_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&p_ready));
        }
        // ---- the row's output: the two threads' sums meet, each writes half the columns ----
        if (ok && !mbar_wait(smem_u32(&p_free[(n_tiles - 1) & 1]), (uint32_t)((n_tiles - 1) >> 1) & 1u)) ok = false;
        tc_fence_after();
        float* pair_sum = reinterpret_cast<float*>(smem);                   // [2][ROWS], where Q was: every product is done
        pair_sum[half * ROWS + r] = row_sum;
        asm volatile("bar.sync 5, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
        if (ok && p.splits > 1) {
            // this range's share of the row: O as it stands, the reference point and the sum of the exponentials
            const size_t row = (size_t)(q_offset + tok0 + (row_ok ? tok : 0)) * p.nq + kvh * group + head;
            const size_t plane = (size_t)blockIdx.z * p.n_rows_total + row;
            if (row_ok && half == 0) {
                p.partial_ms[plane * 2] = row_max;
                p.partial_ms[plane * 2 + 1] = pair_sum[r] + pair_sum[ROWS + r];
            }
            float* dst = p.partial_o + plane * D;
#pragma unroll 1
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 16) {
                float o[16];
                tmem_load16(tmem_o + lane_base + (uint32_t)c0, o);
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 16; c += 4) *reinterpret_cast<float4*>(dst + c0 + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                }
            }
        } else if (ok) {
            const float inv = 1.0f / (pair_sum[r] + pair_sum[ROWS + r]);
            __nv_bfloat16* dst = p.out + ((size_t)(q_offset + tok0 + (row_ok ? tok : 0)) * p.nq + kvh * group + head) * D;
#pragma unroll 1
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 16) {
                float o[16];
                tmem_load16(tmem_o + lane_base + (uint32_t)c0, o);           // every lane takes part in the load
                if (row_ok) {
                    uint32_t packed[8];
#pragma unroll
                    for (int c = 0; c < 16; c += 2) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
                        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    *reinterpret_cast<uint4*>(dst + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        } else if (lane == 0 && p.error_flag) {
            atomicExch(p.error_flag, 3);
        }
    } else if (warp < 4 && n_tiles == 0 && p.splits > 1 && active) {
        // a range without tiles (fewer tiles than ranges): it says so, its output is never read
        const int r = threadIdx.x, tok = r / group, head = r % group;
        if (tok < tok_count) {
            const size_t row = (size_t)(q_offset + tok0 + tok) * p.nq + kvh * group + head;
            const size_t plane = (size_t)blockIdx.z * p.n_rows_total + row;
            p.partial_ms[plane * 2] = -INFINITY;
            p.partial_ms[plane * 2 + 1] = 0.f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == SOFTMAX_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// The ranges of a row put together: for every row of a CTA's tokens
//     out = sum_i 2^(m_i - M) O_i / sum_i 2^(m_i - M) s_i,   M = max_i m_i,
// the ranges in ascending order; the m_i are whole numbers, so the weights are exact powers of two.  Grid as the
// kernel above, its z counting groups of four rows: a warp per row, lane i holding range i's m and s (at most 32
// ranges), every lane a few of the row's elements.
template <int D>
__global__ void __launch_bounds__(128) attention_prefill_merge_kernel(Params p) {
    pdl_launch_dependents();
    const int group = p.nq / p.nkv;
    const int kvh = blockIdx.y;
    int tile = gridDim.x - 1 - blockIdx.x, seg = 0, q_offset = 0, seg_count = 0;
    for (; seg < p.n_segments; ++seg) {
        q_offset = p.segments[seg * 3];
        seg_count = p.segments[seg * 3 + 2];
        const int tiles = (seg_count + p.tokens_per_tile - 1) / p.tokens_per_tile;
        if (tile < tiles) break;
        tile -= tiles;
    }
    const bool active = seg < p.n_segments && p.slots[q_offset] >= 0;
    const int tok0 = tile * p.tokens_per_tile;
    const int tok_count = active ? min(p.tokens_per_tile, seg_count - tok0) : 0;
    constexpr int E = D / 32;                          // elements per lane: 2 or 4
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.z * 4 + warp, tok = r / group, head = r % group;
    pdl_wait();
    if (tok >= tok_count) return;
    const size_t row = (size_t)(q_offset + tok0 + tok) * p.nq + kvh * group + head;
    float m = -INFINITY, sum = 0.f;
    if (lane < p.splits) {
        const float2 ms = *reinterpret_cast<const float2*>(p.partial_ms + ((size_t)lane * p.n_rows_total + row) * 2);
        m = ms.x;
        sum = ms.y;
    }
    float top = m;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
    const float weight = m == -INFINITY ? 0.f : exp2_whole(m - top);     // 0: a range in which the row saw no key
    float acc[E], total = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;
    const float* o = p.partial_o + row * D + lane * E;
#pragma unroll 4
    for (int i = 0; i < p.splits; ++i) {
        const float w = __shfl_sync(0xffffffffu, weight, i), s_i = __shfl_sync(0xffffffffu, sum, i);
        if (w == 0.f) continue;                        // its output may never have been written
        total = fmaf(w, s_i, total);
        const float* src = o + (size_t)i * p.n_rows_total * D;
#pragma unroll
        for (int e = 0; e < E; e += 2) {
            const float2 v = *reinterpret_cast<const float2*>(src + e);
            acc[e] = fmaf(w, v.x, acc[e]);
            acc[e + 1] = fmaf(w, v.y, acc[e + 1]);
        }
    }
    const float inv = 1.0f / total;
    __nv_bfloat16* dst = p.out + row * D + lane * E;
#pragma unroll
    for (int e = 0; e < E; e += 2) *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(acc[e] * inv, acc[e + 1] * inv);
}

template <int D>
int launch(const Params& p, int n_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)ROWS * D * 2 + (size_t)STAGES * 2 * KT * D * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    const int rc = lia_launch(attention_prefill_tc_kernel<D>, dim3(n_tiles, p.nkv, p.splits), dim3(THREADS), smem, stream, p);
    if (rc != LIA_OK || p.splits <= 1) return rc;
    return lia_launch(attention_prefill_merge_kernel<D>, dim3(n_tiles, p.nkv, ROWS / 4), dim3(128), 0, stream, p);
}
}  // namespace

// Tokens of a portion that one CTA takes for `group` query heads per kv head and this head size (0: the tcgen05
// kernel does not take the combination; use lia_attention_prefill).
LIA_EXPORT int lia_attention_prefill_tc_tokens_per_tile(int group, int d) {
    if (d != 64 && d != 128) return 0;
    return group >= 1 && group <= ROWS && ROWS % group == 0 ? ROWS / group : 0;
}

// Arguments as lia_attention_prefill; `n_tiles` = sum over portions of ceil(count / tokens_per_tile) with the
// tokens per tile of this kernel.  With `splits` > 1 every CTA's keys are cut into that many ranges of whole
// 128-key tiles, each range a CTA of its own, and a second kernel merges them (few tokens over a long context
// would otherwise leave most SMs idle); `partial` then holds splits * n_tokens * nq * (head size + 2) 32-bit words,
// `n_tokens` being the tokens of the whole batch that `q` and `out` cover.
LIA_EXPORT int lia_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* segments,
                                        int n_segments, int n_tiles, const int* slots, const int* block_table,
                                        int table_stride, void* out, int nq, int nkv, int d, int page_size, int window,
                                        float scale, int num_pages, int splits, float* partial, int n_tokens,
                                        int* error_flag, cudaStream_t stream) {
    if (n_segments <= 0 || n_tiles <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || nkv > 65535) return LIA_ERR_SIZE;
    if (splits < 1 || splits > 32 || (splits > 1 && (!partial || n_tokens <= 0))) return LIA_ERR_SIZE;
    const int per_tile = lia_attention_prefill_tc_tokens_per_tile(nq / nkv, d);
    if (per_tile == 0) return LIA_ERR_SIZE;
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 15u) || ((uintptr_t)k_pages & 15u) || ((uintptr_t)v_pages & 15u) ||
        ((uintptr_t)partial & 15u))
        return LIA_ERR_ALIGN;
    Params p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.segments = segments; p.slots = slots; p.block_table = block_table; p.out = (__nv_bfloat16*)out;
    p.n_segments = n_segments; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
    p.window = window; p.tokens_per_tile = per_tile; p.scale_log2 = scale * LOG2E; p.error_flag = error_flag;
    p.num_pages = num_pages;
    p.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if (page_size == (1 << b)) p.page_shift = b;
    p.splits = splits;
    p.n_rows_total = (long long)n_tokens * nq;
    p.partial_o = partial;
    p.partial_ms = partial ? partial + (size_t)splits * p.n_rows_total * d : nullptr;
    if (d == 128) return launch<128>(p, n_tiles, stream);
    return launch<64>(p, n_tiles, stream);
}
