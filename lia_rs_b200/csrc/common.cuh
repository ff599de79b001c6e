// Shared helpers of the sm_100a kernel library.
//
// Conventions of every launcher in this library:
//  * exported with C linkage, called from Python through ctypes;
//  * returns 0 on success or a negative code (see LIA_ERR_*), never throws, never allocates;
//  * validates sizes on the host before the launch and refuses what the kernel cannot
//    compute rather than computing it wrongly;
//  * runs on the stream it is given.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LIA_OK 0
#define LIA_ERR_SIZE (-1)        // a size the kernel refuses
#define LIA_ERR_ALIGN (-2)       // a pointer or stride that is not aligned as required
#define LIA_ERR_LAUNCH (-3)      // cudaGetLastError() after the launch was not cudaSuccess
#define LIA_ERR_DRIVER (-4)      // a driver entry point (tensor map encode) is missing or failed
#define LIA_ERR_DTYPE (-5)       // a combination of element types that has no instantiation

#define LIA_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
#define LIA_F32 0
#define LIA_BF16 1

// Kernels launched by this library since it was loaded (every launcher calls lia_check_launch once per
// kernel).  Read through lia_kernel_launches(); a benchmark's own count of its launches.
#include <atomic>
inline std::atomic<long long> lia_launch_counter{0};

static inline int lia_check_launch() {
    lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
}

// Programmatic dependent launch.  A kernel launched through lia_launch may begin while the kernel
// before it in the stream is still running; it must call pdl_wait() before it touches anything that
// kernel wrote or read (weights and other constants may be fetched earlier), and may call
// pdl_launch_dependents() once it no longer matters when the next kernel starts.  Both are no-ops in
// a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1: launches carry the programmatic-serialization attribute (default); 0: ordinary launches.
inline std::atomic<int> lia_pdl_enabled{1};

template <typename... KArgs, typename... Args>
static inline int lia_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = lia_pdl_enabled.load(std::memory_order_relaxed) ? 1 : 0;
    lia_launch_counter.fetch_add(1, std::memory_order_relaxed);
    if (cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...) != cudaSuccess) {
        cudaGetLastError();
        return LIA_ERR_LAUNCH;
    }
    return cudaGetLastError() == cudaSuccess ? LIA_OK : LIA_ERR_LAUNCH;
}

// Row of the paged cache [pages * page_size] that holds position `key` of a request whose block-table row is
// `table`; -1, with error flag 2 raised, when the table names no page of the pool there (the caller then reads
// zeros in place of the key: never memory outside the pool, never what an earlier tile left behind).
// `page_shift` >= 0: page_size is that power of two.
__device__ __forceinline__ int cache_row_of(const int* __restrict__ table, int key, int page_size, int page_shift,
                                            int num_pages, int* __restrict__ error_flag) {
    const int block = page_shift >= 0 ? key >> page_shift : key / page_size;
    const int page = table[block];
    if (page < 0 || page >= num_pages) {
        if (error_flag) atomicExch(error_flag, 2);
        return -1;
    }
    return page * page_size + (key - block * page_size);
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads.  `scratch` holds 32 floats of shared memory.
// The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = (lane < warps) ? scratch[lane] : 0.f;
    total = warp_sum(total);
    return total;
}
