// Library-wide entry points that belong to no kernel.
#include "tcgen05.cuh"

// Kernels launched by this library since it was loaded, counted at the launch sites (a kernel that runs
// again when a captured CUDA graph is replayed is not counted again: the caller multiplies).
LIA_EXPORT long long lia_kernel_launches() { return lia_launch_counter.load(std::memory_order_relaxed); }

// Programmatic dependent launch on (1, the default) or off (0) for every later launch of this library.
LIA_EXPORT int lia_set_pdl(int enabled) {
    lia_pdl_enabled.store(enabled ? 1 : 0, std::memory_order_relaxed);
    return LIA_OK;
}

// The bounded wait of the tensor-core kernels, alone: one thread waits on an mbarrier at which nobody ever
// arrives, gives up after `polls` polls, raises error flag 3 as those kernels do, and returns.  It shows that a
// wait that runs out leaves the context usable and is reported; it is not on any forward path.
namespace {
__global__ void wait_probe_kernel(uint32_t polls, int* __restrict__ error_flag, int* __restrict__ gave_up) {
    __shared__ __align__(8) uint64_t barrier;
    const uint32_t bar = tc5::smem_u32(&barrier);
    tc5::mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!tc5::mbar_wait_limited(bar, 0, polls)) {
        if (error_flag) atomicExch(error_flag, 3);
        if (gave_up) *gave_up = 1;
    }
}
}  // namespace

LIA_EXPORT int lia_wait_probe(int polls, int* error_flag, int* gave_up, cudaStream_t stream) {
    if (polls <= 0 || polls > (1 << 16)) return LIA_ERR_SIZE;          // a few thousand polls: milliseconds at most
    wait_probe_kernel<<<1, 1, 0, stream>>>((uint32_t)polls, error_flag, gave_up);
    return lia_check_launch();
}
