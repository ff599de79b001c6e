// Library-wide entry points that belong to no kernel.
#include "common.cuh"

// Kernels launched by this library since it was loaded, counted at the launch sites (a kernel that runs
// again when a captured CUDA graph is replayed is not counted again: the caller multiplies).
LIA_EXPORT long long lia_kernel_launches() { return lia_launch_counter.load(std::memory_order_relaxed); }

// Programmatic dependent launch on (1, the default) or off (0) for every later launch of this library.
LIA_EXPORT int lia_set_pdl(int enabled) {
    lia_pdl_enabled.store(enabled ? 1 : 0, std::memory_order_relaxed);
    return LIA_OK;
}
