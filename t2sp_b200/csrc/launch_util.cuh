// Shared by the translation units that instantiate and launch the contraction kernels.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace t2sp {

constexpr int kMaxDev = 64;

// Raises a kernel's dynamic shared-memory limit once per device. The flags are only a cache: two host
// threads that both find one clear both make the (idempotent) call; ordinals beyond the table make it
// every time.
template <class Kern>
cudaError_t allow_smem(Kern kern, int bytes, std::atomic<bool>* configured) {
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return e;
    const bool cached = dev >= 0 && dev < kMaxDev;
    if (cached && configured[dev].load(std::memory_order_acquire)) return cudaSuccess;
    if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) return e;
    if (cached) configured[dev].store(true, std::memory_order_release);
    return cudaSuccess;
}

}  // namespace t2sp
