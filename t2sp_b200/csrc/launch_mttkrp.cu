// The accumulate-then-scale MTTKRP kernel: instantiation and launcher.
#include "umma_mttkrp.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

cudaError_t mttkrp2_launch(const CoreParams& p, int grid, cudaStream_t stream) {
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(umma_mttkrp2_kernel, Mttkrp2Cfg::kSmemBytes, configured)) return e;
    umma_mttkrp2_kernel<<<grid, Mttkrp2Cfg::kThreads, Mttkrp2Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace t2sp
