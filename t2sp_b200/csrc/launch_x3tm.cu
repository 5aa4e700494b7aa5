// fp32 CTA-pair kernel with A in tensor memory and bf16 cross terms: instantiations and launch table.
#include "umma_core.cuh"
#include "umma_x3tm.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

namespace {
template <int OP, int STAGES, bool BPRE>
cudaError_t launch_x3tm(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = X3TmCfg<OP, STAGES>;
    auto kern = umma_x3tm_kernel<OP, STAGES, BPRE>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}
}  // namespace

cudaError_t x3tm_launch(int op, const CoreParams& p, int grid, cudaStream_t stream) {
    switch (op) {
        case OP_GEMM: return p.b_pre ? launch_x3tm<OP_GEMM, 4, true>(p, grid, stream) : launch_x3tm<OP_GEMM, 4, false>(p, grid, stream);
        case OP_TTM: return p.b_pre ? launch_x3tm<OP_TTM, 4, true>(p, grid, stream) : launch_x3tm<OP_TTM, 4, false>(p, grid, stream);
        case OP_CONV: return p.b_pre ? launch_x3tm<OP_CONV, 4, true>(p, grid, stream) : launch_x3tm<OP_CONV, 4, false>(p, grid, stream);
        case OP_CAPSULE: return p.b_pre ? cudaErrorInvalidValue : launch_x3tm<OP_CAPSULE, 4, false>(p, grid, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace t2sp
