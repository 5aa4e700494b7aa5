// CTA-pair 3xTF32 kernel (fp32 data): instantiations and launch table.
#include "umma_core.cuh"
#include "umma_x3pair.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

namespace {
template <int OP, int UN, int STAGES, int LOSLOTS>
cudaError_t launch_x3pair(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = X3PairCfg<OP, UN, STAGES, LOSLOTS>;
    auto kern = umma_x3pair_kernel<OP, UN, STAGES, LOSLOTS>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}
}  // namespace

cudaError_t x3pair_launch(int op, int un, const CoreParams& p, int grid, cudaStream_t stream) {
#define T2SP_X3(OPC, UNV, ST, LO) \
    if (op == OPC && un == UNV) return launch_x3pair<OPC, UNV, ST, LO>(p, grid, stream)
    T2SP_X3(OP_GEMM, 256, 3, 3);
    T2SP_X3(OP_GEMM, 128, 5, 3);
    T2SP_X3(OP_TTM, 256, 3, 3);
    T2SP_X3(OP_TTM, 128, 5, 3);
    T2SP_X3(OP_CONV, 256, 3, 3);
    T2SP_X3(OP_CONV, 128, 5, 3);
    T2SP_X3(OP_CAPSULE, 256, 3, 3);
    T2SP_X3(OP_CAPSULE, 128, 5, 3);
#undef T2SP_X3
    return cudaErrorInvalidValue;
}

}  // namespace t2sp
