// CTA-pair GEMM kernels for 16-bit and 8-bit operands (256 x 256 and 512 x 256 tiles): instantiations and launch tables.
#include "umma_core.cuh"
#include "umma_pair.cuh"
#include "umma_pair2.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

namespace {
template <int ARITH, int OP, int STAGES>
cudaError_t launch_pair(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = PairCfg<ARITH, OP, STAGES>;
    auto kern = umma_pair_kernel<ARITH, OP, STAGES>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

template <int ARITH, int OP, int STAGES>
cudaError_t launch_pair2(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = Pair2Cfg<ARITH, OP, STAGES>;
    auto kern = umma_pair2_kernel<ARITH, OP, STAGES>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}
}  // namespace

cudaError_t pair_launch(int arith, int op, const CoreParams& p, int grid, cudaStream_t stream) {
    if (arith == AR_F16 && op == OP_GEMM) return launch_pair<AR_F16, OP_GEMM, 6>(p, grid, stream);
    if (arith == AR_F16 && op == OP_TTM) return launch_pair<AR_F16, OP_TTM, 6>(p, grid, stream);
    if (arith == AR_I8 && op == OP_GEMM) return launch_pair<AR_I8, OP_GEMM, 6>(p, grid, stream);
    if (arith == AR_I8 && op == OP_TTM) return launch_pair<AR_I8, OP_TTM, 6>(p, grid, stream);
    return cudaErrorInvalidValue;
}

cudaError_t pair2_launch(int arith, int op, const CoreParams& p, int grid, cudaStream_t stream) {
    if (arith == AR_F16 && op == OP_GEMM) return launch_pair2<AR_F16, OP_GEMM, 4>(p, grid, stream);
    if (arith == AR_F16 && op == OP_TTM) return launch_pair2<AR_F16, OP_TTM, 4>(p, grid, stream);
    if (arith == AR_I8 && op == OP_GEMM) return launch_pair2<AR_I8, OP_GEMM, 4>(p, grid, stream);
    if (arith == AR_I8 && op == OP_TTM) return launch_pair2<AR_I8, OP_TTM, 4>(p, grid, stream);
    return cudaErrorInvalidValue;
}

}  // namespace t2sp
