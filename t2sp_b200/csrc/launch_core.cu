// Single-CTA contraction kernel, 16-bit and 8-bit arithmetics: instantiations and launch table.
#include "umma_core.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

cudaError_t core_launch_x3(int arith, int op, int bn, const CoreParams& p, int grid, cudaStream_t stream);

namespace {
template <int ARITH, int OP, int BN, int STAGES>
cudaError_t launch_one(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = CoreCfg<ARITH, OP, BN, STAGES>;
    auto kern = umma_contract_kernel<ARITH, OP, BN, STAGES>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}
}  // namespace

cudaError_t core_launch(int arith, int op, int bn, const CoreParams& p, int grid, cudaStream_t stream) {
#define T2SP_CASE(AR, OPC, BNV, ST) \
    if (arith == AR && op == OPC && bn == BNV) return launch_one<AR, OPC, BNV, ST>(p, grid, stream)
    T2SP_CASE(AR_F16, OP_GEMM, 256, 4);
    T2SP_CASE(AR_F16, OP_GEMM, 128, 6);
    T2SP_CASE(AR_F16, OP_TTM, 256, 4);
    T2SP_CASE(AR_F16, OP_TTM, 128, 6);
    T2SP_CASE(AR_I8, OP_GEMM, 256, 4);
    T2SP_CASE(AR_I8, OP_GEMM, 128, 6);
    T2SP_CASE(AR_I8, OP_TTM, 256, 4);
    T2SP_CASE(AR_I8, OP_TTM, 128, 6);
#undef T2SP_CASE
    return core_launch_x3(arith, op, bn, p, grid, stream);
}

}  // namespace t2sp
