// Single-CTA contraction kernel, fp32 data (3xTF32): instantiations and launch table.
#include "umma_core.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

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

// Raw-ring depth of the single-CTA fp32 kernels: what fits beside the lo ring, which holds B tiles only
// when the A operand lives in tensor memory.
constexpr int x3_stages(int op, int bn) {
    const bool a_tmem = bn <= T2SP_ATMEM_MAX_BN;
    if (op == OP_MTTKRP) return bn <= 64 ? (a_tmem ? 7 : 6) : (a_tmem ? 4 : 3);
    return bn <= 64 ? (a_tmem ? 6 : 5) : (a_tmem ? 4 : 3);
}

cudaError_t core_launch_x3(int arith, int op, int bn, const CoreParams& p, int grid, cudaStream_t stream) {
#define T2SP_CASE(AR, OPC, BNV, ST) \
    if (arith == AR && op == OPC && bn == BNV) return launch_one<AR, OPC, BNV, ST>(p, grid, stream)
    T2SP_CASE(AR_TF32X3, OP_GEMM, 128, x3_stages(OP_GEMM, 128));
    T2SP_CASE(AR_TF32X3, OP_GEMM, 64, x3_stages(OP_GEMM, 64));
    T2SP_CASE(AR_TF32X3, OP_TTM, 128, x3_stages(OP_TTM, 128));
    T2SP_CASE(AR_TF32X3, OP_TTM, 64, x3_stages(OP_TTM, 64));
    T2SP_CASE(AR_TF32X3, OP_CONV, 128, x3_stages(OP_CONV, 128));
    T2SP_CASE(AR_TF32X3, OP_CONV, 64, x3_stages(OP_CONV, 64));
    T2SP_CASE(AR_TF32X3, OP_CAPSULE, 128, x3_stages(OP_CAPSULE, 128));
    T2SP_CASE(AR_TF32X3, OP_CAPSULE, 64, x3_stages(OP_CAPSULE, 64));
    T2SP_CASE(AR_TF32X3, OP_MTTKRP, 64, x3_stages(OP_MTTKRP, 64));
    T2SP_CASE(AR_TF32X3, OP_MTTKRP, 128, x3_stages(OP_MTTKRP, 128));
#undef T2SP_CASE
    return cudaErrorInvalidValue;
}

}  // namespace t2sp
