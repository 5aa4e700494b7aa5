// fp32 CTA-pair kernel with A in tensor memory and bf16 cross terms: instantiations and launch table.
#include "umma_core.cuh"
#include "umma_x3tm.cuh"
#include "launch_util.cuh"
#include "umma_launch.h"

namespace t2sp {

namespace {
template <int OP, int UN, bool ONE_CHUNK = false>
cudaError_t launch_x3tm(const CoreParams& p, int grid, cudaStream_t stream) {
    using Cfg = X3TmCfg<OP, UN>;
    auto kern = umma_x3tm_kernel<OP, UN, ONE_CHUNK>;
    static std::atomic<bool> configured[kMaxDev];
    if (cudaError_t e = allow_smem(kern, Cfg::kSmemBytes, configured)) return e;
    // programmatic stream serialization: the grid is set up while the pre-pass that writes B's images still runs; the
    // kernel's producer waits for that grid before its first copy of B, everything before that overlaps
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(Cfg::kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, p);
}
}  // namespace

cudaError_t x3tm_launch(int op, int un, const CoreParams& p, int grid, cudaStream_t stream) {
    if (!p.b_pre || !p.b_images) return cudaErrorInvalidValue;
    // short contractions on the 256-column form: every tile is a single chunk of the accumulator
    if (un == 256 && p.num_kb <= X3TmCfg<OP_GEMM, 256>::kChunkKb) {
        if (op == OP_GEMM) return launch_x3tm<OP_GEMM, 256, true>(p, grid, stream);
        if (op == OP_TTM) return launch_x3tm<OP_TTM, 256, true>(p, grid, stream);
    }
#define T2SP_X3TM(OPC, UNV) \
    if (op == OPC && un == UNV) return launch_x3tm<OPC, UNV>(p, grid, stream)
    T2SP_X3TM(OP_GEMM, 256);
    T2SP_X3TM(OP_GEMM, 128);
    T2SP_X3TM(OP_TTM, 256);
    T2SP_X3TM(OP_TTM, 128);
    T2SP_X3TM(OP_CONV, 256);
    T2SP_X3TM(OP_CONV, 128);
    T2SP_X3TM(OP_CAPSULE, 256);
    T2SP_X3TM(OP_CAPSULE, 128);
#undef T2SP_X3TM
    return cudaErrorInvalidValue;
}

}  // namespace t2sp
