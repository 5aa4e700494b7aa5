// MTTKRP for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc while they run: a service whose memory
// pool was carved up at start-up and that treats any later driver allocation as a fault, a
// real-time loop in which the implicit device synchronisation of cudaMalloc/cudaFree is not
// acceptable, or code running under a framework allocator that owns all of HBM. The regular
// t2sp_b200_mttkrp entry takes its split-K partial sums from the library's caching allocator
// and may stage host buffers on the device; this variant does neither. Inputs and output
// are device pointers supplied by the caller, and the partial sums live in a fixed array
// that is part of the loaded module.
//
// Consequences the caller has to know about:
//  * the array is T2SP_B200_NOALLOC_SCRATCH_BYTES (16 MiB) on every GPU that loads the library,
//    held until the process exits; a problem whose single partial slab (4*I*R bytes) does not
//    fit is rejected, and fewer splits are used when the preferred number does not fit;
//  * all calls on a device share the array and it keeps whatever the last call left in it.
//    Nothing needs clearing: every split overwrites its whole I x R slab before the reduction
//    reads it. Two calls that overlap on the GPU (different streams, or sync == 0 from two
//    threads) race on it and corrupt each other's result;
//  * the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) and sizes the kernel's shared memory; make that first call
//    outside any stream capture.
#include <cudaTypedefs.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "t2sp_b200/runtime.h"
#include "umma_launch.h"

namespace t2sp {
void mttkrp_plan(int L, int I, int Kd, int want_splits, int* splits, int* num_kb);
}

namespace {

constexpr size_t kScratchBytes = T2SP_B200_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDev = 16;

// Split-K partial sums, [split][r][i]. In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float g_noalloc_partials[kScratchBytes / sizeof(float)];
// Raised by a kernel whose bounded wait ran out (same bits as the regular path's status word).
static __device__ __align__(256) unsigned g_noalloc_status[64];

std::mutex g_setup_mu;
float* g_partials_addr[kMaxDev] = {};
unsigned* g_status_addr[kMaxDev] = {};
PFN_cuTensorMapEncodeTiled_v12000 g_encode_fn = nullptr;

int fail(int code, const char* msg) {
    fprintf(stderr, "t2sp_b200_mttkrp_noalloc: %s\n", msg);
    return code;
}

// One-time set-up per device, with that device current.
int setup_device(int dev) {
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_partials_addr[dev]) return 0;
    if (!g_encode_fn) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
            return fail(halide_error_code_device_interface_no_device, "the CUDA driver lacks cuTensorMapEncodeTiled");
        g_encode_fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    float* parts = nullptr;
    unsigned* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&parts), g_noalloc_partials);
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: cudaGetSymbolAddress(partials) failed: %s\n", cudaGetErrorString(e));
        return halide_error_code_device_interface_no_device;
    }
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_noalloc_status);
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: cudaGetSymbolAddress(status) failed: %s\n", cudaGetErrorString(e));
        return halide_error_code_device_interface_no_device;
    }
    g_status_addr[dev] = status;
    g_partials_addr[dev] = parts;
    return 0;
}

}  // namespace

extern "C" int t2sp_b200_mttkrp_noalloc(const float* a, int64_t a_stride_i, int64_t a_stride_k, const float* b,
                                        int64_t b_stride_r, const float* c, int64_t c_stride_r, float* d,
                                        int64_t d_stride_r, int32_t L, int32_t I, int32_t K, int32_t R,
                                        void* cuda_stream, int32_t sync) {
    using namespace t2sp;
    if (!a || !b || !c || !d) return fail(halide_error_code_buffer_argument_is_null, "a, b, c and d must be device pointers");
    if (L <= 0 || I <= 0 || K <= 0 || R <= 0) return fail(halide_error_code_buffer_extents_negative, "L, I, K and R must be positive");
    if (R > 128) return fail(halide_error_code_constraint_violated, "R (columns of the factor matrices) must be at most 128");
    if (a_stride_i < L || a_stride_k < a_stride_i * I || b_stride_r < K || c_stride_r < L || d_stride_r < I)
        return fail(halide_error_code_constraint_violated, "strides are smaller than the extents they span");
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (a_stride_i * 4) % 16 || (a_stride_k * 4) % 16)
        return fail(halide_error_code_constraint_violated, "a must be 16-byte aligned with strides that are multiples of 4 elements");
    const size_t slab = size_t(I) * size_t(R) * sizeof(float);
    if (slab > kScratchBytes) {
        fprintf(stderr,
                "t2sp_b200_mttkrp_noalloc: one partial slab needs 4*I*R = %zu bytes but the built-in scratch array holds "
                "%zu; use t2sp_b200_mttkrp for this size\n",
                slab, kScratchBytes);
        return halide_error_code_buffer_allocation_too_large;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev)
        return fail(halide_error_code_device_interface_no_device, "no current CUDA device");
    if (int e = setup_device(dev)) return e;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);

    int splits = 0, num_kb = 0;
    mttkrp_plan(L, I, K, 0, &splits, &num_kb);
    const int fit = static_cast<int>(kScratchBytes / slab);
    if (splits > fit) mttkrp_plan(L, I, K, fit, &splits, &num_kb);

    const int bn = core_pick_bn(AR_TF32X3, OP_MTTKRP, R);
    CoreParams p;
    memset(&p, 0, sizeof(p));
    {
        cuuint64_t gdim[3] = {cuuint64_t(L), cuuint64_t(I), cuuint64_t(K)};
        cuuint64_t gstr[2] = {cuuint64_t(a_stride_i) * 4, cuuint64_t(a_stride_k) * 4};
        cuuint32_t box[3] = {32, cuuint32_t(kBlockM), 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (g_encode_fn(&p.mapA[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(a), gdim, gstr, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return fail(halide_error_code_constraint_violated, "the tensor `a` cannot be described to TMA (alignment or size)");
    }
    {
        cuuint64_t gdim[2] = {cuuint64_t(L), cuuint64_t(R)};
        cuuint64_t gstr[1] = {cuuint64_t(c_stride_r) * 4};
        cuuint32_t box[2] = {32, cuuint32_t(bn)};
        cuuint32_t estr[2] = {1, 1};
        if ((reinterpret_cast<uintptr_t>(c) & 15) || (c_stride_r * 4) % 16 ||
            g_encode_fn(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(c), gdim, gstr, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return fail(halide_error_code_constraint_violated,
                        "the factor `c` cannot be described to TMA (16-byte aligned base, column stride a multiple of 4 elements)");
    }
    const int lblks = (L + 31) / 32;
    p.M = I; p.N = R; p.tile_rows = kBlockM; p.a_tx_bytes = kBlockM * 128;
    p.total_kb = lblks * K; p.num_kb = num_kb;
    p.tiles_m = (I + kBlockM - 1) / kBlockM; p.tiles_n = splits; p.splits = splits; p.lblks = lblks;
    p.idesc = make_instr_desc(1, 2, false, false, kBlockM, bn);
    p.epi = EPI_COLMAJOR; p.ldo = I;
    p.out = g_partials_addr[dev];
    p.fc = c; p.fb = b; p.ldfc = c_stride_r; p.ldfb = b_stride_r;
    p.L = L; p.Kdim = K; p.R = R;
    p.status = g_status_addr[dev];
    p.group_m = 16;

    const int tiles = p.tiles_m * p.tiles_n;
    const int sms = core_sm_count();
    cudaError_t e = core_launch(AR_TF32X3, OP_MTTKRP, bn, p, tiles < sms ? tiles : sms, stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: kernel launch failed: %s\n", cudaGetErrorString(e));
        return halide_error_code_device_run_failed;
    }
    const float* parts = g_partials_addr[dev];
    e = reduce_partials_launch(parts, d, I, R, d_stride_r, splits, stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: reduction launch failed: %s\n", cudaGetErrorString(e));
        return halide_error_code_device_run_failed;
    }
    if (!sync) return 0;
    unsigned status = 0;
    if (cudaStreamSynchronize(stream) != cudaSuccess ||
        cudaMemcpyFromSymbol(&status, g_noalloc_status, sizeof(unsigned)) != cudaSuccess) {
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: device execution failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return halide_error_code_device_run_failed;
    }
    if (status != 0) {
        const unsigned zero = 0;
        cudaMemcpyToSymbol(g_noalloc_status, &zero, sizeof(unsigned));
        fprintf(stderr, "t2sp_b200_mttkrp_noalloc: a kernel gave up waiting (status 0x%x)\n", status);
        return halide_error_code_device_run_failed;
    }
    return 0;
}
