/* Drop-in for the "gemm.generated_oneapi_header.h" that T2SP's oneAPI back end emits
 * (emitter t2s/src/CodeGen_OneAPI_Dev.cpp:3596-3618; call site
 * t2s/tests/performance/oneapi/src/oneapi-target-4-run.cpp:33,99):
 *
 *     double exec_time = gemm(device_selector, a.raw_buffer(), b.raw_buffer(), c.raw_buffer());
 *
 * Same buffers as the FPGA/AOT interface (A(K,I), B(J,K), 6-D tiled C), one extra leading
 * "device selector" argument, and the return value is the kernels' execution time in
 * nanoseconds. Here the selector is ignored (the work runs on the calling thread's CUDA device)
 * and the time is the CUDA-event time of the launch. On failure the negative halide error code
 * is returned instead of a time. Header-only; link libt2sp_b200.so.
 *
 * The run file names sycl::ext::intel::fpga_selector / fpga_emulator_selector; when no SYCL
 * headers are installed, empty stand-ins for those two types are declared below. */
#ifndef T2SP_B200_GEMM_ONEAPI_HEADER_H
#define T2SP_B200_GEMM_ONEAPI_HEADER_H
#include "t2sp_b200/driver_prelude.h"

#if defined(__has_include)
#if __has_include(<sycl/sycl.hpp>)
#include <sycl/sycl.hpp>
#include <sycl/ext/intel/fpga_extensions.hpp>
#define T2SP_B200_HAVE_SYCL 1
#endif
#endif
#if !defined(T2SP_B200_HAVE_SYCL) && !defined(T2SP_B200_SYCL_STANDINS)
#define T2SP_B200_SYCL_STANDINS 1
namespace sycl { namespace ext { namespace intel {
struct fpga_selector {};
struct fpga_emulator_selector {};
}}}
#endif

template <class DeviceSelector>
inline double gemm(DeviceSelector &, struct halide_buffer_t *A, struct halide_buffer_t *B, struct halide_buffer_t *C) {
    const int rc = t2sp_b200_gemm(A, B, C, 0); /* tile extents of the 6-D output are read from C itself */
    return rc == 0 ? t2sp_b200_last_kernel_ns() : (double)rc;
}
#endif
