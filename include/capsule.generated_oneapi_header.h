/* Drop-in for the "capsule.generated_oneapi_header.h" that T2SP's oneAPI back end emits
 * (emitter t2s/src/CodeGen_OneAPI_Dev.cpp:3596-3618; call site
 * t2s/tests/performance/oneapi/src/oneapi-target-6-run.cpp:27,115):
 *
 *     double exec_time = capsule(device_selector, P.raw_buffer(), W.raw_buffer(), V.raw_buffer());
 *
 * Operands in the oneAPI flow's N-D layouts: P(MK, MX, CI, IY, IX, N), W(MY, MK, CI, CO, KY, KX), the 9-D tiled V
 * (oneapi-target-6-capsule.cpp:57-61). The selector is ignored (the work runs on the calling thread's
 * CUDA device); the return value is the CUDA-event time of the contraction's kernels in nanoseconds,
 * or the negative halide error code. Header-only; link libt2sp_b200.so. */
#ifndef T2SP_B200_CAPSULE_ONEAPI_HEADER_H
#define T2SP_B200_CAPSULE_ONEAPI_HEADER_H
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
inline double capsule(DeviceSelector &, struct halide_buffer_t *P, struct halide_buffer_t *W, struct halide_buffer_t *V) {
    const int rc = t2sp_b200_capsule_nd(P, W, V, 0); /* every constant is read from the extents */
    return rc == 0 ? t2sp_b200_last_kernel_ns() : (double)rc;
}
#endif
