/* Drop-in for the "conv.generated_oneapi_header.h" that T2SP's oneAPI back end emits
 * (emitter t2s/src/CodeGen_OneAPI_Dev.cpp:3596-3618; call site
 * t2s/tests/performance/oneapi/src/oneapi-target-5-run.cpp:33,117):
 *
 *     double exec_time = conv(device_selector, i.raw_buffer(), k.raw_buffer(), o.raw_buffer());
 *
 * Operands in the oneAPI flow's N-D layouts: I(IY, IX, CI, N), K(KY, KX, CI, CO), the 10-D tiled O
 * (oneapi-target-5-conv.cpp:58-62). The selector is ignored (the work runs on the calling thread's
 * CUDA device); the return value is the CUDA-event time of the contraction's kernels in nanoseconds,
 * or the negative halide error code. Header-only; link libt2sp_b200.so. */
#ifndef T2SP_B200_CONV_ONEAPI_HEADER_H
#define T2SP_B200_CONV_ONEAPI_HEADER_H
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
inline double conv(DeviceSelector &, struct halide_buffer_t *I, struct halide_buffer_t *K, struct halide_buffer_t *O) {
    const int rc = t2sp_b200_conv_nd(I, K, O, 0); /* every constant is read from the extents */
    return rc == 0 ? t2sp_b200_last_kernel_ns() : (double)rc;
}
#endif
