/* Drop-in for the "conv-interface.h" that T2SP generates for its conv design
 * (declaration form: t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:8-19; call
 * site: t2s/tests/performance/conv/conv-run-fpga.cpp). Like the generated header it brings the
 * Halide buffer ABI and the C headers the host drivers rely on
 * (t2s/src/AOT-OpenCL-Runtime.h:21-30 in the reference). The symbol is defined by
 * t2sp_b200/csrc/stubs/conv-interface.cpp, compiled against the design's const-parameters.h. */
#ifndef T2SP_B200_CONV_INTERFACE_H
#define T2SP_B200_CONV_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int conv(struct halide_buffer_t *_I_buffer, struct halide_buffer_t *_K_buffer, struct halide_buffer_t *_O_buffer);
#ifdef __cplusplus
}
#endif
#endif
