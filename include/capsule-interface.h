/* Drop-in for the "capsule-interface.h" that T2SP generates for its capsule design
 * (declaration form: t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:8-19; call
 * site: t2s/tests/performance/capsule/capsule-run-fpga.cpp). Like the generated header it brings the
 * Halide buffer ABI and the C headers the host drivers rely on
 * (t2s/src/AOT-OpenCL-Runtime.h:21-30 in the reference). The symbol is defined by
 * t2sp_b200/csrc/stubs/capsule-interface.cpp, compiled against the design's const-parameters.h. */
#ifndef T2SP_B200_CAPSULE_INTERFACE_H
#define T2SP_B200_CAPSULE_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int capsule(struct halide_buffer_t *_P_buffer, struct halide_buffer_t *_W_buffer, struct halide_buffer_t *_V_buffer);
#ifdef __cplusplus
}
#endif
#endif
