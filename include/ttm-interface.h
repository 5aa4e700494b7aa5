/* Host interface for the TTM design of t2s/tests/correctness/buffer/tmm_small.cpp (the reference
 * only realizes it through the JIT; this header gives it the same AOT calling form as the other
 * kernels). Output: 3-D c(I,J,K) or the 9-D device layout of tmm_small.cpp:116-129. */
#ifndef T2SP_B200_TTM_INTERFACE_H
#define T2SP_B200_TTM_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int ttm(struct halide_buffer_t *_a_buffer, struct halide_buffer_t *_b_buffer, struct halide_buffer_t *_c_buffer);
#ifdef __cplusplus
}
#endif
#endif
