/* Host interface for MTTKRP in the argument order of the reference's golden helper
 * get_result_of_mttkrp(a, b, c) (t2s/tests/correctness/util/util.h:464-481), output last. */
#ifndef T2SP_B200_MTTKRP_INTERFACE_H
#define T2SP_B200_MTTKRP_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int mttkrp(struct halide_buffer_t *_a_buffer, struct halide_buffer_t *_b_buffer, struct halide_buffer_t *_c_buffer,
           struct halide_buffer_t *_d_buffer);
#ifdef __cplusplus
}
#endif
#endif
