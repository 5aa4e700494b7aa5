/* Drop-in for the generated "syrk-interface.h" of the PEPPERS BLAS layer
 * (t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:12; specification
 * t2s/tests/performance/syrk/syrk.cpp:52-73): A(K, N), symmetric C(N, N) and the folded 6-D output
 * (III, III, II, II, I+1, I) the design's deserializer fills. The extents of the output buffer carry
 * every tile constant, so the symbol needs no design header; it is defined by
 * t2sp_b200/csrc/stubs/syrk-interface.cpp. */
#ifndef T2SP_B200_SYRK_INTERFACE_H
#define T2SP_B200_SYRK_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int syrk(int32_t _OpA, float _Alpha, float _Beta, struct halide_buffer_t *_A_buffer, struct halide_buffer_t *_C_buffer,
         struct halide_buffer_t *_deserializer_buffer);
#ifdef __cplusplus
}
#endif
#endif
