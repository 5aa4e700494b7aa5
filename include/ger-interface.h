/* Drop-in for the generated "ger-interface.h" of the GER design
 * (t2s/tests/performance/ger/ger.cpp:112 compiles it; used by ger-run-fpga.cpp:19,66): A(TK, TI) with k
 * innermost, X(TI), Y(TK) and the tiled 6-D output (KKK, III, II, KK, K, I) the design's deserializer
 * fills with a(tk, ti) + x(ti) * y(tk). The extents of the output buffer carry every tile constant, so the
 * symbol needs no design header; it is defined by t2sp_b200/csrc/stubs/ger-interface.cpp. */
#ifndef T2SP_B200_GER_INTERFACE_H
#define T2SP_B200_GER_INTERFACE_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int ger(struct halide_buffer_t *_A_buffer, struct halide_buffer_t *_X_buffer, struct halide_buffer_t *_Y_buffer,
        struct halide_buffer_t *_deserializer_buffer);
#ifdef __cplusplus
}
#endif
#endif
