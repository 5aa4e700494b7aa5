/* Drop-in for the "host.h" emitted by t2s/tests/correctness/aot/gemm-generate.cpp:176
 * (`compile_to_host("host", {a, b}, "GEMM", ...)`) and included by aot/gemm-run.cpp:20.
 * The symbol is defined by t2sp_b200/csrc/stubs/host.cpp. */
#ifndef T2SP_B200_AOT_HOST_H
#define T2SP_B200_AOT_HOST_H
#include "t2sp_b200/driver_prelude.h"
#ifdef __cplusplus
extern "C" {
#endif
int GEMM(struct halide_buffer_t *_a_buffer, struct halide_buffer_t *_b_buffer, struct halide_buffer_t *_unloader_buffer);
#ifdef __cplusplus
}
#endif
#endif
