// Stub for the AOT correctness test: GEMM(a, b, out) of t2s/tests/correctness/aot/gemm-generate.cpp
// with the constants that test fixes in both its generator and its runner
// (aot/gemm-run.cpp:35-43: II=JJ=4, III=2, JJJ=4).
#include "host.h"

extern "C" int GEMM(struct halide_buffer_t* a, struct halide_buffer_t* b, struct halide_buffer_t* out) {
    const t2sp_gemm_desc d = {1, /*JJJ*/ 4, /*III*/ 2, /*JJ*/ 4, /*II*/ 4, 0, 0};
    return t2sp_b200_gemm(a, b, out, &d);
}
