// Per-design stub: the counterpart of the generated gemm-interface.cpp. Compile it with the
// include path and the -DTINY / -DS10 / -DGPU flag of the design, exactly as the reference
// compiles its specification (t2s/tests/performance/test-common-funcs.sh:27), so that the inner
// tile extents of const-parameters.h (t2s/tests/performance/gemm/const-parameters.h:24-51) are
// baked in; outer extents come from the buffers (gemm.cpp:44-46).
#include "gemm-interface.h"

#include "const-parameters.h"

// The descriptor's field names coincide with the design's macro names, so it is filled
// positionally: {layout, JJJ, III, JJ, II, precision, trans_b}.
extern "C" int gemm(struct halide_buffer_t* A, struct halide_buffer_t* B, struct halide_buffer_t* C) {
#ifdef GPU
    const t2sp_gemm_desc d = {0, 0, 0, 0, 0, 0, 0};  // the GPU flow realizes a plain 2-D C(total_j, total_i) (gemm.cpp:89)
#else
    const t2sp_gemm_desc d = {1, JJJ, III, JJ, II, 0, 0};  // the FPGA flow realizes c(JJJ,III,JJ,II,J,I) (gemm-run-fpga.cpp:69)
#endif
    return t2sp_b200_gemm(A, B, C, &d);
}
