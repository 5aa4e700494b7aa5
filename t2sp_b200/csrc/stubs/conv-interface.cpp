// Per-design stub for the 2-D convolution: compile with the design's const-parameters.h
// (t2s/tests/performance/conv/const-parameters.h:22-83) and -DTINY / -DS10 / -DGPU.
#include "conv-interface.h"

#include "const-parameters.h"

// Filled positionally because the field names coincide with the design's macro names:
// {layout, CI, CO, KY, KX, OY, OX, COOO, YYY, XXX, COO, YY, XX, Y, X, precision}.
extern "C" int conv(struct halide_buffer_t* I, struct halide_buffer_t* K, struct halide_buffer_t* O) {
#ifdef GPU
    // plain O(co + CO*n, oy + OY*ox) (conv.cpp:54)
    const t2sp_conv_desc d = {0, TOTAL_CI, TOTAL_CO, KY, KX, TOTAL_OY, TOTAL_OX, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#else
    // o(COOO,YYY,XXX,COO,YY,XX,Y,X,CO,N) (conv-run-fpga.cpp:68)
    const t2sp_conv_desc d = {1, TOTAL_CI, TOTAL_CO, KY, KX, TOTAL_OY, TOTAL_OX, COOO, YYY, XXX, COO, YY, XX, Y, X, 0};
#endif
    return t2sp_b200_conv(I, K, O, &d);
}
