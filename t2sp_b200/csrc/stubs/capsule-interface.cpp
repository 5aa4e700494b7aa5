// Per-design stub for the capsule convolution: compile with the design's const-parameters.h
// (t2s/tests/performance/capsule/const-parameters.h:22-78) and -DTINY / -DS10 / -DGPU.
// The reference fixes the spatial stride at 2 (capsule.cpp:40-41).
#include "capsule-interface.h"

#include "const-parameters.h"

// Filled positionally because the field names coincide with the design's macro names:
// {layout, CI, CII, CO, KY, KX, OY, OX, MY, MX, MK, NN, stride, COOO, YYY_XXX, YY_XX, Y_X, COO, precision}.
extern "C" int capsule(struct halide_buffer_t* P, struct halide_buffer_t* W, struct halide_buffer_t* V) {
#ifdef GPU
    // plain V(co + CO*my + CO*MY*mx + CO*MY*MX*nn, oy + OY*ox + OY*OX*n) (capsule.cpp:54)
    const t2sp_capsule_desc d = {0, TOTAL_CI, CII, TOTAL_CO, KY, KX, OY, OX, MY, MX, MK, NN, 2, 0, 0, 0, 0, 0, 0};
#else
    // V(COOO,YYY_XXX,YY_XX,Y_X,MY,MX,COO,NN,CO,N) (capsule-run-fpga.cpp:73)
    const t2sp_capsule_desc d = {1, TOTAL_CI, CII, TOTAL_CO, KY, KX, OY, OX, MY, MX, MK, NN, 2,
                                 COOO, YYY_XXX, YY_XX, Y_X, COO, 0};
#endif
    return t2sp_b200_capsule(P, W, V, &d);
}
