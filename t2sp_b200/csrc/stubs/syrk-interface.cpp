// Stub for the generated syrk-interface.cpp (t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.cpp:26):
// the folded output buffer carries III, II and I in its extents, so nothing is baked in here.
#include "syrk-interface.h"

extern "C" int syrk(int32_t OpA, float Alpha, float Beta, struct halide_buffer_t* A, struct halide_buffer_t* C,
                    struct halide_buffer_t* deserializer) {
    return t2sp_b200_syrk(OpA, Alpha, Beta, A, C, deserializer);
}
