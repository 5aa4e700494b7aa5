// ttm(a, b, c) and mttkrp(a, b, c, d): these two need no design constants (every extent is
// carried by the buffers), so one stub serves all sizes.
#include "mttkrp-interface.h"
#include "ttm-interface.h"

extern "C" int ttm(struct halide_buffer_t* a, struct halide_buffer_t* b, struct halide_buffer_t* c) {
    return t2sp_b200_ttm(a, b, c, 0);
}

extern "C" int mttkrp(struct halide_buffer_t* a, struct halide_buffer_t* b, struct halide_buffer_t* c,
                      struct halide_buffer_t* d) {
    return t2sp_b200_mttkrp(a, b, c, d, 0);
}
