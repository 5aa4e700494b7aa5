// ssyrk(uplo, trans, n, k, alpha, a, lda, beta, c, ldc) of the PEPPERS BLAS layer over the generated
// syrk interface (reference flow: t2s/peppers/blas/level3/syrk/release/s10/blas-syrk.cpp:13-86).
// Compile with the design's const-parameters.h on the include path: III and II are the design's
// tile extents, and n must be a multiple of 2 * III * II. Like the reference wrapper this one reads
// a as n rows of k values, treats c as symmetric (the triangle named by uplo is the one that is read)
// and leaves the whole updated matrix, both triangles, in c.
#include <stdio.h>
#include <string.h>

#include <vector>

#include "syrk-interface.h"

#include "const-parameters.h"  // after the interface: the design's macros (I, III, ...) are common identifiers

namespace {
struct Dims {
    halide_dimension_t d[6];
};
halide_buffer_t dense(float* host, Dims& dims, int nd, const int* ext) {
    halide_buffer_t b = {};
    b.host = reinterpret_cast<uint8_t*>(host);
    const uint32_t f32 = 2u | (32u << 8) | (1u << 16);  // halide_type_t{float, 32 bits, 1 lane}
    memcpy(&b.type, &f32, 4);
    b.dimensions = nd;
    b.dim = dims.d;
    int stride = 1;
    for (int i = 0; i < nd; ++i) {
        dims.d[i].min = 0; dims.d[i].extent = ext[i]; dims.d[i].stride = stride; dims.d[i].flags = 0;
        stride *= ext[i];
    }
    return b;
}
}  // namespace

void ssyrk(char uplo, char trans, int n, int k, float alpha, float* a, int lda, float beta, float* c, int ldc) {
    (void)lda; (void)ldc;
    const int tile = III * II;
    if (n <= 0 || n % (2 * tile)) {
        fprintf(stderr, "ssyrk: n = %d is not a multiple of 2*III*II = %d\n", n, 2 * tile);
        return;
    }
    const int blocks = n / tile;  // I of the design
    const bool upper = (uplo == 'U' || uplo == 'u');
    // full symmetric copy of c: element (row, col) comes from the stored triangle
    std::vector<float> full(size_t(n) * n);
    for (int r = 0; r < n; ++r)
        for (int col = 0; col < n; ++col) {
            const bool stored = upper ? (r <= col) : (r >= col);
            full[size_t(r) * n + col] = stored ? c[size_t(r) * n + col] : c[size_t(col) * n + r];
        }
    std::vector<float> folded(size_t(tile) * tile * (blocks + 1) * blocks);
    Dims da, dc, dout;
    const int ea[2] = {k, n}, ec[2] = {n, n}, eo[6] = {III, III, II, II, blocks + 1, blocks};
    halide_buffer_t A = dense(a, da, 2, ea), C = dense(full.data(), dc, 2, ec), O = dense(folded.data(), dout, 6, eo);
    const int opa = (trans == 'N' || trans == 'n') ? 0 : 1;
    const int rc = syrk(opa, alpha, beta, &A, &C, &O);
    if (rc != 0) {
        fprintf(stderr, "ssyrk: syrk failed with halide error %d\n", rc);
        return;
    }
    // Unfold: block row bi < blocks/2 of the upper triangle sits in row bi of the folded buffer at
    // column bj + 1; block row bi >= blocks/2 sits mirrored (every index reversed) in row blocks-1-bi.
    auto at = [&](int jjj, int iii, int jj, int ii, int j, int i) -> float {
        return folded[jjj + size_t(III) * (iii + size_t(III) * (jj + size_t(II) * (ii + size_t(II) * (j + size_t(blocks + 1) * i))))];
    };
    for (int r = 0; r < n; ++r)
        for (int col = r; col < n; ++col) {
            const int bi = r / tile, ii = (r % tile) / III, iii = r % III;
            const int bj = col / tile, jj = (col % tile) / III, jjj = col % III;
            const float v = (2 * bi < blocks) ? at(jjj, iii, jj, ii, bj + 1, bi)
                                              : at(III - 1 - jjj, III - 1 - iii, II - 1 - jj, II - 1 - ii, blocks - 1 - bj, blocks - 1 - bi);
            c[size_t(r) * n + col] = v;
            c[size_t(col) * n + r] = v;
        }
}
