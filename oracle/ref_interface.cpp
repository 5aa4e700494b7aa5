// TEST INFRASTRUCTURE ONLY: exposes the CPU oracle under the symbols of the reference's
// generated host interface (gemm / conv / capsule / GEMM), so that the reference's own,
// unmodified host drivers (t2s/tests/performance/*/*-run-fpga.cpp with -DTINY,
// t2s/tests/correctness/aot/gemm-run.cpp) can be linked against it and their in-driver golden
// loops validate the oracle and its tiled output layouts. Built per kernel with
// -DREF_GEMM / -DREF_AOT_GEMM / -DREF_CONV / -DREF_CAPSULE / -DREF_SYRK / -DREF_GER / -DREF_ONEAPI_CONV /
// -DREF_ONEAPI_CAPSULE and the design's include path.
// Never part of libt2sp_b200.so.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "t2sp_b200/abi.h"

extern "C" {
void oracle_gemm_f32(const float*, const float*, float*, int, int, int, int);
void oracle_gemm_tile_layout(const float*, float*, int, int, int, int, int, int);
void oracle_conv_f32(const float*, const float*, float*, int, int, int, int, int, int, int, int, int);
void oracle_conv_tile_layout(const float*, float*, int, int, int, int, int, int, int, int, int, int);
void oracle_capsule_f32(const float*, const float*, float*, int, int, int, int, int, int, int, int, int, int, int, int,
                        int, int);
void oracle_capsule_tile_layout(const float*, float*, int, int, int, int, int, int, int, int, int, int, int, int);
void oracle_syrk_f32(const float*, const float*, float*, int, int, int, int, int, int, float, float, int);
void oracle_ger_f32(const float*, const float*, const float*, float*, int, int, int, int, int, int, int);
void oracle_conv_nd_to_2d(const float*, const float*, float*, float*, int, int, int, int, int, int, int);
void oracle_capsule_nd_to_2d(const float*, const float*, float*, float*, int, int, int, int, int, int, int, int, int, int);
}

#if defined(REF_GEMM) || defined(REF_AOT_GEMM)
#ifdef REF_GEMM
#include "const-parameters.h"
#define REF_NAME gemm
#else
#define III 2
#define JJJ 4
#define II 4
#define JJ 4
#define REF_NAME GEMM
#endif
extern "C" int REF_NAME(halide_buffer_t* A, halide_buffer_t* B, halide_buffer_t* C) {
    const int K = A->dim[0].extent, M = A->dim[1].extent, N = B->dim[0].extent;
    std::vector<float> plain(size_t(M) * N);
    oracle_gemm_f32(reinterpret_cast<const float*>(A->host), reinterpret_cast<const float*>(B->host), plain.data(), M,
                    N, K, 0);
    oracle_gemm_tile_layout(plain.data(), reinterpret_cast<float*>(C->host), JJJ, III, JJ, II, N / (JJJ * JJ),
                            M / (III * II));
    return 0;
}
#endif

#ifdef REF_CONV
#include "const-parameters.h"
extern "C" int conv(halide_buffer_t* I, halide_buffer_t* K, halide_buffer_t* O) {
    const int N = I->dim[0].extent / (TOTAL_CI);
    std::vector<float> plain(size_t(TOTAL_CO) * N * (TOTAL_OY) * (TOTAL_OX));
    oracle_conv_f32(reinterpret_cast<const float*>(I->host), reinterpret_cast<const float*>(K->host), plain.data(), N,
                    TOTAL_CI, TOTAL_CO, KY, KX, TOTAL_OY, TOTAL_OX, CII, 0);
    oracle_conv_tile_layout(plain.data(), reinterpret_cast<float*>(O->host), N, COOO, YYY, XXX, COO, YY, XX, Y, X, CO);
    return 0;
}
#endif

#ifdef REF_CAPSULE
#include "const-parameters.h"
extern "C" int capsule(halide_buffer_t* P, halide_buffer_t* W, halide_buffer_t* V) {
    const int N = P->dim[1].extent / ((TOTAL_IY) * (TOTAL_IX));
    std::vector<float> plain(size_t(TOTAL_CO) * MY * MX * NN * OY * OX * N);
    oracle_capsule_f32(reinterpret_cast<const float*>(P->host), reinterpret_cast<const float*>(W->host), plain.data(),
                       N, NN, TOTAL_CI, CII, TOTAL_CO, KY, KX, OY, OX, MY, MX, MK, 2, 0);
    oracle_capsule_tile_layout(plain.data(), reinterpret_cast<float*>(V->host), N, NN, COOO, COO, CO, YYY_XXX, YY_XX,
                               Y_X, MY, MX, OY, OX);
    return 0;
}
#endif

#ifdef REF_SYRK
// the generated syrk(OpA, Alpha, Beta, A, C, deserializer) of t2s/tests/performance/syrk/syrk.cpp
extern "C" int syrk(int32_t, float alpha, float beta, halide_buffer_t* A, halide_buffer_t* C, halide_buffer_t* O) {
    oracle_syrk_f32(reinterpret_cast<const float*>(A->host), reinterpret_cast<const float*>(C->host),
                    reinterpret_cast<float*>(O->host), A->dim[0].extent, O->dim[0].extent, O->dim[2].extent,
                    O->dim[4].extent - 1, O->dim[5].extent, C->dim[1].stride, alpha, beta, 0);
    return 0;
}
#endif

#ifdef REF_GER
// the generated ger(A, X, Y, deserializer) of t2s/tests/performance/ger/ger.cpp
extern "C" int ger(halide_buffer_t* A, halide_buffer_t* X, halide_buffer_t* Y, halide_buffer_t* O) {
    oracle_ger_f32(reinterpret_cast<const float*>(A->host), reinterpret_cast<const float*>(X->host),
                   reinterpret_cast<const float*>(Y->host), reinterpret_cast<float*>(O->host), O->dim[0].extent,
                   O->dim[1].extent, O->dim[2].extent, O->dim[3].extent, O->dim[4].extent, O->dim[5].extent,
                   A->dim[1].stride);
    return 0;
}
#endif

#ifdef REF_ONEAPI_CONV
extern "C" int oracle_pin_conv_nd(halide_buffer_t* I, halide_buffer_t* K, halide_buffer_t* O) {
    const int IY = I->dim[0].extent, IX = I->dim[1].extent, CI = I->dim[2].extent, N = I->dim[3].extent;
    const int KY = K->dim[0].extent, KX = K->dim[1].extent, CO = K->dim[3].extent;
    const int OY = IY - KY + 1, OX = IX - KX + 1;
    std::vector<float> i2(size_t(CI) * N * IY * IX), k2(size_t(CO) * KX * CI * KY), plain(size_t(CO) * N * OY * OX);
    oracle_conv_nd_to_2d(reinterpret_cast<const float*>(I->host), reinterpret_cast<const float*>(K->host), i2.data(),
                         k2.data(), N, CI, CO, KY, KX, IY, IX);
    oracle_conv_f32(i2.data(), k2.data(), plain.data(), N, CI, CO, KY, KX, OY, OX, 0, 0);
    oracle_conv_tile_layout(plain.data(), reinterpret_cast<float*>(O->host), N, O->dim[0].extent, O->dim[1].extent,
                            O->dim[2].extent, O->dim[3].extent, O->dim[4].extent, O->dim[5].extent, O->dim[6].extent,
                            O->dim[7].extent, O->dim[8].extent);
    return 0;
}
#endif

#ifdef REF_ONEAPI_CAPSULE
extern "C" int oracle_pin_capsule_nd(halide_buffer_t* P, halide_buffer_t* W, halide_buffer_t* V) {
    const int MK = P->dim[0].extent, MX = P->dim[1].extent, CI = P->dim[2].extent, IY = P->dim[3].extent,
              IX = P->dim[4].extent, N = P->dim[5].extent;
    const int MY = W->dim[0].extent, CO = W->dim[3].extent, KY = W->dim[4].extent, KX = W->dim[5].extent;
    const int s = 2, OY = (IY - KY + s) / s, OX = (IX - KX + s) / s;  // the reference's stride (capsule.cpp:40-41)
    std::vector<float> p2(size_t(CI) * MK * MX * IY * IX * N), w2(size_t(CO) * MY * CI * KY * KX * MK),
        plain(size_t(CO) * MY * MX * OY * OX * N);
    oracle_capsule_nd_to_2d(reinterpret_cast<const float*>(P->host), reinterpret_cast<const float*>(W->host), p2.data(),
                            w2.data(), N, CI, CO, KY, KX, IY, IX, MY, MX, MK);
    oracle_capsule_f32(p2.data(), w2.data(), plain.data(), N, 1, CI, CI, CO, KY, KX, OY, OX, MY, MX, MK, s, 0);
    oracle_capsule_tile_layout(plain.data(), reinterpret_cast<float*>(V->host), N, 1, V->dim[0].extent, V->dim[6].extent,
                               V->dim[7].extent, V->dim[1].extent, V->dim[2].extent, V->dim[3].extent, MY, MX, OY, OX);
    return 0;
}
#endif
