// sgemm(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc) of the PEPPERS BLAS layer
// (t2s/peppers/blas/level3/gemm/release/a10/blas-gemm.cpp:11-49). Needs no design constants: any
// m, n, k go straight to the library, which reads the caller's row-major arrays in place.
#include <stdio.h>

#include "t2sp_b200/runtime.h"

void sgemm(char transa, char transb, int m, int n, int k, float alpha, float* a, int lda, float* b, int ldb, float beta,
           float* c, int ldc) {
    const int rc = t2sp_b200_sgemm(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    if (rc != 0) fprintf(stderr, "sgemm: t2sp_b200_sgemm failed with halide error %d\n", rc);
}
