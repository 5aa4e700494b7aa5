/* Drop-in for the PEPPERS BLAS header t2s/peppers/blas/level3/gemm/release/a10/blas-gemm.h:5:
 * the same C++ `sgemm` declaration, row-major arrays, C = alpha*op(A)*op(B) + beta*C. It is
 * defined by t2sp_b200/csrc/stubs/blas-gemm.cpp (the counterpart of the reference's
 * blas-gemm.cpp:11-49, which copies the arrays into Halide buffers around the generated gemm). */
#ifndef T2SP_B200_BLAS_GEMM_H
#define T2SP_B200_BLAS_GEMM_H
void sgemm(char transa, char transb, int m, int n, int k, float alpha, float *a, int lda, float *b, int ldb,
           float beta, float *c, int ldc);
#endif
