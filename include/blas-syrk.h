/* Drop-in for the PEPPERS BLAS header t2s/peppers/blas/level3/syrk/release/s10/blas-syrk.h:5: the
 * same C++ `ssyrk` declaration, row-major arrays. Defined by t2sp_b200/csrc/stubs/blas-syrk.cpp, the
 * counterpart of the reference's blas-syrk.cpp:13-86 (Halide buffers around the generated syrk, then
 * the folded output is spread over both triangles of c). */
#ifndef T2SP_B200_BLAS_SYRK_H
#define T2SP_B200_BLAS_SYRK_H
void ssyrk(char uplo, char transa, int n, int k, float alpha, float *a, int lda, float beta, float *c, int ldc);
#endif
