/* Design constants of a made-up "test design" used only to compile the per-design stubs in
 * the CPU test-suite (tests/test_abi_symbols.py). One file serves the GEMM, conv and capsule
 * stubs; the values are this repository's own, not those of any reference design. */
#ifndef T2SP_B200_TEST_DESIGN_H
#define T2SP_B200_TEST_DESIGN_H
#define KKK 2
#define JJJ 2
#define III 2
#define JJ 3
#define II 3
#define KK 2
#define KY 3
#define KX 3
#define CII 8
#define CI 2
#define COOO 4
#define COO 2
#define CO 2
#define YYY 2
#define XXX 2
#define YY 2
#define XX 1
#define Y 1
#define X 2
#define TOTAL_OX (XXX * XX * X)
#define TOTAL_OY (YYY * YY * Y)
#define TOTAL_CO (COOO * COO * CO)
#define TOTAL_CI (CII * CI)
#define OX 5
#define OY 5
#define MY 4
#define MX 4
#define MK 4
#define YYY_XXX 5
#define YY_XX 5
#define Y_X 1
#define NN 2
#endif
