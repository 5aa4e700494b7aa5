/* Stand-in for the CM samples' common/cm_rt_helpers.h as the reference's CM-flow drivers use it
 * (gemm-run-gpu-cm.cpp:29): cm_result_check(expression) stops the program on a non-zero result. */
#ifndef T2SP_B200_CM_RT_HELPERS_H
#define T2SP_B200_CM_RT_HELPERS_H
#include <stdio.h>
#include <stdlib.h>
#define cm_result_check(t2sp_expr)                                                                       \
    do {                                                                                                 \
        const int t2sp_result = (t2sp_expr);                                                             \
        if (t2sp_result != 0) {                                                                          \
            fprintf(stderr, "%s:%d: %s failed with %d\n", __FILE__, __LINE__, #t2sp_expr, t2sp_result);  \
            exit(1);                                                                                     \
        }                                                                                                \
    } while (0)
#endif
