/* What every generated "<k>-interface.h" gives a host driver besides the function itself:
 * the standard C headers and the Halide buffer structs (the reference's runtime header includes
 * them, t2s/src/AOT-OpenCL-Runtime.h:21-30,183-185, and the drivers use fabs, printf, assert
 * without including anything else first). */
#ifndef T2SP_B200_DRIVER_PRELUDE_H
#define T2SP_B200_DRIVER_PRELUDE_H
#include <assert.h>
#include <float.h>
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef __cplusplus
#include <iostream>
#endif
#include "t2sp_b200/runtime.h"
#endif
