/* The argument type of every entry point: Halide's halide_buffer_t.
 *
 * Reference: Halide/src/runtime/HalideRuntime.h:1356-1420 (halide_buffer_t),
 * :1338-1353 (halide_dimension_t), :399-455 (halide_type_code_t / halide_type_t).
 * The generated host interfaces include a runtime header that carries these structs
 * (t2s/src/AOT-OpenCL-Runtime.h:183-185), so callers see them through "<k>-interface.h"
 * whichever of HalideBuffer.h and the interface header comes first.
 *
 * When the real HalideRuntime.h is on the include path it is used as is (its include
 * guard makes either include order work). Otherwise a minimal, layout-compatible
 * restatement is provided for plain C and FFI callers; sizes and offsets are asserted.
 */
#ifndef T2SP_B200_ABI_H
#define T2SP_B200_ABI_H

#include <stddef.h>
#include <stdint.h>

#if defined(__has_include)
#if __has_include("HalideRuntime.h")
#include "HalideRuntime.h"
#endif
#endif

#ifndef HALIDE_HALIDERUNTIME_H

#ifdef __cplusplus
extern "C" {
#endif

/* Type codes of halide_type_t::code. */
enum { halide_type_int = 0, halide_type_uint = 1, halide_type_float = 2, halide_type_handle = 3, halide_type_bfloat = 4 };

/* 4 bytes: element kind, bits per lane, lanes (always 1 here). */
struct halide_type_t {
    uint8_t code;
    uint8_t bits;
    uint16_t lanes;
};

/* 16 bytes: one dimension of a buffer; stride is in elements. */
typedef struct halide_dimension_t {
    int32_t min, extent, stride;
    uint32_t flags;
} halide_dimension_t;

struct halide_buffer_t;
struct halide_device_interface_impl_t;

/* 128 bytes: the table of device functions a buffer's `device_interface` points to
 * (HalideRuntime.h:713-738). Halide::Runtime::Buffer calls through it, e.g. device_free
 * in its destructor and copy_to_host (HalideBuffer.h:229-252,1615). */
struct halide_device_interface_t {
    int (*device_malloc)(void *user_context, struct halide_buffer_t *buf,
                         const struct halide_device_interface_t *device_interface);
    int (*device_free)(void *user_context, struct halide_buffer_t *buf);
    int (*device_sync)(void *user_context, struct halide_buffer_t *buf);
    void (*device_release)(void *user_context, const struct halide_device_interface_t *device_interface);
    int (*copy_to_host)(void *user_context, struct halide_buffer_t *buf);
    int (*copy_to_device)(void *user_context, struct halide_buffer_t *buf,
                          const struct halide_device_interface_t *device_interface);
    int (*device_and_host_malloc)(void *user_context, struct halide_buffer_t *buf,
                                  const struct halide_device_interface_t *device_interface);
    int (*device_and_host_free)(void *user_context, struct halide_buffer_t *buf);
    int (*buffer_copy)(void *user_context, struct halide_buffer_t *src,
                       const struct halide_device_interface_t *dst_device_interface, struct halide_buffer_t *dst);
    int (*device_crop)(void *user_context, const struct halide_buffer_t *src, struct halide_buffer_t *dst);
    int (*device_slice)(void *user_context, const struct halide_buffer_t *src, int slice_dim, int slice_pos,
                        struct halide_buffer_t *dst);
    int (*device_release_crop)(void *user_context, struct halide_buffer_t *buf);
    int (*wrap_native)(void *user_context, struct halide_buffer_t *buf, uint64_t handle,
                       const struct halide_device_interface_t *device_interface);
    int (*detach_native)(void *user_context, struct halide_buffer_t *buf);
    int (*compute_capability)(void *user_context, int *major, int *minor);
    const struct halide_device_interface_impl_t *impl;
};

enum { halide_buffer_flag_host_dirty = 1, halide_buffer_flag_device_dirty = 2 };

/* 56 bytes. */
typedef struct halide_buffer_t {
    uint64_t device;                                  /* opaque device handle, 0 = none */
    const struct halide_device_interface_t *device_interface;
    uint8_t *host;                                    /* host pointer to element (min0, min1, ...) */
    uint64_t flags;                                   /* halide_buffer_flag_* */
    struct halide_type_t type;
    int32_t dimensions;
    halide_dimension_t *dim;                          /* dimensions entries, dim[0] innermost */
    void *padding;
} halide_buffer_t;

#ifdef __cplusplus
}
#endif

#define T2SP_B200_OWN_HALIDE_ABI 1
#endif /* HALIDE_HALIDERUNTIME_H */

#ifdef __cplusplus
static_assert(sizeof(struct halide_type_t) == 4, "halide_type_t must be 4 bytes");
static_assert(sizeof(halide_dimension_t) == 16, "halide_dimension_t must be 16 bytes");
static_assert(sizeof(halide_buffer_t) == 56, "halide_buffer_t must be 56 bytes");
static_assert(sizeof(struct halide_device_interface_t) == 16 * sizeof(void *), "halide_device_interface_t is 15 functions and impl");
static_assert(offsetof(halide_buffer_t, host) == 16 && offsetof(halide_buffer_t, flags) == 24 &&
                  offsetof(halide_buffer_t, type) == 32 && offsetof(halide_buffer_t, dimensions) == 36 &&
                  offsetof(halide_buffer_t, dim) == 40,
              "halide_buffer_t field offsets");
#endif

#endif /* T2SP_B200_ABI_H */
