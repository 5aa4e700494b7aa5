/* Drop-in for t2s/tests/performance/util/l0_rt_helpers.h: the helper layer over Level Zero that the
 * reference's GPU-flow drivers are written against (gemm-run-gpu.cpp:66-129, conv-run-gpu.cpp:67-125,
 * capsule-run-gpu.cpp:74-131). Same helper names and argument lists; behind them there is no Level
 * Zero, SPIR-V module or surface state: a 2-D R32F image is a dense device buffer of this library
 * (width = dimension 0), "creating a kernel" from <design>_genx.bin selects the operator, binding
 * images records them, and the launch runs the operator on the calling thread's CUDA device and
 * returns when it has finished. Put this directory on the include path in place of the reference's
 * util/ directory and link t2sp_b200/csrc/stubs/l0_shim.cpp and libt2sp_b200.so.
 *
 * The reference bakes a design's constants into its kernel binary. Here they are captured from the
 * macros of the design's const-parameters.h, which every driver includes before this header
 * (conv-run-gpu.cpp:22-26): the conv / capsule constants are read where createKernel is compiled.
 * Identifiers in this header are long on purpose: the design headers define macros such as I, K, N, X. */
#ifndef L0_RT_HELPERS_H
#define L0_RT_HELPERS_H
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <initializer_list>
#include <limits>
#include <tuple>

extern "C" {
void *t2sp_l0_image_create(unsigned t2sp_width, unsigned t2sp_height, const void *t2sp_data);
int t2sp_l0_image_read(void *t2sp_image, void *t2sp_dst);
void t2sp_l0_image_destroy(void *t2sp_image);
/* t2sp_op: 0 gemm, 1 conv, 2 capsule; images in (input, input, output) order */
int t2sp_l0_run(int t2sp_op, const int *t2sp_design, void *const *t2sp_images);
}

typedef int ze_result_t;
#define ZE_RESULT_SUCCESS 0
#define L0_SAFE_CALL(t2sp_call)                                                                     \
    do {                                                                                            \
        const ze_result_t t2sp_status = (t2sp_call);                                                \
        if (t2sp_status != ZE_RESULT_SUCCESS) {                                                     \
            fprintf(stderr, "%s:%d: call failed with halide error %d\n", __FILE__, __LINE__, (int)t2sp_status); \
            exit(1);                                                                                \
        }                                                                                           \
    } while (0)

struct t2sp_l0_driver_tag;
struct t2sp_l0_device_tag;
struct t2sp_l0_context_tag;
struct t2sp_l0_cmdlist_tag;
struct t2sp_l0_event_tag;
struct t2sp_l0_image_tag;
typedef t2sp_l0_driver_tag *ze_driver_handle_t;
typedef t2sp_l0_device_tag *ze_device_handle_t;
typedef t2sp_l0_context_tag *ze_context_handle_t;
typedef t2sp_l0_cmdlist_tag *ze_command_list_handle_t;
typedef t2sp_l0_event_tag *ze_event_handle_t;
typedef t2sp_l0_image_tag *ze_image_handle_t;

enum { ZE_IMAGE_FORMAT_LAYOUT_32 = 2 };
enum { ZE_IMAGE_FORMAT_TYPE_FLOAT = 4 };
typedef struct {
    int t2sp_layout;
    int t2sp_type;
} ze_image_format_t;
typedef struct {
    uint32_t groupCountX, groupCountY, groupCountZ;
} ze_group_count_t;

struct t2sp_l0_kernel_record {
    int t2sp_op;
    int t2sp_design[16];
    ze_image_handle_t t2sp_bound[8];
    unsigned t2sp_nbound;
};
typedef t2sp_l0_kernel_record *ze_kernel_handle_t;

inline double getTimeStamp() {
    namespace t2sp_sc = std::chrono;
    return t2sp_sc::duration_cast<t2sp_sc::microseconds>(t2sp_sc::system_clock::now().time_since_epoch()).count() / 1e6;
}

inline auto findDriverAndDevice() {
    return std::make_tuple((ze_driver_handle_t) nullptr, (ze_device_handle_t) nullptr, (ze_context_handle_t) nullptr);
}
inline ze_command_list_handle_t createImmCommandList(ze_context_handle_t, ze_device_handle_t) { return nullptr; }

inline ze_image_handle_t createImage2D(ze_context_handle_t, ze_device_handle_t, ze_command_list_handle_t,
                                       ze_image_format_t &t2sp_fmt, unsigned int t2sp_width, unsigned int t2sp_height,
                                       const void *t2sp_data = nullptr) {
    if (t2sp_fmt.t2sp_layout != ZE_IMAGE_FORMAT_LAYOUT_32 || t2sp_fmt.t2sp_type != ZE_IMAGE_FORMAT_TYPE_FLOAT) {
        fprintf(stderr, "createImage2D: only 32-bit float images are supported\n");
        exit(1);
    }
    void *t2sp_img = t2sp_l0_image_create(t2sp_width, t2sp_height, t2sp_data);
    if (!t2sp_img) {
        fprintf(stderr, "createImage2D: device allocation or upload failed\n");
        exit(1);
    }
    return (ze_image_handle_t)t2sp_img;
}

/* The constants of the design this translation unit was compiled for. */
inline void t2sp_l0_capture_design(int *t2sp_out) {
    for (int t2sp_i = 0; t2sp_i < 16; ++t2sp_i) t2sp_out[t2sp_i] = 0;
#if defined(MK) && defined(MX) && defined(MY) && defined(TOTAL_CI) && defined(TOTAL_CO)
    /* capsule (t2s/tests/performance/capsule/const-parameters.h): stride 2 is part of the design (capsule.cpp:40-41) */
    const int t2sp_vals[12] = {TOTAL_CI, CII, TOTAL_CO, KY, KX, OY, OX, MY, MX, MK, NN, 2};
    for (int t2sp_i = 0; t2sp_i < 12; ++t2sp_i) t2sp_out[t2sp_i] = t2sp_vals[t2sp_i];
#elif defined(TOTAL_OY) && defined(TOTAL_OX) && defined(TOTAL_CI) && defined(TOTAL_CO)
    /* conv (t2s/tests/performance/conv/const-parameters.h) */
    const int t2sp_vals[6] = {TOTAL_CI, TOTAL_CO, KY, KX, TOTAL_OY, TOTAL_OX};
    for (int t2sp_i = 0; t2sp_i < 6; ++t2sp_i) t2sp_out[t2sp_i] = t2sp_vals[t2sp_i];
#endif
}

inline ze_kernel_handle_t createKernel(ze_context_handle_t, ze_device_handle_t, const char *t2sp_file, const char *) {
    ze_kernel_handle_t t2sp_k = new t2sp_l0_kernel_record();
    t2sp_k->t2sp_op = strstr(t2sp_file, "capsule") ? 2 : (strstr(t2sp_file, "conv") ? 1 : 0);
    t2sp_k->t2sp_nbound = 0;
    t2sp_l0_capture_design(t2sp_k->t2sp_design);
    return t2sp_k;
}

inline void t2sp_l0_bind(ze_kernel_handle_t t2sp_k, ze_image_handle_t *t2sp_img) {
    if (t2sp_k->t2sp_nbound < 8) t2sp_k->t2sp_bound[t2sp_k->t2sp_nbound++] = *t2sp_img;
}
template <typename t2sp_scalar>
inline void t2sp_l0_bind(ze_kernel_handle_t, t2sp_scalar *) {} /* extents: the images carry them */

template <typename... t2sp_args>
inline void setKernelArgs(ze_kernel_handle_t t2sp_k, t2sp_args... t2sp_a) {
    t2sp_k->t2sp_nbound = 0;
    (void)std::initializer_list<int>{(t2sp_l0_bind(t2sp_k, t2sp_a), 0)...};
}

inline ze_result_t zeKernelSetGroupSize(ze_kernel_handle_t, uint32_t, uint32_t, uint32_t) { return ZE_RESULT_SUCCESS; }
inline ze_event_handle_t createEvent(ze_context_handle_t, ze_device_handle_t &) { return nullptr; }
inline ze_result_t zeEventHostSynchronize(ze_event_handle_t, uint64_t) { return ZE_RESULT_SUCCESS; } /* launches are synchronous */

inline void appendLaunchKernel(ze_command_list_handle_t, ze_kernel_handle_t t2sp_k, ze_group_count_t *,
                               ze_event_handle_t = nullptr, unsigned = 0, ze_event_handle_t * = nullptr) {
    /* binding order: gemm (A, B, C) gemm-run-gpu.cpp:86; conv (I, K, O) conv-run-gpu.cpp:85;
     * capsule (V, P, W) capsule-run-gpu.cpp:92 */
    void *t2sp_images[3];
    if (t2sp_k->t2sp_nbound != 3) {
        fprintf(stderr, "appendLaunchKernel: expected three images, %u bound\n", t2sp_k->t2sp_nbound);
        exit(1);
    }
    if (t2sp_k->t2sp_op == 2) {
        t2sp_images[0] = t2sp_k->t2sp_bound[1]; t2sp_images[1] = t2sp_k->t2sp_bound[2]; t2sp_images[2] = t2sp_k->t2sp_bound[0];
    } else {
        t2sp_images[0] = t2sp_k->t2sp_bound[0]; t2sp_images[1] = t2sp_k->t2sp_bound[1]; t2sp_images[2] = t2sp_k->t2sp_bound[2];
    }
    L0_SAFE_CALL(t2sp_l0_run(t2sp_k->t2sp_op, t2sp_k->t2sp_design, t2sp_images));
}

inline void copyToMemory(ze_command_list_handle_t, void *t2sp_dst, ze_image_handle_t t2sp_src, ze_event_handle_t = nullptr) {
    L0_SAFE_CALL(t2sp_l0_image_read((void *)t2sp_src, t2sp_dst));
}

inline void destroy(ze_context_handle_t) {}
inline void destroy(ze_command_list_handle_t) {}
inline void destroy(ze_image_handle_t t2sp_img) { t2sp_l0_image_destroy((void *)t2sp_img); }
#endif
