/* Stand-in for the C-for-Metal runtime header the reference's CM-flow drivers include
 * (t2s/tests/performance/gemm/gemm-run-gpu-cm.cpp:28-30, 64-157; conv-run-gpu-cm.cpp, capsule-run-gpu-cm.cpp):
 * only the classes, methods and constants those drivers use, with their call signatures, over this
 * library. A 2-D R32F surface is a dense device buffer (width = dimension 0); the "program" is the
 * design's name, read from the name of the .isa file; enqueueing the task runs the operator on the
 * calling thread's CUDA device and the event reports its CUDA-event time. Put this directory on the
 * include path in place of the CM runtime's and link t2sp_b200/csrc/stubs/l0_shim.cpp and
 * libt2sp_b200.so. The conv / capsule constants are captured from the macros of the design's
 * const-parameters.h, which the drivers include first; identifiers here are long because those
 * headers define macros such as I, K, N, X. */
#ifndef T2SP_B200_CM_RT_H
#define T2SP_B200_CM_RT_H
/* the drivers rely on this header for the C library (fabs, rand, time, SIZE_MAX) */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <string>

extern "C" {
void *t2sp_l0_image_create(unsigned t2sp_width, unsigned t2sp_height, const void *t2sp_data);
int t2sp_l0_image_write(void *t2sp_image, const void *t2sp_src);
int t2sp_l0_image_read(void *t2sp_image, void *t2sp_dst);
void t2sp_l0_image_destroy(void *t2sp_image);
int t2sp_l0_run(int t2sp_op, const int *t2sp_design, void *const *t2sp_images);
double t2sp_l0_last_kernel_ns(void);
}

typedef unsigned long long UINT64;
typedef int INT;
typedef unsigned int UINT;
enum { CM_SUCCESS = 0, CM_FAILURE = -1 };
enum CM_SURFACE_FORMAT { CM_SURFACE_FORMAT_R32F = 114 };

struct SurfaceIndex {
    void *t2sp_image;
};

class CmEvent {
  public:
    UINT64 t2sp_ns = 0;
    INT WaitForTaskFinished(UINT = 0) { return CM_SUCCESS; } /* enqueueing already waited */
    INT GetExecutionTime(UINT64 &t2sp_time) { t2sp_time = t2sp_ns; return CM_SUCCESS; }
};

class CmSurface2D {
  public:
    SurfaceIndex t2sp_index{nullptr};
    INT WriteSurface(const unsigned char *t2sp_src, CmEvent *) { return t2sp_l0_image_write(t2sp_index.t2sp_image, t2sp_src); }
    INT ReadSurface(unsigned char *t2sp_dst, CmEvent *) { return t2sp_l0_image_read(t2sp_index.t2sp_image, t2sp_dst); }
    INT GetIndex(SurfaceIndex *&t2sp_out) { t2sp_out = &t2sp_index; return CM_SUCCESS; }
};

class CmProgram {
  public:
    int t2sp_op = 0;
};

class CmKernel {
  public:
    int t2sp_op = 0;
    int t2sp_design[16] = {0};
    void *t2sp_bound[8] = {nullptr};
    /* surfaces are told from scalars by the size of the argument */
    INT SetKernelArg(UINT t2sp_slot, size_t t2sp_size, const void *t2sp_value) {
        if (t2sp_slot >= 8) return CM_FAILURE;
        t2sp_bound[t2sp_slot] = t2sp_size == sizeof(SurfaceIndex) ? static_cast<const SurfaceIndex *>(t2sp_value)->t2sp_image : nullptr;
        return CM_SUCCESS;
    }
};

class CmTask {
  public:
    CmKernel *t2sp_kernel = nullptr;
    INT AddKernel(CmKernel *t2sp_k) { t2sp_kernel = t2sp_k; return CM_SUCCESS; }
};

class CmThreadGroupSpace {};

class CmQueue {
  public:
    INT EnqueueWithGroup(CmTask *t2sp_task, CmEvent *&t2sp_event, const CmThreadGroupSpace *) {
        CmKernel *t2sp_k = t2sp_task ? t2sp_task->t2sp_kernel : nullptr;
        if (!t2sp_k) return CM_FAILURE;
        void *t2sp_surfaces[3];
        int t2sp_count = 0;
        for (int t2sp_i = 0; t2sp_i < 8 && t2sp_count < 3; ++t2sp_i)
            if (t2sp_k->t2sp_bound[t2sp_i]) t2sp_surfaces[t2sp_count++] = t2sp_k->t2sp_bound[t2sp_i];
        if (t2sp_count != 3) return CM_FAILURE;
        /* binding order: gemm (A, B, C) gemm-run-gpu-cm.cpp:110-113, conv (I, K, O) conv-run-gpu-cm.cpp:110-112,
         * capsule (V, P, W) capsule-run-gpu-cm.cpp:117-119 */
        void *t2sp_images[3] = {t2sp_surfaces[0], t2sp_surfaces[1], t2sp_surfaces[2]};
        if (t2sp_k->t2sp_op == 2) { t2sp_images[0] = t2sp_surfaces[1]; t2sp_images[1] = t2sp_surfaces[2]; t2sp_images[2] = t2sp_surfaces[0]; }
        const int t2sp_rc = t2sp_l0_run(t2sp_k->t2sp_op, t2sp_k->t2sp_design, t2sp_images);
        t2sp_event = new CmEvent();
        t2sp_event->t2sp_ns = (UINT64)t2sp_l0_last_kernel_ns();
        return t2sp_rc;
    }
};

class CmDevice {
  public:
    INT LoadProgram(void *t2sp_code, UINT, CmProgram *&t2sp_program) {
        /* the "code" is the name of the .isa file (common/isa_helpers.h of this directory) */
        const char *t2sp_name = static_cast<const char *>(t2sp_code);
        t2sp_program = new CmProgram();
        t2sp_program->t2sp_op = strstr(t2sp_name, "capsule") ? 2 : (strstr(t2sp_name, "conv") ? 1 : 0);
        return CM_SUCCESS;
    }
    INT CreateKernel(CmProgram *t2sp_program, const char *, CmKernel *&t2sp_kernel) {
        t2sp_kernel = new CmKernel();
        t2sp_kernel->t2sp_op = t2sp_program->t2sp_op;
#if defined(MK) && defined(MX) && defined(MY) && defined(TOTAL_CI) && defined(TOTAL_CO)
        const int t2sp_vals[12] = {TOTAL_CI, CII, TOTAL_CO, KY, KX, OY, OX, MY, MX, MK, NN, 2};
        for (int t2sp_i = 0; t2sp_i < 12; ++t2sp_i) t2sp_kernel->t2sp_design[t2sp_i] = t2sp_vals[t2sp_i];
#elif defined(TOTAL_OY) && defined(TOTAL_OX) && defined(TOTAL_CI) && defined(TOTAL_CO)
        const int t2sp_vals[6] = {TOTAL_CI, TOTAL_CO, KY, KX, TOTAL_OY, TOTAL_OX};
        for (int t2sp_i = 0; t2sp_i < 6; ++t2sp_i) t2sp_kernel->t2sp_design[t2sp_i] = t2sp_vals[t2sp_i];
#endif
        return CM_SUCCESS;
    }
    INT CreateQueue(CmQueue *&t2sp_queue) { t2sp_queue = new CmQueue(); return CM_SUCCESS; }
    INT CreateSurface2D(UINT t2sp_width, UINT t2sp_height, CM_SURFACE_FORMAT t2sp_format, CmSurface2D *&t2sp_surface) {
        if (t2sp_format != CM_SURFACE_FORMAT_R32F) return CM_FAILURE;
        void *t2sp_img = t2sp_l0_image_create(t2sp_width, t2sp_height, nullptr);
        if (!t2sp_img) return CM_FAILURE;
        t2sp_surface = new CmSurface2D();
        t2sp_surface->t2sp_index.t2sp_image = t2sp_img;
        return CM_SUCCESS;
    }
    INT CreateTask(CmTask *&t2sp_task) { t2sp_task = new CmTask(); return CM_SUCCESS; }
    INT DestroyTask(CmTask *&t2sp_task) { delete t2sp_task; t2sp_task = nullptr; return CM_SUCCESS; }
    INT CreateThreadGroupSpace(UINT, UINT, UINT, UINT, CmThreadGroupSpace *&t2sp_space) { t2sp_space = new CmThreadGroupSpace(); return CM_SUCCESS; }
    INT CreateThreadGroupSpaceEx(UINT, UINT, UINT, UINT, UINT, UINT, CmThreadGroupSpace *&t2sp_space) { t2sp_space = new CmThreadGroupSpace(); return CM_SUCCESS; }
    INT InitPrintBuffer(size_t = 0) { return CM_SUCCESS; }
    INT FlushPrintBuffer() { return CM_SUCCESS; }
};

inline INT CreateCmDevice(CmDevice *&t2sp_device, UINT &t2sp_version) {
    t2sp_device = new CmDevice();
    t2sp_version = 0;
    return CM_SUCCESS;
}
inline INT DestroyCmDevice(CmDevice *&t2sp_device) {
    delete t2sp_device;
    t2sp_device = nullptr;
    return CM_SUCCESS;
}
#endif
