// Host-side device runtime: per-thread device/stream, a caching device allocator, TMA
// descriptor encoding, the kernel status word and the Halide-style error reporters.
// Replaces t2s/src/AOT-OpenCL-Runtime.cpp (context/queue set-up :128-274, device malloc
// :74-117, blocking copies :402-441, launch+wait+timing :312-397, error printers :443-727).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "t2sp_b200/runtime.h"
#include "umma_launch.h"

namespace t2sp {

// A device view of a caller's buffer for the duration of one call.
struct DeviceView {
    void* ptr = nullptr;      // device address of element (min0, min1, ...)
    bool borrowed = false;    // true: the caller's own device allocation; false: from the cache
    size_t bytes = 0;
};

struct ThreadState {
    int device = 0;
    cudaStream_t user_stream = nullptr;
    bool has_user_stream = false;
    bool async = false;
    double last_kernel_ns = 0.0;
};

ThreadState& tls();

// Lazily initialises the device (stream, status word, driver entry points). Returns 0 or a
// negative halide_error_code_t; never exits the process.
int rt_ensure_device();
cudaStream_t rt_stream();
unsigned* rt_status_word();           // device address
int rt_check_status(const char* who); // after a stream sync: maps a raised status bit to device_run_failed

void* rt_alloc(size_t bytes);         // cached device allocation (nullptr on failure)
void rt_free(void* p);
void rt_release_all();

void rt_count_launch(int n);
uint64_t rt_launch_count();

// Encodes a tiled TMA descriptor. dims/strides innermost first; strides in bytes for
// dims 1..rank-1 (stride of dim 0 is the element size). The shared-memory side uses the 128-byte
// swizzle, with 32-byte atoms when `atom32` (the layout MN-major fp32 UMMA operands need).
// `promote256` lets L2 fetch 256-byte lines (good when the neighbouring 128 bytes are wanted next,
// wasteful when they are not). Returns false when the driver rejects it.
bool rt_encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, bool atom32 = false,
                    bool promote256 = true);

void rt_write_exec_time(const char* kernel_name, double ns);

// element helpers on halide_buffer_t
inline int64_t buf_elems_span(const halide_buffer_t* b) {
    int64_t span = 1;
    for (int d = 0; d < b->dimensions; ++d) {
        if (b->dim[d].extent <= 0) return 0;
        int64_t s = b->dim[d].stride < 0 ? -(int64_t)b->dim[d].stride : (int64_t)b->dim[d].stride;
        span += s * (b->dim[d].extent - 1);
    }
    return span;
}
inline bool buf_is_bounds_query(const halide_buffer_t* b) { return b->host == nullptr && b->device == 0; }
inline bool buf_on_our_device(const halide_buffer_t* b) {
    return b->device != 0 && b->device_interface == t2sp_b200_device_interface();
}

// Brings an input to the device (borrowing the caller's allocation when it is current).
int rt_input_view(halide_buffer_t* b, const char* name, DeviceView* v);
// Provides device memory for an output.
int rt_output_view(halide_buffer_t* b, const char* name, DeviceView* v);
// Publishes the output: leaves it on the device (device_dirty) or copies to host (host_dirty).
int rt_finish_output(halide_buffer_t* b, const char* name, DeviceView* v);
void rt_drop_view(DeviceView* v);
cudaEvent_t rt_event(int which);
// Two side streams (host->device, device->host) and a pool of untimed events for overlapping the
// copies of a large host-buffer call with its kernels. Created on first use; false on failure.
bool rt_side_resources(cudaStream_t* h2d, cudaStream_t* d2h, cudaEvent_t** pool, int* pool_size);

}  // namespace t2sp
