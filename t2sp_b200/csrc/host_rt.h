// Host-side device runtime: per-thread device/stream, a caching device allocator, TMA
// descriptor encoding, the kernel status word and the Halide-style error reporters.
// Replaces t2s/src/AOT-OpenCL-Runtime.cpp (context/queue set-up :128-274, device malloc
// :74-117, blocking copies :402-441, launch+wait+timing :312-397, error printers :443-727).
//
// Threads: every host thread gets, per device it uses, a slot of its own (stream, timing event
// pair, status word, the side streams of the pipelined host path). Slots are pooled: a thread
// that exits hands its slots back and a later thread takes them over. Cached device blocks carry
// the stream they were last used on and an event recorded when they were released; a block that
// moves to another stream makes that stream wait for the event first.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

#include "t2sp_b200/runtime.h"
#include "umma_launch.h"

namespace t2sp {

constexpr int kMaxDevices = 64;

// A device view of a caller's buffer for the duration of one call.
struct DeviceView {
    void* ptr = nullptr;      // device address of element (min0, min1, ...)
    bool borrowed = false;    // true: the caller's own device allocation; false: from the cache
    bool preloaded = false;   // output, not borrowed: the host span was uploaded first, so the whole span may go back
    size_t bytes = 0;
};

struct Slot;

struct ThreadState {
    int device = 0;
    cudaStream_t user_stream = nullptr;
    bool has_user_stream = false;
    bool async = false;
    double last_kernel_ns = 0.0;
    Slot* slot[kMaxDevices] = {};
    ~ThreadState();
};

ThreadState& tls();

// Environment knobs, read once when the library is first used and again on t2sp_b200_reload_env().
struct Env {
    bool no_tma_store = false, no_pair = false, pair128 = false, no_splitk = false, no_pipeline = false, log = false;
    bool no_presplit = false;  // fp32 pair kernel: B's bf16 tiles always from the split warps, never from a pre-pass
    bool no_tm128 = false;     // fp32 outputs of exactly 128 columns never on the 256 x 128 form of the tensor-memory pair kernel
    bool no_x3tm = false;      // fp32 pair tiles through the all-shared-memory 3xTF32 kernel instead of the tensor-memory one
    bool mttkrp_v1 = false;    // MTTKRP through the Khatri-Rao-tile kernel even where the accumulate-then-scale kernel applies
    int splitk = 0;            // forced number of split-K ranges of the fp32 pair kernel, 0 = choose
    int precision = 0;         // T2SP_PRECISION_* that T2SP_PRECISION_DEFAULT resolves to
    int group_m = 0;           // rasterisation group, 0 = per-kernel default
    int pair2 = -1;            // 512-row pair tiles: -1 = choose, 0 / 1 = forced
    unsigned long long fail_alloc_above = 0;  // host-side fault injection: allocations of at least this many bytes fail (0 = off)
    long long wait_cycles = 0;                // bounded-wait limit of the kernels in SM cycles, 0 = default
    int test_skip_stage = 0;                  // test hook: the single-CTA kernel's producer leaves out this k-block's copies
    std::string exec_time_path;               // where exec_time.txt goes, empty = nowhere
};
const Env& rt_env();

// Lazily initialises the device (driver entry points) and this thread's slot on it. Returns 0 or a
// negative halide_error_code_t; never exits the process.
int rt_ensure_device();
cudaStream_t rt_stream();
unsigned* rt_status_word();           // device address (this thread's)
int rt_check_status(const char* who); // after a stream sync: maps a raised status bit to device_run_failed

void* rt_alloc(size_t bytes);         // cached device allocation (nullptr on failure)
void rt_free(void* p);                // back to the cache; later users on other streams wait for this stream's work so far
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
                    bool promote256 = true, int swizzle_bytes = 128);

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
// Publishes the output: leaves it on the device (device_dirty) or copies the buffer's region (not the
// padding between its rows) to host (host_dirty).
int rt_finish_output(halide_buffer_t* b, const char* name, DeviceView* v);
void rt_drop_view(DeviceView* v);
// Zeroes the buffer's region (elements inside its extents only) in the device copy whose element
// (min0, min1, ...) is at `dev`.
void rt_zero_region(const halide_buffer_t* b, void* dev);
// Copies a device-resident buffer's content between b->host and b->device on the thread's stream (no wait).
bool rt_move_buffer(const halide_buffer_t* b, bool to_host);
cudaEvent_t rt_event(int which);
// Two side streams (host->device, device->host) and a pool of untimed events for overlapping the
// copies of a large host-buffer call with its kernels; this thread's own. Created on first use; false on failure.
bool rt_side_resources(cudaStream_t* h2d, cudaStream_t* d2h, cudaEvent_t** pool, int* pool_size);

}  // namespace t2sp
