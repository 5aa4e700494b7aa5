// Device runtime behind the C ABI. See host_rt.h for the reference files it replaces.
#include "host_rt.h"

#include <cudaTypedefs.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace t2sp {

namespace {

constexpr int kMaxDevices = 16;

struct DeviceState {
    bool ready = false;
    int init_error = 0;
    cudaStream_t stream = nullptr;
    unsigned* status_dev = nullptr;
    unsigned* status_host = nullptr;  // pinned
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // copy/compute overlap of large host-buffer calls: two side streams and a pool of ordering events
    cudaStream_t side[2] = {nullptr, nullptr};
    cudaEvent_t pool[64] = {};
    bool side_ready = false;
    // caching allocator: free blocks by size, live blocks by address
    std::multimap<size_t, void*> free_blocks;
    std::map<void*, size_t> live_blocks;
};

std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
std::atomic<uint64_t> g_launches{0};
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

size_t round_up_block(size_t bytes) {
    // 2 MiB granularity above 1 MiB, 64 KiB below: few distinct sizes, good reuse.
    const size_t g = bytes > (1u << 20) ? (2u << 20) : (64u << 10);
    return (bytes + g - 1) / g * g;
}

}  // namespace

ThreadState& tls() {
    static thread_local ThreadState st;
    return st;
}

int rt_ensure_device() {
    ThreadState& ts = tls();
    if (ts.device < 0 || ts.device >= kMaxDevices) return halide_error_code_device_interface_no_device;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[ts.device];
    if (d.ready) {
        return cudaSetDevice(ts.device) == cudaSuccess ? 0 : halide_error_code_device_interface_no_device;
    }
    if (d.init_error) return d.init_error;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || ts.device >= count) {
        cudaGetLastError();
        fprintf(stderr, "t2sp_b200: no CUDA device %d is available; this library has no CPU path\n", ts.device);
        return halide_error_code_device_interface_no_device;  // not latched: a later call may find a device
    }
    if (cudaSetDevice(ts.device) != cudaSuccess) return halide_error_code_device_interface_no_device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ts.device) != cudaSuccess || prop.major != 10) {
        fprintf(stderr, "t2sp_b200: device %d is not an sm_100 GPU; the kernels are built for sm_100a only\n",
                ts.device);
        d.init_error = halide_error_code_device_interface_no_device;
        return d.init_error;
    }
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) {
            fprintf(stderr, "t2sp_b200: the CUDA driver does not provide cuTensorMapEncodeTiled\n");
            d.init_error = halide_error_code_device_interface_no_device;
            return d.init_error;
        }
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    if (cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&d.status_dev, sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(d.status_dev, 0, sizeof(unsigned)) != cudaSuccess ||
        cudaMallocHost(&d.status_host, sizeof(unsigned)) != cudaSuccess ||
        cudaEventCreate(&d.ev0) != cudaSuccess || cudaEventCreate(&d.ev1) != cudaSuccess) {
        cudaGetLastError();
        d.init_error = halide_error_code_device_malloc_failed;
        return d.init_error;
    }
    *d.status_host = 0;
    d.ready = true;
    return 0;
}

cudaStream_t rt_stream() {
    ThreadState& ts = tls();
    if (ts.has_user_stream) return ts.user_stream;
    return g_dev[ts.device].stream;
}

unsigned* rt_status_word() { return g_dev[tls().device].status_dev; }

cudaEvent_t rt_event(int which) { return which ? g_dev[tls().device].ev1 : g_dev[tls().device].ev0; }

bool rt_side_resources(cudaStream_t* h2d, cudaStream_t* d2h, cudaEvent_t** pool, int* pool_size) {
    DeviceState& d = g_dev[tls().device];
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d.side_ready) {
        for (int i = 0; i < 2; ++i)
            if (cudaStreamCreateWithFlags(&d.side[i], cudaStreamNonBlocking) != cudaSuccess) return false;
        for (int i = 0; i < 64; ++i)
            if (cudaEventCreateWithFlags(&d.pool[i], cudaEventDisableTiming) != cudaSuccess) return false;
        d.side_ready = true;
    }
    *h2d = d.side[0];
    *d2h = d.side[1];
    *pool = d.pool;
    *pool_size = 64;
    return true;
}

int rt_check_status(const char* who) {
    DeviceState& d = g_dev[tls().device];
    cudaStream_t s = rt_stream();
    if (cudaMemcpyAsync(d.status_host, d.status_dev, sizeof(unsigned), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        fprintf(stderr, "t2sp_b200: %s: device execution failed: %s\n", who, cudaGetErrorString(e));
        return halide_error_code_device_run_failed;
    }
    if (*d.status_host != 0) {
        fprintf(stderr, "t2sp_b200: %s: a kernel gave up waiting (status 0x%x: %s%s%s%s)\n", who, *d.status_host,
                (*d.status_host & ST_TIMEOUT_PRODUCER) ? "producer " : "", (*d.status_host & ST_TIMEOUT_MMA) ? "mma " : "",
                (*d.status_host & ST_TIMEOUT_EPILOGUE) ? "epilogue " : "",
                (*d.status_host & ST_TIMEOUT_SPLITTER) ? "splitter " : "");
        cudaMemsetAsync(d.status_dev, 0, sizeof(unsigned), s);
        cudaStreamSynchronize(s);
        *d.status_host = 0;
        return halide_error_code_device_run_failed;
    }
    return 0;
}

void* rt_alloc(size_t bytes) {
    if (bytes == 0) bytes = 16;
    const size_t want = round_up_block(bytes);
    // Host-side fault injection for tests: fail every allocation of at least this many bytes.
    if (const char* lim = getenv("T2SP_B200_FAIL_ALLOC_ABOVE")) {
        if (want >= strtoull(lim, nullptr, 10)) return nullptr;
    }
    DeviceState& d = g_dev[tls().device];
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = d.free_blocks.lower_bound(want);
        if (it != d.free_blocks.end() && it->first <= want * 2) {
            void* p = it->second;
            d.live_blocks[p] = it->first;
            d.free_blocks.erase(it);
            return p;
        }
    }
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        // Return cached blocks to the driver and retry once.
        {
            std::lock_guard<std::mutex> lk(g_mu);
            for (auto& kv : d.free_blocks) cudaFree(kv.second);
            d.free_blocks.clear();
        }
        if (cudaMalloc(&p, want) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
    }
    std::lock_guard<std::mutex> lk(g_mu);
    d.live_blocks[p] = want;
    return p;
}

void rt_free(void* p) {
    if (!p) return;
    DeviceState& d = g_dev[tls().device];
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = d.live_blocks.find(p);
    if (it == d.live_blocks.end()) return;
    d.free_blocks.emplace(it->second, p);
    d.live_blocks.erase(it);
}

void rt_release_all() {
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < kMaxDevices; ++i) {
        DeviceState& d = g_dev[i];
        if (!d.ready) continue;
        cudaSetDevice(i);
        cudaDeviceSynchronize();
        for (auto& kv : d.free_blocks) cudaFree(kv.second);
        d.free_blocks.clear();
    }
}

void rt_count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n)); }
uint64_t rt_launch_count() { return g_launches.load(); }

bool rt_encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, bool atom32, bool promote256) {
    if (!g_encode) return false;
    cuuint64_t gdim[5];
    cuuint64_t gstr[4];
    cuuint32_t bdim[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i];
    }
    CUresult r = g_encode(out, dtype, static_cast<cuuint32_t>(rank), base, gdim, gstr, bdim, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                          promote256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (getenv("T2SP_B200_LOG"))
            fprintf(stderr, "t2sp_b200: cuTensorMapEncodeTiled failed (%d) rank=%d base=%p dims0=%llu box0=%u\n", (int)r,
                    rank, base, (unsigned long long)dims[0], box[0]);
        return false;
    }
    return true;
}

void rt_write_exec_time(const char* kernel_name, double ns) {
    // Same format as the reference runtime's exec_time.txt: first line the overall time, then
    // one "<kernel> <ns>" line per kernel (AOT-OpenCL-Runtime.cpp:380-395, read by Roofline.cpp:113-140).
    std::string path;
    if (const char* bs = getenv("BITSTREAM")) {
        std::string b(bs);
        size_t pos = b.find_last_of('/');
        path = (pos == std::string::npos ? std::string(".") : b.substr(0, pos)) + "/exec_time.txt";
    } else if (const char* f = getenv("T2SP_B200_EXEC_TIME_FILE")) {
        path = f;
    } else {
        return;
    }
    if (FILE* fp = fopen(path.c_str(), "w")) {
        fprintf(fp, "%.0f\n%s %.0f\nkernel_unloader %.0f\n", ns, kernel_name, ns, ns);
        fclose(fp);
    }
}

// ------------------------------------------------------------------ buffer movement
namespace {

bool is_dense_span(const halide_buffer_t* b) { return b->dimensions > 0; }

// Copies the span [host, host + span) <-> device. Buffers are moved as their whole address
// span (strides are kept on the device), which is exact for dense buffers and still
// correct, if wasteful, for padded ones.
size_t span_bytes(const halide_buffer_t* b) { return static_cast<size_t>(buf_elems_span(b)) * ((b->type.bits + 7) / 8); }

}  // namespace

int rt_input_view(halide_buffer_t* b, const char* name, DeviceView* v) {
    (void)is_dense_span;
    v->bytes = span_bytes(b);
    const bool host_dirty = (b->flags & 1u) != 0;
    if (buf_on_our_device(b) && !(host_dirty && b->host)) {
        v->ptr = reinterpret_cast<void*>(b->device);
        v->borrowed = true;
        return 0;
    }
    if (!b->host) {
        fprintf(stderr, "t2sp_b200: Input buffer %s has neither host data nor a device allocation of this library\n",
                name);
        return halide_error_code_host_is_null;
    }
    if (buf_on_our_device(b)) {
        v->ptr = reinterpret_cast<void*>(b->device);
        v->borrowed = true;
    } else {
        v->ptr = rt_alloc(v->bytes);
        v->borrowed = false;
        if (!v->ptr) {
            fprintf(stderr, "t2sp_b200: device allocation of %zu bytes for %s failed\n", v->bytes, name);
            return halide_error_code_device_malloc_failed;
        }
    }
    if (v->bytes &&
        cudaMemcpyAsync(v->ptr, b->host, v->bytes, cudaMemcpyHostToDevice, rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        rt_drop_view(v);
        return halide_error_code_copy_to_device_failed;
    }
    if (v->borrowed) b->flags &= ~uint64_t(1);
    return 0;
}

int rt_output_view(halide_buffer_t* b, const char* name, DeviceView* v) {
    v->bytes = span_bytes(b);
    if (buf_on_our_device(b)) {
        v->ptr = reinterpret_cast<void*>(b->device);
        v->borrowed = true;
        return 0;
    }
    v->ptr = rt_alloc(v->bytes);
    v->borrowed = false;
    if (!v->ptr) {
        fprintf(stderr, "t2sp_b200: device allocation of %zu bytes for %s failed\n", v->bytes, name);
        return halide_error_code_device_malloc_failed;
    }
    return 0;
}

int rt_finish_output(halide_buffer_t* b, const char* name, DeviceView* v) {
    (void)name;
    if (v->borrowed) {
        b->flags |= 2u;   // device_dirty
        b->flags &= ~uint64_t(1);
        return 0;
    }
    if (v->bytes &&
        cudaMemcpyAsync(b->host, v->ptr, v->bytes, cudaMemcpyDeviceToHost, rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        return halide_error_code_copy_to_host_failed;
    }
    b->flags |= 1u;  // host_dirty
    b->flags &= ~uint64_t(2);
    return 0;
}

void rt_drop_view(DeviceView* v) {
    if (v->ptr && !v->borrowed) rt_free(v->ptr);
    v->ptr = nullptr;
}

}  // namespace t2sp

// ---------------------------------------------------------------------- C ABI: runtime part
using namespace t2sp;

extern "C" {

// A distinct address is all callers need from the device interface: it tags buffers whose
// `device` field holds a CUDA device pointer owned or wrapped by this library.
struct t2sp_b200_device_interface_tag {
    char name[32];
};
static const t2sp_b200_device_interface_tag g_interface_tag = {"t2sp_b200/cuda"};

const struct halide_device_interface_t* t2sp_b200_device_interface(void) {
    return reinterpret_cast<const struct halide_device_interface_t*>(&g_interface_tag);
}

int t2sp_b200_device_malloc(halide_buffer_t* buf) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    if (buf->device) return 0;
    if (int e = rt_ensure_device()) return e;
    const size_t bytes = static_cast<size_t>(buf_elems_span(buf)) * ((buf->type.bits + 7) / 8);
    void* p = rt_alloc(bytes);
    if (!p) return halide_error_code_device_malloc_failed;
    buf->device = reinterpret_cast<uint64_t>(p);
    buf->device_interface = t2sp_b200_device_interface();
    return 0;
}

int t2sp_b200_device_free(halide_buffer_t* buf) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    if (!buf_on_our_device(buf)) return 0;
    if (int e = rt_ensure_device()) return e;
    cudaStreamSynchronize(rt_stream());
    rt_free(reinterpret_cast<void*>(buf->device));
    buf->device = 0;
    buf->device_interface = nullptr;
    buf->flags &= ~uint64_t(2);
    return 0;
}

int t2sp_b200_copy_to_device(halide_buffer_t* buf) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    if (!buf->host) return halide_error_code_host_is_null;
    if (int e = t2sp_b200_device_malloc(buf)) return e;
    if (!buf_on_our_device(buf)) return halide_error_code_copy_to_device_failed;
    const size_t bytes = static_cast<size_t>(buf_elems_span(buf)) * ((buf->type.bits + 7) / 8);
    if (cudaMemcpyAsync(reinterpret_cast<void*>(buf->device), buf->host, bytes, cudaMemcpyHostToDevice,
                        rt_stream()) != cudaSuccess ||
        cudaStreamSynchronize(rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        return halide_error_code_copy_to_device_failed;
    }
    buf->flags &= ~uint64_t(1);
    return 0;
}

int t2sp_b200_copy_to_host(halide_buffer_t* buf) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    if (!buf_on_our_device(buf)) return 0;
    if (!buf->host) return halide_error_code_host_is_null;
    if (int e = rt_ensure_device()) return e;
    const size_t bytes = static_cast<size_t>(buf_elems_span(buf)) * ((buf->type.bits + 7) / 8);
    if (cudaMemcpyAsync(buf->host, reinterpret_cast<void*>(buf->device), bytes, cudaMemcpyDeviceToHost,
                        rt_stream()) != cudaSuccess ||
        cudaStreamSynchronize(rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        return halide_error_code_copy_to_host_failed;
    }
    buf->flags &= ~uint64_t(2);
    return 0;
}

int t2sp_b200_wrap_device_ptr(halide_buffer_t* buf, uint64_t device_ptr) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    if (buf->device != 0) return -32;  // halide_error_code_device_wrap_native_failed
    buf->device = device_ptr;
    buf->device_interface = t2sp_b200_device_interface();
    return 0;
}

int t2sp_b200_detach_device_ptr(halide_buffer_t* buf) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    buf->device = 0;
    buf->device_interface = nullptr;
    return 0;
}

int t2sp_b200_set_device(int ordinal) {
    if (ordinal < 0 || ordinal >= 16) return halide_error_code_device_interface_no_device;
    tls().device = ordinal;
    return 0;
}

int t2sp_b200_set_stream(void* cuda_stream) {
    ThreadState& ts = tls();
    ts.user_stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    ts.has_user_stream = true;
    return 0;
}

int t2sp_b200_set_async(int enable) {
    tls().async = enable != 0;
    return 0;
}

int t2sp_b200_sync(void) {
    if (int e = rt_ensure_device()) return e;
    return rt_check_status("t2sp_b200_sync");
}

void t2sp_b200_release(void) { rt_release_all(); }
uint64_t t2sp_b200_kernel_launches(void) { return rt_launch_count(); }
double t2sp_b200_last_kernel_ns(void) { return tls().last_kernel_ns; }
const char* t2sp_b200_version(void) { return "t2sp_b200 0.1 (sm_100a)"; }

int t2sp_b200_device_info(int* sm_count, int* sm_clock_khz) {
    if (int e = rt_ensure_device()) return e;
    int sms = 0, khz = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, tls().device) != cudaSuccess ||
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, tls().device) != cudaSuccess)
        return halide_error_code_device_interface_no_device;
    if (sm_count) *sm_count = sms;
    if (sm_clock_khz) *sm_clock_khz = khz;
    return 0;
}

}  // extern "C"
