// Device runtime behind the C ABI. See host_rt.h for the reference files it replaces.
#include "host_rt.h"

#include <cudaTypedefs.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace t2sp {

// What one host thread owns on one device.
struct Slot {
    cudaStream_t stream = nullptr;
    unsigned* status_dev = nullptr;
    unsigned* status_host = nullptr;  // pinned
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // copy/compute overlap of large host-buffer calls: two side streams and a pool of ordering events
    cudaStream_t side[2] = {nullptr, nullptr};
    cudaEvent_t pool[64] = {};
    bool side_ready = false;
};

namespace {

// A cached device block: the stream whose work touched it last and an event recorded on that stream
// when the block was released.
struct Block {
    size_t size = 0;
    cudaEvent_t released = nullptr;
    cudaStream_t stream = nullptr;
};

struct DeviceState {
    bool ready = false;
    int init_error = 0;
    std::vector<Slot*> idle_slots;
    // caching allocator: free blocks by size, live blocks by address
    std::multimap<size_t, std::pair<void*, Block>> free_blocks;
    std::map<void*, Block> live_blocks;
};

std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
std::atomic<uint64_t> g_launches{0};
std::atomic<const Env*> g_env{nullptr};
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

size_t round_up_block(size_t bytes) {
    // 2 MiB granularity above 1 MiB, 64 KiB below: few distinct sizes, good reuse.
    const size_t g = bytes > (1u << 20) ? (2u << 20) : (64u << 10);
    return (bytes + g - 1) / g * g;
}

const Env* read_env() {
    Env* e = new Env;
    e->no_tma_store = getenv("T2SP_B200_NO_TMA_STORE") != nullptr;
    e->no_pair = getenv("T2SP_B200_NO_PAIR") != nullptr;
    e->pair128 = getenv("T2SP_B200_PAIR128") != nullptr;
    e->no_splitk = getenv("T2SP_B200_NO_SPLITK") != nullptr;
    e->no_pipeline = getenv("T2SP_B200_NO_PIPELINE") != nullptr;
    e->log = getenv("T2SP_B200_LOG") != nullptr;
    e->mttkrp_v1 = getenv("T2SP_B200_MTTKRP_V1") != nullptr;
    e->no_x3tm = getenv("T2SP_B200_NO_X3TM") != nullptr;
    e->no_tm128 = getenv("T2SP_B200_NO_TM128") != nullptr;
    e->no_presplit = getenv("T2SP_B200_NO_PRESPLIT") != nullptr;
    if (const char* f = getenv("T2SP_B200_SPLITK")) e->splitk = std::max(1, atoi(f));
    e->precision = T2SP_PRECISION_TF32X3;
    if (const char* p = getenv("T2SP_B200_PRECISION")) {
        if (strcmp(p, "tf32") == 0) e->precision = T2SP_PRECISION_TF32;
        else if (strcmp(p, "tf32x3") != 0 && strcmp(p, "") != 0)
            fprintf(stderr, "t2sp_b200: unknown T2SP_B200_PRECISION '%s', using tf32x3\n", p);
    }
    if (const char* g = getenv("T2SP_B200_GROUP_M")) e->group_m = std::max(1, atoi(g));
    if (const char* p2 = getenv("T2SP_B200_PAIR2")) e->pair2 = atoi(p2) != 0 ? 1 : 0;
    if (const char* lim = getenv("T2SP_B200_FAIL_ALLOC_ABOVE")) e->fail_alloc_above = std::max(1ull, strtoull(lim, nullptr, 10));
    if (const char* w = getenv("T2SP_B200_WAIT_CYCLES")) e->wait_cycles = std::max(0ll, atoll(w));
    if (const char* k = getenv("T2SP_B200_TEST_SKIP_STAGE")) e->test_skip_stage = std::max(0, atoi(k));
    if (const char* bs = getenv("BITSTREAM")) {
        std::string b(bs);
        size_t pos = b.find_last_of('/');
        e->exec_time_path = (pos == std::string::npos ? std::string(".") : b.substr(0, pos)) + "/exec_time.txt";
    } else if (const char* f = getenv("T2SP_B200_EXEC_TIME_FILE")) {
        e->exec_time_path = f;
    }
    return e;
}

Slot* make_slot() {
    Slot* s = new Slot;
    if (cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&s->status_dev, sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(s->status_dev, 0, sizeof(unsigned)) != cudaSuccess ||
        cudaMallocHost(&s->status_host, sizeof(unsigned)) != cudaSuccess ||
        cudaEventCreate(&s->ev0) != cudaSuccess || cudaEventCreate(&s->ev1) != cudaSuccess) {
        cudaGetLastError();
        delete s;  // what was created stays with the context; this path means the device is out of resources
        return nullptr;
    }
    *s->status_host = 0;
    return s;
}

Slot* cur_slot() {
    ThreadState& ts = tls();
    return ts.slot[ts.device];
}

}  // namespace

const Env& rt_env() {
    const Env* e = g_env.load(std::memory_order_acquire);
    if (!e) {
        const Env* fresh = read_env();
        if (g_env.compare_exchange_strong(e, fresh, std::memory_order_acq_rel)) e = fresh;
        else delete fresh;
    }
    return *e;
}

ThreadState& tls() {
    static thread_local ThreadState st;
    return st;
}

ThreadState::~ThreadState() {
    // hand this thread's slots to whoever comes next; no CUDA call here (the thread may be ending with the process)
    std::lock_guard<std::mutex> lk(g_mu);
    for (int d = 0; d < kMaxDevices; ++d)
        if (slot[d]) {
            g_dev[d].idle_slots.push_back(slot[d]);
            slot[d] = nullptr;
        }
}

int rt_ensure_device() {
    ThreadState& ts = tls();
    if (ts.device < 0 || ts.device >= kMaxDevices) return halide_error_code_device_interface_no_device;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& d = g_dev[ts.device];
    if (d.init_error) return d.init_error;
    if (!d.ready) {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || ts.device >= count) {
            cudaGetLastError();
            fprintf(stderr, "t2sp_b200: no CUDA device %d is available; this library has no CPU path\n", ts.device);
            return halide_error_code_device_interface_no_device;  // not latched: a later call may find a device
        }
    }
    if (cudaSetDevice(ts.device) != cudaSuccess) return halide_error_code_device_interface_no_device;
    if (!d.ready) {
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
        d.ready = true;
    }
    if (!ts.slot[ts.device]) {
        Slot* s = nullptr;
        if (!d.idle_slots.empty()) {
            s = d.idle_slots.back();
            d.idle_slots.pop_back();
        } else {
            s = make_slot();
        }
        if (!s) return halide_error_code_device_malloc_failed;
        ts.slot[ts.device] = s;
    }
    return 0;
}

cudaStream_t rt_stream() {
    ThreadState& ts = tls();
    if (ts.has_user_stream) return ts.user_stream;
    return cur_slot()->stream;
}

unsigned* rt_status_word() { return cur_slot()->status_dev; }

cudaEvent_t rt_event(int which) { return which ? cur_slot()->ev1 : cur_slot()->ev0; }

bool rt_side_resources(cudaStream_t* h2d, cudaStream_t* d2h, cudaEvent_t** pool, int* pool_size) {
    Slot& d = *cur_slot();
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
    Slot& d = *cur_slot();
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
    const unsigned long long lim = rt_env().fail_alloc_above;
    if (lim && want >= lim) return nullptr;
    DeviceState& d = g_dev[tls().device];
    const cudaStream_t cur = rt_stream();
    {
        std::unique_lock<std::mutex> lk(g_mu);
        // the smallest block that fits, preferring one this stream used last (no wait needed)
        auto pick = d.free_blocks.end();
        for (auto it = d.free_blocks.lower_bound(want); it != d.free_blocks.end() && it->first <= want * 2; ++it) {
            if (pick == d.free_blocks.end()) pick = it;
            if (it->second.second.stream == cur) { pick = it; break; }
        }
        if (pick != d.free_blocks.end()) {
            void* p = pick->second.first;
            Block blk = pick->second.second;
            d.free_blocks.erase(pick);
            d.live_blocks[p] = blk;
            lk.unlock();
            // work the previous stream had queued when it released the block must finish first
            if (blk.stream != cur && blk.released) cudaStreamWaitEvent(cur, blk.released, 0);
            return p;
        }
    }
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        // Return cached blocks to the driver and retry once.
        {
            std::lock_guard<std::mutex> lk(g_mu);
            cudaDeviceSynchronize();
            for (auto& kv : d.free_blocks) {
                cudaFree(kv.second.first);
                if (kv.second.second.released) cudaEventDestroy(kv.second.second.released);
            }
            d.free_blocks.clear();
        }
        if (cudaMalloc(&p, want) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
    }
    std::lock_guard<std::mutex> lk(g_mu);
    Block blk;
    blk.size = want;
    d.live_blocks[p] = blk;
    return p;
}

void rt_free(void* p) {
    if (!p) return;
    DeviceState& d = g_dev[tls().device];
    const cudaStream_t cur = rt_stream();
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = d.live_blocks.find(p);
    if (it == d.live_blocks.end()) return;
    Block blk = it->second;
    d.live_blocks.erase(it);
    // Everything this thread queued on its stream so far may still use the block: whoever takes it over
    // on another stream waits for this point of the stream.
    if (!blk.released && cudaEventCreateWithFlags(&blk.released, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        blk.released = nullptr;
        cudaStreamSynchronize(cur);
    }
    if (blk.released) cudaEventRecord(blk.released, cur);
    blk.stream = cur;
    d.free_blocks.emplace(blk.size, std::make_pair(p, blk));
}

void rt_release_all() {
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < kMaxDevices; ++i) {
        DeviceState& d = g_dev[i];
        if (!d.ready) continue;
        cudaSetDevice(i);
        cudaDeviceSynchronize();
        for (auto& kv : d.free_blocks) {
            cudaFree(kv.second.first);
            if (kv.second.second.released) cudaEventDestroy(kv.second.second.released);
        }
        d.free_blocks.clear();
    }
    const ThreadState& ts = tls();
    if (ts.device >= 0 && ts.device < kMaxDevices && g_dev[ts.device].ready) cudaSetDevice(ts.device);
}

void rt_count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n)); }
uint64_t rt_launch_count() { return g_launches.load(); }

bool rt_encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, bool atom32, bool promote256, int swizzle_bytes) {
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
    CUtensorMapSwizzle sw = atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
    else if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
    else if (swizzle_bytes == 0) sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = g_encode(out, dtype, static_cast<cuuint32_t>(rank), base, gdim, gstr, bdim, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          promote256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (rt_env().log)
            fprintf(stderr, "t2sp_b200: cuTensorMapEncodeTiled failed (%d) rank=%d base=%p dims0=%llu box0=%u\n", (int)r,
                    rank, base, (unsigned long long)dims[0], box[0]);
        return false;
    }
    return true;
}

void rt_write_exec_time(const char* kernel_name, double ns) {
    // Same format as the reference runtime's exec_time.txt: first line the overall time, then
    // one "<kernel> <ns>" line per kernel (AOT-OpenCL-Runtime.cpp:380-395, read by Roofline.cpp:113-140).
    const std::string& path = rt_env().exec_time_path;
    if (path.empty()) return;
    if (FILE* fp = fopen(path.c_str(), "w")) {
        fprintf(fp, "%.0f\n%s %.0f\nkernel_unloader %.0f\n", ns, kernel_name, ns, ns);
        fclose(fp);
    }
}

// ------------------------------------------------------------------ buffer movement
namespace {

size_t elem_bytes(const halide_buffer_t* b) { return (b->type.bits + 7) / 8; }
size_t span_bytes(const halide_buffer_t* b) { return static_cast<size_t>(buf_elems_span(b)) * elem_bytes(b); }

// The elements inside a buffer's extents as a set of pitched 2-D pieces: every piece is `rows` runs of
// `run` consecutive elements, `pitch` elements apart; one piece per index of the outer dimensions that
// are left after adjacent dimensions have been merged.
struct Region {
    bool ok = false;      // strides are positive and the innermost run is contiguous
    bool dense = false;   // the region is the whole address span: one plain copy moves it
    int64_t run = 1, pitch = 1, rows = 1;
    int nouter = 0;
    int64_t oext[16] = {}, ostr[16] = {};
    int64_t pieces = 1;
};

Region region_of(const halide_buffer_t* b) {
    Region r;
    struct G { int64_t stride, extent; };
    G g[16];
    int n = 0;
    for (int d = 0; d < b->dimensions && d < 16; ++d) {
        if (b->dim[d].extent <= 0) { r.ok = true; r.dense = true; r.pieces = 0; return r; }
        if (b->dim[d].extent == 1) continue;
        if (b->dim[d].stride <= 0) return r;
        g[n++] = {b->dim[d].stride, b->dim[d].extent};
    }
    std::sort(g, g + n, [](const G& x, const G& y) { return x.stride < y.stride; });
    G m[16];
    int k = 0;
    for (int i = 0; i < n; ++i) {
        if (k > 0 && g[i].stride == m[k - 1].stride * m[k - 1].extent) m[k - 1].extent *= g[i].extent;
        else m[k++] = g[i];
    }
    if (k > 0 && m[0].stride != 1) return r;
    r.ok = true;
    r.dense = k <= 1;
    if (k > 0) r.run = m[0].extent;
    r.pitch = r.run;
    if (k > 1) { r.pitch = m[1].stride; r.rows = m[1].extent; }
    for (int i = 2; i < k; ++i) {
        r.oext[r.nouter] = m[i].extent;
        r.ostr[r.nouter] = m[i].stride;
        r.pieces *= m[i].extent;
        r.nouter++;
    }
    return r;
}

// Calls f(element offset of the piece) for every piece of the region; stops at the first false.
template <class F>
bool for_each_piece(const Region& r, F f) {
    int64_t idx[16] = {};
    for (int64_t n = 0; n < r.pieces; ++n) {
        int64_t off = 0;
        for (int i = 0; i < r.nouter; ++i) off += idx[i] * r.ostr[i];
        if (!f(off)) return false;
        for (int i = 0; i < r.nouter; ++i) {
            if (++idx[i] < r.oext[i]) break;
            idx[i] = 0;
        }
    }
    return true;
}

constexpr int64_t kMaxPieces = 256;  // beyond this a padded buffer travels as its whole span

bool copy_region(const halide_buffer_t* b, const Region& r, void* dev, uint8_t* host, bool to_host, cudaStream_t s) {
    const size_t es = elem_bytes(b);
    return for_each_piece(r, [&](int64_t off) {
        char* d = static_cast<char*>(dev) + off * es;
        uint8_t* h = host + off * es;
        const cudaError_t e = to_host ? cudaMemcpy2DAsync(h, r.pitch * es, d, r.pitch * es, r.run * es, r.rows, cudaMemcpyDeviceToHost, s)
                                      : cudaMemcpy2DAsync(d, r.pitch * es, h, r.pitch * es, r.run * es, r.rows, cudaMemcpyHostToDevice, s);
        return e == cudaSuccess;
    });
}

// Moves a buffer's content between its host memory and `dev`: the region alone when it is a few pitched
// pieces (what lies between the rows of a padded buffer, or beside a crop, is left alone), else the span.
bool move_buffer(const halide_buffer_t* b, void* dev, size_t bytes, bool to_host, cudaStream_t s) {
    const Region r = region_of(b);
    if (r.ok && !r.dense && r.pieces <= kMaxPieces) return copy_region(b, r, dev, b->host, to_host, s);
    if (bytes == 0) return true;
    return (to_host ? cudaMemcpyAsync(b->host, dev, bytes, cudaMemcpyDeviceToHost, s)
                    : cudaMemcpyAsync(dev, b->host, bytes, cudaMemcpyHostToDevice, s)) == cudaSuccess;
}
bool upload(const halide_buffer_t* b, void* dev, size_t bytes, cudaStream_t s) { return move_buffer(b, dev, bytes, false, s); }

}  // namespace

bool rt_move_buffer(const halide_buffer_t* b, bool to_host) {
    return move_buffer(b, reinterpret_cast<void*>(b->device), span_bytes(b), to_host, rt_stream());
}

void rt_zero_region(const halide_buffer_t* b, void* dev) {
    const Region r = region_of(b);
    const size_t es = elem_bytes(b);
    cudaStream_t s = rt_stream();
    if (!r.ok || r.dense) {
        // dense, or a layout whose padding cannot be told apart cheaply (non-positive strides)
        cudaMemsetAsync(dev, 0, span_bytes(b), s);
        return;
    }
    for_each_piece(r, [&](int64_t off) {
        return cudaMemset2DAsync(static_cast<char*>(dev) + off * es, r.pitch * es, 0, r.run * es, r.rows, s) == cudaSuccess;
    });
}

int rt_input_view(halide_buffer_t* b, const char* name, DeviceView* v) {
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
    if (!upload(b, v->ptr, v->bytes, rt_stream())) {
        cudaGetLastError();
        rt_drop_view(v);
        return halide_error_code_copy_to_device_failed;
    }
    if (v->borrowed) b->flags &= ~uint64_t(1);
    return 0;
}

int rt_output_view(halide_buffer_t* b, const char* name, DeviceView* v) {
    v->bytes = span_bytes(b);
    v->preloaded = false;
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
    // A padded output whose region cannot go back as a few pitched copies goes back as its whole span:
    // bring the host's bytes up first so that the padding returns unchanged.
    const Region r = region_of(b);
    if (!r.dense && (!r.ok || r.pieces > kMaxPieces) && b->host && v->bytes) {
        if (cudaMemcpyAsync(v->ptr, b->host, v->bytes, cudaMemcpyHostToDevice, rt_stream()) != cudaSuccess) {
            cudaGetLastError();
            rt_drop_view(v);
            return halide_error_code_copy_to_device_failed;
        }
        v->preloaded = true;
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
    const Region r = region_of(b);
    bool ok = true;
    if (r.dense || v->preloaded || !r.ok || r.pieces > kMaxPieces)
        ok = v->bytes == 0 || cudaMemcpyAsync(b->host, v->ptr, v->bytes, cudaMemcpyDeviceToHost, rt_stream()) == cudaSuccess;
    else
        ok = copy_region(b, r, v->ptr, b->host, true, rt_stream());  // only what lies inside the extents
    if (!ok) {
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
void* halide_malloc(void*, size_t);
void halide_free(void*, void*);
}

namespace {

// ---- the device interface table (HalideRuntime.h:713-738). Halide::Runtime::Buffer calls through it
// (copy_to_host, device_free in its destructor, crops and slices: HalideBuffer.h:229-252,388,418,1615-1713).
// `device` is a plain CUDA device address, so a crop or a slice is the same allocation at an offset.
int di_device_malloc(void*, halide_buffer_t* b, const halide_device_interface_t*) { return t2sp_b200_device_malloc(b); }
int di_device_free(void*, halide_buffer_t* b) { return t2sp_b200_device_free(b); }
int di_device_sync(void*, halide_buffer_t*) { return t2sp_b200_sync(); }
void di_device_release(void*, const halide_device_interface_t*) { t2sp_b200_release(); }
int di_copy_to_host(void*, halide_buffer_t* b) {
    if (!b) return halide_error_code_buffer_argument_is_null;
    if (!(b->flags & 2u)) return 0;  // the host copy is current
    return t2sp_b200_copy_to_host(b);
}
int di_copy_to_device(void*, halide_buffer_t* b, const halide_device_interface_t*) {
    if (!b) return halide_error_code_buffer_argument_is_null;
    if (b->device && !(b->flags & 1u)) return 0;  // the device copy is current
    return t2sp_b200_copy_to_device(b);
}
int di_device_and_host_malloc(void* uc, halide_buffer_t* b, const halide_device_interface_t*) {
    if (!b) return halide_error_code_buffer_argument_is_null;
    b->host = static_cast<uint8_t*>(halide_malloc(uc, static_cast<size_t>(buf_elems_span(b)) * ((b->type.bits + 7) / 8)));
    if (!b->host) return halide_error_code_out_of_memory;
    const int rc = t2sp_b200_device_malloc(b);
    if (rc != 0) {
        halide_free(uc, b->host);
        b->host = nullptr;
    }
    return rc;
}
int di_device_and_host_free(void* uc, halide_buffer_t* b) {
    if (!b) return halide_error_code_buffer_argument_is_null;
    const int rc = t2sp_b200_device_free(b);
    if (b->host) {
        halide_free(uc, b->host);
        b->host = nullptr;
    }
    b->flags &= ~uint64_t(3);
    return rc;
}
// Same-shape copy between two buffers; either side may live on the host (dst_iface == NULL: the
// destination's host memory) or on this library's device.
int di_buffer_copy(void*, halide_buffer_t* src, const halide_device_interface_t* dst_iface, halide_buffer_t* dst) {
    if (!src || !dst) return halide_error_code_buffer_argument_is_null;
    if (dst_iface && dst_iface != t2sp_b200_device_interface()) return halide_error_code_device_buffer_copy_failed;
    if (src->dimensions != dst->dimensions || src->type.bits != dst->type.bits) return halide_error_code_device_buffer_copy_failed;
    for (int d = 0; d < src->dimensions; ++d)
        if (src->dim[d].extent != dst->dim[d].extent || src->dim[d].stride != dst->dim[d].stride)
            return halide_error_code_device_buffer_copy_failed;
    const bool from_dev = buf_on_our_device(src) && (!(src->flags & 1u) || !src->host);
    const bool to_dev = dst_iface != nullptr;
    if (!from_dev && !src->host) return halide_error_code_host_is_null;
    if (to_dev) {
        if (int e = t2sp_b200_device_malloc(dst)) return e;
        if (!buf_on_our_device(dst)) return halide_error_code_device_buffer_copy_failed;
    } else if (!dst->host) {
        return halide_error_code_host_is_null;
    }
    if (int e = rt_ensure_device()) return e;
    const size_t bytes = static_cast<size_t>(buf_elems_span(src)) * ((src->type.bits + 7) / 8);
    const void* from = from_dev ? reinterpret_cast<const void*>(src->device) : static_cast<const void*>(src->host);
    void* to = to_dev ? reinterpret_cast<void*>(dst->device) : static_cast<void*>(dst->host);
    if (bytes && (cudaMemcpyAsync(to, from, bytes, cudaMemcpyDefault, rt_stream()) != cudaSuccess ||
                  cudaStreamSynchronize(rt_stream()) != cudaSuccess)) {
        cudaGetLastError();
        return halide_error_code_device_buffer_copy_failed;
    }
    if (to_dev) { dst->flags |= 2u; dst->flags &= ~uint64_t(1); }
    else { dst->flags |= 1u; dst->flags &= ~uint64_t(2); }
    return 0;
}
int di_device_crop(void*, const halide_buffer_t* src, halide_buffer_t* dst) {
    if (!src || !dst) return halide_error_code_buffer_argument_is_null;
    if (!buf_on_our_device(src) || src->dimensions != dst->dimensions) return halide_error_code_device_buffer_copy_failed;
    int64_t off = 0;  // dst's shape is already the cropped one: the offset is where its mins sit inside src
    for (int d = 0; d < src->dimensions; ++d) off += int64_t(dst->dim[d].min - src->dim[d].min) * src->dim[d].stride;
    dst->device = src->device + off * ((src->type.bits + 7) / 8);
    dst->device_interface = src->device_interface;
    return 0;
}
int di_device_slice(void*, const halide_buffer_t* src, int slice_dim, int slice_pos, halide_buffer_t* dst) {
    if (!src || !dst) return halide_error_code_buffer_argument_is_null;
    if (!buf_on_our_device(src) || slice_dim < 0 || slice_dim >= src->dimensions || dst->dimensions != src->dimensions - 1)
        return halide_error_code_device_buffer_copy_failed;
    int64_t off = int64_t(slice_pos - src->dim[slice_dim].min) * src->dim[slice_dim].stride;
    for (int d = 0, e = 0; d < src->dimensions; ++d) {
        if (d == slice_dim) continue;
        off += int64_t(dst->dim[e].min - src->dim[d].min) * src->dim[d].stride;
        ++e;
    }
    dst->device = src->device + off * ((src->type.bits + 7) / 8);
    dst->device_interface = src->device_interface;
    return 0;
}
int di_device_release_crop(void*, halide_buffer_t* b) {
    if (!b) return halide_error_code_buffer_argument_is_null;
    b->device = 0;  // the allocation belongs to the buffer the crop was taken from
    b->device_interface = nullptr;
    return 0;
}
int di_wrap_native(void*, halide_buffer_t* b, uint64_t handle, const halide_device_interface_t*) {
    return t2sp_b200_wrap_device_ptr(b, handle);
}
int di_detach_native(void*, halide_buffer_t* b) { return t2sp_b200_detach_device_ptr(b); }
int di_compute_capability(void*, int* major, int* minor) {
    if (int e = rt_ensure_device()) return e;
    int dev = tls().device;
    if (cudaDeviceGetAttribute(major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess)
        return halide_error_code_device_interface_no_device;
    return 0;
}

const halide_device_interface_t g_interface = {
    di_device_malloc, di_device_free, di_device_sync, di_device_release, di_copy_to_host, di_copy_to_device,
    di_device_and_host_malloc, di_device_and_host_free, di_buffer_copy, di_device_crop, di_device_slice,
    di_device_release_crop, di_wrap_native, di_detach_native, di_compute_capability, nullptr};

}  // namespace

extern "C" {

const struct halide_device_interface_t* t2sp_b200_device_interface(void) { return &g_interface; }

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
    if (int e = rt_ensure_device()) return e;
    if (!rt_move_buffer(buf, false) || cudaStreamSynchronize(rt_stream()) != cudaSuccess) {
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
    if (!rt_move_buffer(buf, true) || cudaStreamSynchronize(rt_stream()) != cudaSuccess) {
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
    if (ordinal < 0 || ordinal >= kMaxDevices) return halide_error_code_device_interface_no_device;
    tls().device = ordinal;
    return 0;
}

int t2sp_b200_set_stream(void* cuda_stream) {
    ThreadState& ts = tls();
    ts.user_stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    ts.has_user_stream = cuda_stream != nullptr;
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

void t2sp_b200_reload_env(void) {
    g_env.store(read_env(), std::memory_order_release);  // the previous snapshot may still be in use by a call: not freed
}

void t2sp_b200_release(void) { rt_release_all(); }
uint64_t t2sp_b200_kernel_launches(void) { return rt_launch_count(); }
double t2sp_b200_last_kernel_ns(void) { return tls().last_kernel_ns; }
const char* t2sp_b200_version(void) { return "t2sp_b200 0.2 (sm_100a)"; }

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
