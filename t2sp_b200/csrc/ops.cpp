// The five operator entry points: argument validation in the order the generated host
// code performs it (null -> bounds query -> type -> dimensions -> extents -> output coverage
// -> innermost stride -> sizes -> host pointer; t2s/peppers/blas/level3/syrk/release/s10/
// syrk-interface.cpp:29-928), then lowering to one launch of the contraction kernel.
// The host serializer/deserializer loops of the reference (syrk-interface.cpp:976-1240,
// 2143-2317) have no counterpart: TMA strides and the epilogue's address maps read and write
// the caller's layouts in place.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "host_rt.h"

extern "C" {
int halide_error_bad_type(void*, const char*, uint32_t, uint32_t);
int halide_error_bad_dimensions(void*, const char*, int32_t, int32_t);
int halide_error_access_out_of_bounds(void*, const char*, int, int, int, int, int);
int halide_error_buffer_allocation_too_large(void*, const char*, uint64_t, uint64_t);
int halide_error_buffer_extents_negative(void*, const char*, int, int);
int halide_error_buffer_extents_too_large(void*, const char*, int64_t, int64_t);
int halide_error_constraint_violated(void*, const char*, int, const char*, int);
int halide_error_buffer_argument_is_null(void*, const char*);
int halide_error_host_is_null(void*, const char*);
}

namespace t2sp {
cudaEvent_t rt_event(int which);

namespace {

constexpr uint32_t type_word(int code, int bits) { return uint32_t(code) | (uint32_t(bits) << 8) | (1u << 16); }
constexpr uint32_t kF32 = type_word(2, 32), kBF16 = type_word(4, 16), kF16 = type_word(2, 16), kI8 = type_word(0, 8),
                   kI32 = type_word(0, 32);

uint32_t buf_type_word(const halide_buffer_t* b) {
    uint32_t w;
    memcpy(&w, &b->type, 4);
    return w;
}

struct Arg {
    halide_buffer_t* b;
    const char* name;   // "A"
    bool is_output;
    int dims;
    std::string role() const { return std::string(is_output ? "Output buffer " : "Input buffer ") + name; }
};

// Fills a bounds-query buffer with a dense shape of the given extents.
void fill_query(halide_buffer_t* b, uint32_t tword, int dims, const int* ext) {
    memcpy(&b->type, &tword, 4);
    b->dimensions = dims;
    int64_t stride = 1;
    for (int d = 0; d < dims; ++d) {
        b->dim[d].min = 0;
        b->dim[d].extent = ext[d];
        b->dim[d].stride = static_cast<int32_t>(stride);
        b->dim[d].flags = 0;
        stride *= ext[d];
    }
}

int check_null(const Arg* args, int n) {
    // the generated code tests the output first, then the inputs last to first
    for (int i = n - 1; i >= 0; --i)
        if (!args[i].b) return halide_error_buffer_argument_is_null(nullptr, args[i].name);
    return 0;
}

int check_type_dims(const Arg& a, uint32_t want) {
    if (buf_type_word(a.b) != want) return halide_error_bad_type(nullptr, a.role().c_str(), buf_type_word(a.b), want);
    if (a.b->dimensions != a.dims)
        return halide_error_bad_dimensions(nullptr, a.role().c_str(), a.b->dimensions, a.dims);
    return 0;
}

int check_extents_nonneg(const Arg& a) {
    for (int d = 0; d < a.b->dimensions; ++d)
        if (a.b->dim[d].extent < 0)
            return halide_error_buffer_extents_negative(nullptr, a.role().c_str(), d, a.b->dim[d].extent);
    return 0;
}

// The buffer must cover [0, need-1] in dimension d.
int check_covers(const Arg& a, int d, int need) {
    const int mn = a.b->dim[d].min, mx = mn + a.b->dim[d].extent - 1;
    if (mn > 0 || mx < need - 1)
        return halide_error_access_out_of_bounds(nullptr, a.role().c_str(), d, 0, need - 1, mn, mx);
    return 0;
}

int check_stride0(const Arg& a) {
    if (a.b->dim[0].stride != 1) {
        std::string v = std::string(a.name) + ".stride.0";
        return halide_error_constraint_violated(nullptr, v.c_str(), a.b->dim[0].stride, "1", 1);
    }
    return 0;
}

int check_sizes(const Arg& a) {
    const int64_t span = buf_elems_span(a.b);
    const int64_t bytes = span * ((a.b->type.bits + 7) / 8);
    // The reference caps a buffer at 2^31-1 bytes because its indices are 32-bit
    // (syrk-interface.cpp:368-432); here indices are 64-bit and the cap is the 2^31-1 limit
    // of Halide's int32 extents and strides themselves.
    int64_t prod = 1;
    for (int d = 0; d < a.b->dimensions; ++d) {
        prod *= std::max(a.b->dim[d].extent, 1);
        if (prod > (int64_t(1) << 40))
            return halide_error_buffer_extents_too_large(nullptr, a.name, prod, int64_t(1) << 40);
    }
    if (bytes > (int64_t(1) << 40))
        return halide_error_buffer_allocation_too_large(nullptr, a.name, bytes, uint64_t(1) << 40);
    return 0;
}

int check_host(const Arg& a) {
    if (!a.b->host && !buf_on_our_device(a.b)) return halide_error_host_is_null(nullptr, a.role().c_str());
    return 0;
}

int constraint(const char* var, int val, const char* want_name, int want) {
    return halide_error_constraint_violated(nullptr, var, val, want_name, want);
}

// Offset (elements) from the buffer's first stored element to coordinate 0 in every dimension.
int64_t origin_offset(const halide_buffer_t* b) {
    int64_t off = 0;
    for (int d = 0; d < b->dimensions; ++d) off -= int64_t(b->dim[d].min) * b->dim[d].stride;
    return off;
}

bool tma_ok(const void* base, std::initializer_list<int64_t> strides_bytes) {
    if (reinterpret_cast<uintptr_t>(base) & 15) return false;
    for (int64_t s : strides_bytes)
        if (s <= 0 || (s & 15)) return false;
    return true;
}

int tma_unsupported(const char* name) {
    fprintf(stderr,
            "t2sp_b200: buffer %s cannot be read by TMA in place (base address and every outer stride must be "
            "16-byte aligned)\n",
            name);
    return halide_error_code_constraint_violated;
}

// Row-major fp32/int32 output [M][N] with row pitch `ld` elements: use the TMA-store epilogue when
// the pitch and base allow a tensor map, otherwise plain vector stores.
void set_rowmajor_epilogue(CoreParams& p, void* out, int M, int N, int64_t ld) {
    p.epi = EPI_ROWMAJOR;
    p.ldo = ld;
    if (rt_env().no_tma_store) return;
    if (p.tile_rows != kBlockM) return;  // a warp's 32-row store would spill into the next tile's rows
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (ld * 4) % 16 || ld <= 0) return;
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)}, str[2] = {4, uint64_t(ld) * 4};
    uint32_t box[2] = {32, 32};
    if (rt_encode_tmap(&p.mapC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, str, box)) p.epi = EPI_TMA;
}

// Column-major fp32 output (element (m, n) at m + n * ld): the TMA-store epilogue with a transposed staging tile
// when the pitch and base allow a tensor map, otherwise one plain store instruction per column.
void set_colmajor_epilogue(CoreParams& p, void* out, long long M, int N, int64_t ld) {
    p.epi = EPI_COLMAJOR;
    p.ldo = ld;
    p.tma_t = 0;
    if (rt_env().no_tma_store) return;
    if (p.tile_rows != kBlockM) return;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (ld * 4) % 16 || ld <= 0 || M <= 0 || N <= 0) return;
    uint64_t dims[2] = {uint64_t(M), uint64_t(N)}, str[2] = {4, uint64_t(ld) * 4};
    uint32_t box[2] = {32, 32};
    if (rt_encode_tmap(&p.mapC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, str, box, false, true, 0)) {
        p.epi = EPI_TMA;
        p.tma_t = 1;
    }
}

void add_digit2(Digits& d, int div, int mod, int div2, int mod2, long long stride) {
    if (d.n >= kMaxDigits) return;
    d.div[d.n] = div;
    d.mod[d.n] = mod <= 0 ? 1 : mod;
    d.div2[d.n] = div2;
    d.mod2[d.n] = mod2 <= 0 ? 1 : mod2;
    d.stride[d.n] = stride;
    d.n++;
}
void add_digit(Digits& d, int div, int mod, long long stride) { add_digit2(d, div, mod, 1, 1 << 30, stride); }

// fp32 contractions move to CTA pairs (256 x 256 or 256 x 128 tiles) when such tiles, cut along the
// contraction where that pays (x3_pick_splits), occupy most SM pairs; returns the pair tile width or 0.
int x3_pick_splits(int tiles, int total_kb, bool scatter = false);
int x3_pair_width(long long M, int N, int tile_rows, int num_kb, bool tm128 = false) {
    // 256 x 128 pair tiles did not beat the single-CTA kernel (capsule, N = 128: 133 us vs 108 us), so
    // pairs are used for wide outputs only unless $T2SP_B200_PAIR128 asks otherwise.
    if (rt_env().no_pair || tile_rows != kBlockM || N < 128) return 0;
    // (tm128: the caller would run the 128-column form of the tensor-memory kernel, which is another matter)
    if (N <= 128 && !rt_env().pair128 && !tm128) return 0;
    const int un = N > 128 ? 256 : 128;
    const long long tiles = ((M + 255) / 256) * ((N + un - 1) / un);
    if (tiles > (1 << 20)) return un;
    return tiles * x3_pick_splits(static_cast<int>(tiles), num_kb) >= core_sm_count() / 4 ? un : 0;
}

// How many ranges to cut the contraction of an fp32 pair launch into: the one that minimises
// (waves of work items) x (k-blocks per item) plus the cost of the summing pass, counted in
// k-block times; 1 when the tiles already fill the SM pairs or the contraction is short.
int x3_pick_splits(int tiles, int total_kb, bool scatter) {
    if (rt_env().no_splitk || total_kb <= 1) return 1;
    if (rt_env().splitk) {  // forced number of ranges (tests)
        const int s = std::max(1, std::min(rt_env().splitk, total_kb));
        const int per = (total_kb + s - 1) / s;
        return (total_kb + per - 1) / per;
    }
    const int pairs = std::max(1, core_sm_count() / 2);
    int best = 1;
    long long best_cost = static_cast<long long>((tiles + pairs - 1) / pairs) * total_kb;
    for (int s = 2; s <= 8; ++s) {
        const int per = (total_kb + s - 1) / s;
        if (per < 8) break;
        const int eff = (total_kb + per - 1) / per;
        const long long waves = (static_cast<long long>(tiles) * eff + pairs - 1) / pairs;
        // the summing pass decodes a mixed-radix address per element for the tiled layouts: measured
        // about 30 k-block times dearer than the row-major one at the published conv size
        const long long cost = waves * per + 8 + eff + (scatter ? 32 : 0);
        if (cost < best_cost) { best_cost = cost; best = eff; }
    }
    return best;
}

int resolve_precision(int p) {
    if (p == T2SP_PRECISION_DEFAULT) return rt_env().precision;
    return p == T2SP_PRECISION_TF32 ? T2SP_PRECISION_TF32 : T2SP_PRECISION_TF32X3;
}

// Cuts the row space (ext[0] fastest) into TMA boxes: whole leading dimensions, then a divisor
// of the first dimension that does not fit. box[] gets the box extents.
void plan_rows(RowSpace& rs, int* box) {
    int remaining = kBlockM;
    int rows = 1;
    bool partial = false;
    for (int d = 0; d < rs.nd; ++d) {
        int b = 1;
        if (!partial) {
            for (int c = std::min(rs.ext[d], remaining); c >= 1; --c)
                if (rs.ext[d] % c == 0) { b = c; break; }
            if (b < rs.ext[d]) partial = true;
            remaining /= b;
        }
        box[d] = b;
        rows *= b;
    }
    rs.rows_per_box = rows;
    rs.boxes_per_tile = std::max(1, kBlockM / rows);
}

struct Timing {
    bool on = false;
};

// Runs one lowered contraction: launch, optional timing, status check.
int run_core(const char* who, int arith, int op, int bn, CoreParams& p, bool sync_after, bool pair = false,
             bool pair2 = false) {
    ThreadState& ts = tls();
    cudaStream_t s = rt_stream();
    p.status = rt_status_word();
    p.wait_cycles = rt_env().wait_cycles;
    p.skip_stage = rt_env().test_skip_stage;
    if (p.group_m <= 0) p.group_m = pair ? 8 : 16;
#ifdef T2SP_DEBUG_KNOBS
    static long long* trace_dev = nullptr;
    const char* trace_path = getenv("T2SP_B200_TRACE");
    p.trace = nullptr;
    if (trace_path) {
        if (!trace_dev) cudaMalloc(&trace_dev, 48 * 1024 * sizeof(long long));
        cudaMemsetAsync(trace_dev, 0, 48 * 1024 * sizeof(long long), s);
        p.trace = trace_dev;
    }
#endif
    if (rt_env().group_m) p.group_m = rt_env().group_m;
    const int tiles = p.tiles_m * p.tiles_n;
    // fp32 pair kernel with fewer tiles than SM pairs: cut the contraction into ranges that run as
    // work items of their own, partial tiles go to scratch and a second kernel sums them in order
    // and applies the call's real epilogue.
    float* partials = nullptr;
    CoreParams final_p;
    int slab_rows = 0, ld_part = 0;
    if (pair && arith == AR_TF32X3) {
        const int splits = x3_pick_splits(tiles, p.total_kb, p.epi == EPI_SCATTER);
        if (splits > 1) {
            slab_rows = p.tiles_m * 256;
            ld_part = p.tiles_n * bn;
            partials = static_cast<float*>(rt_alloc(size_t(splits) * slab_rows * ld_part * sizeof(float)));
            if (!partials) return halide_error_code_device_malloc_failed;
            final_p = p;
            if (final_p.epi == EPI_TMA) final_p.epi = final_p.tma_t ? EPI_COLMAJOR : EPI_ROWMAJOR;
            p.tma_t = 0;  // the partial tiles are row-major
            uint64_t dims[2] = {uint64_t(ld_part), uint64_t(splits) * slab_rows}, str[2] = {4, uint64_t(ld_part) * 4};
            uint32_t box[2] = {32, 32};
            if (!rt_encode_tmap(&p.mapC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, partials, dims, str, box)) {
                rt_free(partials);
                return halide_error_code_device_run_failed;
            }
            p.epi = EPI_TMA;
            p.out = partials;
            p.ldo = ld_part;
            p.use_ab = 0;
            p.num_kb = (p.total_kb + splits - 1) / splits;
            p.splits = (p.total_kb + p.num_kb - 1) / p.num_kb;
            p.slab_rows = slab_rows;
            p.M = p.splits * slab_rows;  // the kernel's store guard now covers the partial slabs
            p.N = ld_part;
        }
    }
    const int items = tiles * std::max(1, (pair && arith == AR_TF32X3) ? p.splits : 1);
    int grid = std::max(1, std::min(tiles, core_sm_count()));
    if (pair) grid = 2 * std::max(1, std::min(items, core_sm_count() / 2));  // one cluster of 2 CTAs per work item slot
    if (sync_after) cudaEventRecord(rt_event(0), s);
    cudaError_t e = !pair ? core_launch(arith, op, bn, p, grid, s)
                          : (arith == AR_TF32X3 ? (p.b_pre ? x3tm_launch(op, bn, p, grid, s) : x3pair_launch(op, bn, p, grid, s))
                                                : (pair2 ? pair2_launch(arith, op, p, grid, s) : pair_launch(arith, op, p, grid, s)));
    if (e == cudaSuccess && partials) {
        e = splitk_finalize_launch(partials, ld_part, slab_rows, p.splits, final_p, s);
        rt_count_launch(1);
    }
    // stream order keeps the scratch block safe for whoever gets it next on this stream
    if (partials) rt_free(partials);
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200: %s: kernel launch failed: %s\n", who, cudaGetErrorString(e));
        return halide_error_code_device_run_failed;
    }
    rt_count_launch(1);
    if (sync_after) cudaEventRecord(rt_event(1), s);
#ifdef T2SP_DEBUG_KNOBS
    // T2SP_B200_TRACE_AT=<n>: only the n-th traced launch is waited for and written out, so that the
    // launches before it run back to back as in a timed loop
    static int trace_calls = 0;
    const char* trace_at = getenv("T2SP_B200_TRACE_AT");
    if (trace_path && (!trace_at || ++trace_calls == atoi(trace_at))) {
        std::vector<long long> host(48 * 1024);
        cudaStreamSynchronize(s);
        cudaMemcpy(host.data(), trace_dev, host.size() * sizeof(long long), cudaMemcpyDeviceToHost);
        if (FILE* f = fopen(trace_path, "wb")) { fwrite(host.data(), sizeof(long long), host.size(), f); fclose(f); }
    }
#endif
    (void)ts;
    return 0;
}

int finish_call(const char* who, const char* kernel_name, bool sync_after) {
    if (!sync_after) return 0;
    int rc = rt_check_status(who);
    if (rc) return rc;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, rt_event(0), rt_event(1)) == cudaSuccess) {
        tls().last_kernel_ns = double(ms) * 1e6;
        rt_write_exec_time(kernel_name, tls().last_kernel_ns);
    }
    if (rt_env().log) fprintf(stderr, "t2sp_b200: %s: kernels %.1f us\n", who, tls().last_kernel_ns * 1e-3);
    return 0;
}

bool all_resident(std::initializer_list<const halide_buffer_t*> bufs) {
    for (auto* b : bufs)
        if (!buf_on_our_device(b) || ((b->flags & 1u) && b->host)) return false;
    return true;
}

struct Views {
    DeviceView v[8];
    int n = 0;
    ~Views() {
        for (int i = 0; i < n; ++i) rt_drop_view(&v[i]);
    }
};

// TMA needs a 16-byte aligned base and row pitch. A 2-D operand that does not have them is copied
// once, on the device, into a scratch block with a padded pitch (cudaMemcpy2DAsync), and the kernel
// reads the copy. `ptr` / `ld_bytes` are updated in place.
int repack_if_unaligned(Views& vw, char*& ptr, int64_t& ld_bytes, int64_t row_bytes, int64_t rows) {
    if (tma_ok(ptr, {ld_bytes}) || rows <= 0 || row_bytes <= 0) return 0;
    const int64_t pitch = (row_bytes + 15) / 16 * 16;
    void* q = rt_alloc(size_t(pitch) * rows);
    if (!q) return halide_error_code_device_malloc_failed;
    vw.v[vw.n].ptr = q; vw.v[vw.n].borrowed = false; vw.n++;
    if (pitch != row_bytes) cudaMemsetAsync(q, 0, size_t(pitch) * rows, rt_stream());
    if (cudaMemcpy2DAsync(q, pitch, ptr, ld_bytes, row_bytes, rows, cudaMemcpyDeviceToDevice, rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        return halide_error_code_device_run_failed;
    }
    ptr = static_cast<char*>(q);
    ld_bytes = pitch;
    return 0;
}

// fp32 pair kernel with 256-column tiles (umma_x3tm.cuh): is B worth a pre-pass? Only when many row tiles re-read it
// (the pre-pass costs a launch and a read and write of B) and full precision is asked for.
bool presplit_worthwhile(int un, int prec, long long M, long long b_bytes) {
    return (un == 256 || un == 128) && prec != T2SP_PRECISION_TF32 && !rt_env().no_x3tm && !rt_env().no_presplit && (M + 255) / 256 >= 16 &&
           b_bytes > 0 && b_bytes <= (256ll << 20);
}
// Runs the pre-pass that writes B's slot images into scratch and points the kernel at them. Leaves p.b_pre = 0 (the
// kernel then loads B through mapB and splits it itself) when anything is in the way.
void prepack_b(Views& vw, CoreParams& p, BImageParams q, int un, int n_extent) {
    q.halves = 2 * ((n_extent + un - 1) / un);
    q.half_cols = un / 2;
    const size_t bytes = size_t(q.num_kb) * q.halves * q.half_cols * 256;
    if (vw.n >= 8 || bytes == 0 || bytes > (size_t(512) << 20)) return;
    void* scratch = rt_alloc(bytes);
    if (!scratch) return;
    vw.v[vw.n].ptr = scratch; vw.v[vw.n].borrowed = false; vw.n++;
    if (b_images_launch(q, scratch, rt_stream()) != cudaSuccess) { cudaGetLastError(); return; }
    rt_count_launch(1);
    p.b_images = scratch;
    p.b_halves = q.halves;
    p.b_pre = 1;
}

uint32_t idesc_for(int arith, uint32_t in_type, bool b_mn_major, int bn) {
    if (arith == AR_F16) return make_instr_desc(1, in_type == kBF16 ? 1 : 0, false, b_mn_major, kBlockM, bn);
    if (arith == AR_TF32X3) return make_instr_desc(1, 2, false, b_mn_major, kBlockM, bn);
    return make_instr_desc(2, 1, false, b_mn_major, kBlockM, bn);
}

CUtensorMapDataType tmap_type(uint32_t tword) {
    if (tword == kF32) return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    if (tword == kBF16) return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (tword == kF16) return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

int arith_for(uint32_t tword) {
    if (tword == kF32) return AR_TF32X3;
    if (tword == kI8) return AR_I8;
    return AR_F16;
}

int block_k_for(int arith) { return arith == AR_F16 ? 64 : (arith == AR_TF32X3 ? 32 : 128); }

}  // namespace
}  // namespace t2sp

using namespace t2sp;

// ======================================================================================= GEMM
namespace t2sp {
namespace {

// Large GEMM on host buffers: instead of "copy everything in, compute, copy everything out" the
// operands travel in slabs (rows of A, columns of B) on a host->device stream, every
// (row slab, column slab) block of C is computed as soon as its two slabs have arrived, and
// leaves on a device->host stream while later blocks are still being computed. PCIe is full
// duplex, so the call approaches max(bytes in, bytes out) / link rate instead of their sum.
// The blocks are ordinary calls of t2sp_b200_gemm on device-resident sub-buffers (same memory,
// shifted base, full pitch). Returns 1 if it handled the call, 0 if the caller should take the
// plain path, or a negative halide error.
int gemm_host_pipelined(halide_buffer_t* A, halide_buffer_t* B, halide_buffer_t* C, const t2sp_gemm_desc* desc,
                        int M, int N, int K, bool* done) {
    *done = false;
    if (rt_env().no_pipeline) return 0;
    if (desc && (desc->layout || desc->trans_a || desc->trans_b || desc->scale)) return 0;
    if (A->device || B->device || C->device) return 0;
    if (A->dim[0].min || A->dim[1].min || B->dim[0].min || B->dim[1].min || C->dim[0].min || C->dim[1].min) return 0;
    const int es = (A->type.bits + 7) / 8;
    const double bytes = double(M) * K * es + double(K) * N * es + double(M) * N * 4;
    if (bytes < 96e6 || M < 2048 || N < 2048) return 0;
    if ((int64_t(A->dim[1].stride) * es) % 16 || (int64_t(B->dim[1].stride) * es) % 16 || (N * es) % 16) return 0;
    cudaStream_t s_in, s_out, s_main = rt_stream();
    cudaEvent_t* ev;
    int nev;
    if (!rt_side_resources(&s_in, &s_out, &ev, &nev)) return 0;
    const int GM = 4, GN = 4;
    const int ms = ((M + GM - 1) / GM + 511) / 512 * 512, ns = ((N + GN - 1) / GN + 255) / 256 * 256;
    const int nm = (M + ms - 1) / ms, nn = (N + ns - 1) / ns;
    if (2 + nm + nn + nm * nn > nev) return 0;

    // dense device copies of A (pitch K), B (pitch N), C (pitch N)
    DeviceView va, vb, vc;
    va.ptr = rt_alloc(size_t(M) * K * es); vb.ptr = rt_alloc(size_t(K) * N * es); vc.ptr = rt_alloc(size_t(M) * N * 4);
    struct Guard { DeviceView *a, *b, *c; ~Guard() { rt_drop_view(a); rt_drop_view(b); rt_drop_view(c); } } guard{&va, &vb, &vc};
    if (!va.ptr || !vb.ptr || !vc.ptr) return halide_error_code_device_malloc_failed;
    char* dA = static_cast<char*>(va.ptr);
    char* dB = static_cast<char*>(vb.ptr);
    char* dC = static_cast<char*>(vc.ptr);

    cudaEvent_t e_start = ev[0], e_done = ev[1];
    cudaEvent_t* eA = ev + 2;
    cudaEvent_t* eB = eA + nm;
    cudaEvent_t* eC = eB + nn;
    cudaEventRecord(rt_event(0), s_main);
    cudaEventRecord(e_start, s_main);
    cudaStreamWaitEvent(s_in, e_start, 0);
    cudaStreamWaitEvent(s_out, e_start, 0);
    bool ok = true;
    auto copy_a = [&](int i) {
        const int r0 = i * ms, rows = std::min(ms, M - r0);
        ok &= cudaMemcpy2DAsync(dA + size_t(r0) * K * es, size_t(K) * es, A->host + size_t(r0) * A->dim[1].stride * es,
                                size_t(A->dim[1].stride) * es, size_t(K) * es, rows, cudaMemcpyHostToDevice, s_in) == cudaSuccess;
        cudaEventRecord(eA[i], s_in);
    };
    auto copy_b = [&](int j) {
        const int c0 = j * ns, cols = std::min(ns, N - c0);
        ok &= cudaMemcpy2DAsync(dB + size_t(c0) * es, size_t(N) * es, B->host + size_t(c0) * es, size_t(B->dim[1].stride) * es,
                                size_t(cols) * es, K, cudaMemcpyHostToDevice, s_in) == cudaSuccess;
        cudaEventRecord(eB[j], s_in);
    };
    // Arrival order: A and B slabs alternate (A0, B0, B1, A1, B2, A2, ...), so that after every slab
    // some new C blocks have both of their operands on the device; each of them is launched at once and
    // its result starts downstream while the next slabs are still coming up.
    ThreadState& ts = tls();
    const bool was_async = ts.async;
    ts.async = true;
    int rc = 0;
    std::vector<char> launched(size_t(nm) * nn, 0);
    int ua = 0, ub = 0;  // slabs of A / B uploaded so far
    auto launch_ready = [&]() {
        for (int i = 0; i < ua && rc == 0; ++i) {
            const int r0 = i * ms, rows = std::min(ms, M - r0);
            for (int j = 0; j < ub && rc == 0; ++j) {
                if (launched[size_t(i) * nn + j]) continue;
                launched[size_t(i) * nn + j] = 1;
                const int c0 = j * ns, cols = std::min(ns, N - c0);
                cudaStreamWaitEvent(s_main, eA[i], 0);
                cudaStreamWaitEvent(s_main, eB[j], 0);
                halide_dimension_t da[2] = {{0, K, 1, 0}, {0, rows, K, 0}};
                halide_dimension_t db[2] = {{0, cols, 1, 0}, {0, K, N, 0}};
                halide_dimension_t dc[2] = {{0, cols, 1, 0}, {0, rows, N, 0}};
                halide_buffer_t a = *A, b = *B, c = *C;
                a.host = b.host = c.host = nullptr;
                a.flags = b.flags = c.flags = 0;
                a.dim = da; b.dim = db; c.dim = dc;
                a.device = reinterpret_cast<uint64_t>(dA + size_t(r0) * K * es);
                b.device = reinterpret_cast<uint64_t>(dB + size_t(c0) * es);
                c.device = reinterpret_cast<uint64_t>(dC + (size_t(r0) * N + c0) * 4);
                a.device_interface = b.device_interface = c.device_interface = t2sp_b200_device_interface();
                rc = t2sp_b200_gemm(&a, &b, &c, desc);
                cudaEvent_t done_ij = eC[i * nn + j];
                cudaEventRecord(done_ij, s_main);
                cudaStreamWaitEvent(s_out, done_ij, 0);
                ok &= cudaMemcpy2DAsync(C->host + (size_t(r0) * C->dim[1].stride + c0) * 4, size_t(C->dim[1].stride) * 4,
                                        dC + (size_t(r0) * N + c0) * 4, size_t(N) * 4, size_t(cols) * 4, rows,
                                        cudaMemcpyDeviceToHost, s_out) == cudaSuccess;
            }
        }
    };
    while ((ua < nm || ub < nn) && rc == 0) {
        // keep the two counts within one of each other, A first, then two of B, then alternate
        const bool take_a = ub >= nn || (ua < nm && ua <= ub - (ua ? 1 : 0));
        if (take_a) copy_a(ua++);
        else copy_b(ub++);
        launch_ready();
    }
    ts.async = was_async;
    cudaEventRecord(e_done, s_out);
    cudaStreamWaitEvent(s_main, e_done, 0);
    cudaEventRecord(rt_event(1), s_main);
    // the copies and kernels above reference the device blocks: finish before they go back to the cache
    const int src = rt_check_status("gemm");
    float ms_total = 0.f;
    if (cudaEventElapsedTime(&ms_total, rt_event(0), rt_event(1)) == cudaSuccess) ts.last_kernel_ns = double(ms_total) * 1e6;
    if (rc) return rc;
    if (!ok) { cudaGetLastError(); return halide_error_code_copy_to_device_failed; }
    if (src) return src;
    C->flags |= 1u;
    *done = true;
    return 0;
}

}  // namespace
}  // namespace t2sp

extern "C" int t2sp_b200_gemm(halide_buffer_t* A, halide_buffer_t* B, halide_buffer_t* C,
                              const t2sp_gemm_desc* desc) {
    int layout = desc ? desc->layout : (C && C->dimensions == 6 ? 1 : 0);
    Arg args[3] = {{A, "A", false, 2}, {B, "B", false, 2}, {C, "C", true, layout ? 6 : 2}};
    if (int e = check_null(args, 3)) return e;

    // ---- bounds queries: fill in what can be inferred and return
    if (buf_is_bounds_query(A) || buf_is_bounds_query(B) || buf_is_bounds_query(C)) {
        int K = 0, M = 0, N = 0;
        if (!buf_is_bounds_query(A) && A->dimensions == 2) { K = A->dim[0].extent; M = A->dim[1].extent; }
        if (!buf_is_bounds_query(B) && B->dimensions == 2) { N = B->dim[0].extent; if (!K) K = B->dim[1].extent; }
        if (!buf_is_bounds_query(C)) {
            if (layout == 0 && C->dimensions == 2) { if (!N) N = C->dim[0].extent; if (!M) M = C->dim[1].extent; }
            if (layout == 1 && C->dimensions == 6) {
                if (!N) N = C->dim[0].extent * C->dim[2].extent * C->dim[4].extent;
                if (!M) M = C->dim[1].extent * C->dim[3].extent * C->dim[5].extent;
            }
        }
        const uint32_t in_t = !buf_is_bounds_query(A) ? buf_type_word(A) : (!buf_is_bounds_query(B) ? buf_type_word(B) : kF32);
        const uint32_t out_t = in_t == kI8 ? kI32 : kF32;
        if (buf_is_bounds_query(A)) { int e2[2] = {K, M}; fill_query(A, in_t, 2, e2); }
        if (buf_is_bounds_query(B)) { int e2[2] = {N, K}; fill_query(B, in_t, 2, e2); }
        if (buf_is_bounds_query(C)) {
            if (layout == 0) { int e2[2] = {N, M}; fill_query(C, out_t, 2, e2); }
            else {
                const int JJJ = desc && desc->JJJ ? desc->JJJ : 1, III = desc && desc->III ? desc->III : 1;
                const int JJ = desc && desc->JJ ? desc->JJ : 1, II = desc && desc->II ? desc->II : 1;
                int e6[6] = {JJJ, III, JJ, II, N / (JJJ * JJ), M / (III * II)};
                fill_query(C, out_t, 6, e6);
            }
        }
        return 0;
    }

    // ---- types and dimensionality
    const uint32_t in_t = buf_type_word(A);
    if (in_t != kF32 && in_t != kBF16 && in_t != kF16 && in_t != kI8)
        return halide_error_bad_type(nullptr, args[0].role().c_str(), in_t, kF32);
    if (int e = check_type_dims(args[0], in_t)) return e;
    if (int e = check_type_dims(args[1], in_t)) return e;
    if (int e = check_type_dims(args[2], in_t == kI8 ? kI32 : kF32)) return e;
    for (auto& a : args)
        if (int e = check_extents_nonneg(a)) return e;

    const bool trans_b = desc && desc->trans_b;
    const bool trans_a = desc && desc->trans_a;
    const bool scale = desc && desc->scale;
    if (trans_a && in_t != kF32) return halide_error_bad_type(nullptr, "Input buffer A (transposed)", in_t, kF32);
    if (scale && (in_t == kI8 || layout != 0)) return constraint("gemm.desc.scale", 1, "fp32 output in the plain layout", 0);
    const int K = A->dim[trans_a ? 1 : 0].extent, M = A->dim[trans_a ? 0 : 1].extent, N = B->dim[trans_b ? 1 : 0].extent;
    if (B->dim[trans_b ? 0 : 1].extent != K)
        return constraint(trans_b ? "B.extent.0" : "B.extent.1", B->dim[trans_b ? 0 : 1].extent, "A.extent.0", K);

    // ---- output coverage
    int JJJ = 1, III = 1, JJ = 1, II = 1;
    if (layout == 0) {
        if (int e = check_covers(args[2], 0, N)) return e;
        if (int e = check_covers(args[2], 1, M)) return e;
    } else {
        JJJ = desc && desc->JJJ ? desc->JJJ : C->dim[0].extent;
        III = desc && desc->III ? desc->III : C->dim[1].extent;
        JJ = desc && desc->JJ ? desc->JJ : C->dim[2].extent;
        II = desc && desc->II ? desc->II : C->dim[3].extent;
        if (JJJ <= 0 || III <= 0 || JJ <= 0 || II <= 0) return constraint("C.tile.extent", 0, "positive", 1);
        if (N % (JJJ * JJ)) return constraint("B.extent.0", N, "multiple of JJJ*JJ", JJJ * JJ);
        if (M % (III * II)) return constraint("A.extent.1", M, "multiple of III*II", III * II);
        const int need[6] = {JJJ, III, JJ, II, N / (JJJ * JJ), M / (III * II)};
        for (int d = 0; d < 6; ++d)
            if (int e = check_covers(args[2], d, need[d])) return e;
    }
    for (auto& a : args)
        if (int e = check_stride0(a)) return e;
    for (auto& a : args)
        if (int e = check_sizes(a)) return e;
    for (auto& a : args)
        if (int e = check_host(a)) return e;
    if (M == 0 || N == 0) return 0;

    // ---- device
    if (int e = rt_ensure_device()) return e;
    const bool resident = all_resident({A, B, C});
    const bool sync_after = !(resident && tls().async);
    if (!resident && K > 0) {
        bool done = false;
        if (int e = gemm_host_pipelined(A, B, C, desc, M, N, K, &done)) return e;
        if (done) return 0;
    }
    Views vw;
    if (int e = rt_input_view(A, "A", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(B, "B", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_output_view(C, "C", &vw.v[vw.n])) return e;
    vw.n++;
    if (scale && desc->beta != 0.f && !vw.v[2].borrowed) {
        // C is an input too: bring the caller's values to the device copy
        if (cudaMemcpyAsync(vw.v[2].ptr, C->host, vw.v[2].bytes, cudaMemcpyHostToDevice, rt_stream()) != cudaSuccess)
            return halide_error_code_copy_to_device_failed;
    }
    const int es = (A->type.bits + 7) / 8;
    char* pa = static_cast<char*>(vw.v[0].ptr) + origin_offset(A) * es;
    char* pb = static_cast<char*>(vw.v[1].ptr) + origin_offset(B) * es;
    uint32_t* pc = static_cast<uint32_t*>(vw.v[2].ptr) + origin_offset(C);

    if (K == 0 && scale) {
        return constraint("A.extent.0", 0, "positive when alpha/beta scaling is requested", 1);
    } else if (K == 0) {
        // empty contraction: the result is all zeros (inside C's extents; padding between rows is not C's)
        rt_zero_region(C, vw.v[2].ptr);
    } else {
        const int arith = arith_for(in_t);
        const int prec = arith == AR_TF32X3 ? resolve_precision(desc ? desc->precision : 0) : 0;
        const int bk = block_k_for(arith);
        const int op = trans_b ? OP_TTM : OP_GEMM;  // OP_TTM is the "both operands K-major" loader
        // Large 16-bit / 8-bit problems run on CTA pairs with 256 x 256 tiles.
        // exactly 128 columns and many row tiles: the 256 x 128 form of the tensor-memory pair kernel (capsule cfg4,
        // which is such a shape: 100 -> 71 us against the single-CTA kernel)
        const bool tm128 = arith == AR_TF32X3 && !rt_env().no_tm128 && N == 128 &&
                           presplit_worthwhile(128, prec, M, int64_t(K) * N * 4);
        const int x3un = arith == AR_TF32X3 ? x3_pair_width(M, N, kBlockM, (K + bk - 1) / bk, tm128) : 0;
        const bool pair = x3un || (arith != AR_TF32X3 && M >= 512 && N >= 512 && !rt_env().no_pair);
        const int bn = x3un ? x3un : (pair ? 256 : core_pick_bn(arith, op, N, M));
        int64_t lda = int64_t(A->dim[1].stride) * es;
        const int64_t ldb = int64_t(B->dim[1].stride) * es;
        if (trans_a) {
            // A arrives as (I_tot, K_tot), i innermost: make the K-major copy the kernel reads, with a
            // row pitch that TMA accepts whatever K is
            const int64_t pitch = (int64_t(K) + 3) / 4 * 4;
            void* at = rt_alloc(size_t(M) * pitch * 4);
            if (!at) return halide_error_code_device_malloc_failed;
            vw.v[vw.n].ptr = at; vw.v[vw.n].borrowed = false; vw.n++;
            if (pitch != K) cudaMemsetAsync(at, 0, size_t(M) * pitch * 4, rt_stream());
            if (transpose32_launch(pa, A->dim[1].stride, at, pitch, K, M, rt_stream()) != cudaSuccess)
                return halide_error_code_device_run_failed;
            rt_count_launch(1);
            pa = static_cast<char*>(at);
            lda = pitch * 4;
        }
        int64_t ldb2 = ldb;
        if (int e = repack_if_unaligned(vw, pa, lda, int64_t(K) * es, M)) return e;
        if (int e = repack_if_unaligned(vw, pb, ldb2, int64_t(trans_b ? K : N) * es, trans_b ? N : K)) return e;
        if (!tma_ok(pa, {lda})) return tma_unsupported("A");
        if (!tma_ok(pb, {ldb2})) return tma_unsupported("B");
        CoreParams p;
        memset(&p, 0, sizeof(p));
        {
            uint64_t dims[2] = {uint64_t(K), uint64_t(M)}, str[2] = {uint64_t(es), uint64_t(lda)};
            uint32_t box[2] = {uint32_t(bk), uint32_t(kBlockM)};
            if (!rt_encode_tmap(&p.mapA[0], tmap_type(in_t), 2, pa, dims, str, box)) return tma_unsupported("A");
        }
        if (trans_b) {
            uint64_t dims[2] = {uint64_t(K), uint64_t(N)}, str[2] = {uint64_t(es), uint64_t(ldb2)};
            uint32_t box[2] = {uint32_t(bk), uint32_t(pair ? bn / 2 : bn)};
            if (!rt_encode_tmap(&p.mapB, tmap_type(in_t), 2, pb, dims, str, box)) return tma_unsupported("B");
            if (presplit_worthwhile(x3un, prec, M, int64_t(N) * ldb2)) {
                BImageParams q{reinterpret_cast<const float*>(pb), 1, ldb2 / 4, K, N, (K + 31) / 32};
                prepack_b(vw, p, q, x3un, N);
            }
        } else {
            uint64_t dims[2] = {uint64_t(N), uint64_t(K)}, str[2] = {uint64_t(es), uint64_t(ldb2)};
            uint32_t box[2] = {uint32_t(128 / es), uint32_t(bk)};
            if (!rt_encode_tmap(&p.mapB, tmap_type(in_t), 2, pb, dims, str, box, arith == AR_TF32X3)) return tma_unsupported("B");
            if (presplit_worthwhile(x3un, prec, M, int64_t(K) * ldb2)) {
                BImageParams q{reinterpret_cast<const float*>(pb), 0, ldb2 / 4, K, N, (K + 31) / 32};
                prepack_b(vw, p, q, x3un, N);
            }
        }
        p.M = M; p.N = N; p.tile_rows = kBlockM; p.a_tx_bytes = kBlockM * 128;
        p.single_pass = prec == T2SP_PRECISION_TF32;
        p.num_kb = (K + bk - 1) / bk; p.total_kb = p.num_kb;
        p.tiles_m = (M + kBlockM - 1) / kBlockM; p.tiles_n = (N + bn - 1) / bn;
        p.idesc = idesc_for(arith, in_t, !trans_b, bn);
        // 512-row pair tiles when there are enough of them to fill the SM pairs several times over
        // (measured: 8192^3 bf16 1436 -> 1536 TFLOP/s, 16384^3 1367 -> 1481; with K = 1024 the tile's
        // drain no longer hides behind the next tile and the 256-row tiles win, 1191 vs 957)
        const bool long_k = (K + bk - 1) / bk >= 64;
        const bool pair2 = pair && !x3un && M >= 1024 && (rt_env().pair2 >= 0 ? rt_env().pair2 != 0 : long_k);
        if (pair) {
            p.tiles_m = pair2 ? (M + 511) / 512 : (M + 255) / 256;
            p.idesc = make_instr_desc(arith == AR_I8 ? 2 : 1, arith == AR_I8 ? 1 : (arith == AR_TF32X3 ? 2 : (in_t == kBF16 ? 1 : 0)),
                                      false, !trans_b, 256, bn);
        }
        p.out = pc;
        if (layout == 0 && scale) {
            p.epi = EPI_ROWMAJOR;
            p.ldo = C->dim[1].stride;
            p.use_ab = 1; p.alpha = desc->alpha; p.beta = desc->beta;
        } else if (layout == 0) {
            set_rowmajor_epilogue(p, pc, M, N, C->dim[1].stride);
        } else {
            p.epi = EPI_SCATTER;
            add_digit(p.dm, 1, III, C->dim[1].stride);
            add_digit(p.dm, III, II, C->dim[3].stride);
            add_digit(p.dm, III * II, 1 << 30, C->dim[5].stride);
            add_digit(p.dn, 1, JJJ, C->dim[0].stride);
            add_digit(p.dn, JJJ, JJ, C->dim[2].stride);
            add_digit(p.dn, JJJ * JJ, 1 << 30, C->dim[4].stride);
        }
        if (int e = run_core("gemm", arith, op, bn, p, sync_after, pair, pair2)) return e;
    }
    if (int e = rt_finish_output(C, "C", &vw.v[2])) return e;
    return finish_call("gemm", "kernel_Out", sync_after);
}

// ======================================================================================= SGEMM
extern "C" int t2sp_b200_sgemm(char transa, char transb, int m, int n, int k, float alpha, const float* a, int lda,
                               const float* b, int ldb, float beta, float* c, int ldc) {
    if (!a || !b || !c) return halide_error_buffer_argument_is_null(nullptr, !a ? "a" : (!b ? "b" : "c"));
    if (m < 0 || n < 0 || k < 0) return halide_error_buffer_extents_negative(nullptr, "sgemm", 0, m < 0 ? m : (n < 0 ? n : k));
    const bool ta = !(transa == 'N' || transa == 'n'), tb = !(transb == 'N' || transb == 'n');
    // row-major arrays as Halide buffers: the contiguous (last) index is dimension 0
    const int a0 = ta ? m : k, a1 = ta ? k : m;
    const int b0 = tb ? k : n, b1 = tb ? n : k;
    if (lda <= 0) lda = a0;
    if (ldb <= 0) ldb = b0;
    if (ldc <= 0) ldc = n;
    if (lda < a0 || ldb < b0 || ldc < n) return constraint("sgemm.ld", lda < a0 ? lda : (ldb < b0 ? ldb : ldc), "at least the row length", 0);
    halide_dimension_t da[2] = {{0, a0, 1, 0}, {0, a1, lda, 0}};
    halide_dimension_t db[2] = {{0, b0, 1, 0}, {0, b1, ldb, 0}};
    halide_dimension_t dc[2] = {{0, n, 1, 0}, {0, m, ldc, 0}};
    halide_buffer_t A, B, C;
    memset(&A, 0, sizeof(A)); memset(&B, 0, sizeof(B)); memset(&C, 0, sizeof(C));
    const uint32_t f32 = kF32;
    A.host = reinterpret_cast<uint8_t*>(const_cast<float*>(a)); A.dimensions = 2; A.dim = da; memcpy(&A.type, &f32, 4);
    B.host = reinterpret_cast<uint8_t*>(const_cast<float*>(b)); B.dimensions = 2; B.dim = db; memcpy(&B.type, &f32, 4);
    C.host = reinterpret_cast<uint8_t*>(c); C.dimensions = 2; C.dim = dc; memcpy(&C.type, &f32, 4);
    t2sp_gemm_desc d;
    memset(&d, 0, sizeof(d));
    d.trans_a = ta; d.trans_b = tb; d.scale = 1; d.alpha = alpha; d.beta = beta;
    return t2sp_b200_gemm(&A, &B, &C, &d);
}

// ======================================================================================= TTM
extern "C" int t2sp_b200_ttm(halide_buffer_t* a, halide_buffer_t* b, halide_buffer_t* c, const t2sp_ttm_desc* desc) {
    int layout = desc ? desc->layout : (c && c->dimensions == 9 ? 1 : 0);
    Arg args[3] = {{a, "a", false, 3}, {b, "b", false, 2}, {c, "c", true, layout ? 9 : 3}};
    if (int e = check_null(args, 3)) return e;
    if (buf_is_bounds_query(a) || buf_is_bounds_query(b) || buf_is_bounds_query(c)) {
        int L = 0, I = 0, J = 0, Kn = 0;
        if (!buf_is_bounds_query(a) && a->dimensions == 3) { L = a->dim[0].extent; I = a->dim[1].extent; J = a->dim[2].extent; }
        if (!buf_is_bounds_query(b) && b->dimensions == 2) { if (!L) L = b->dim[0].extent; Kn = b->dim[1].extent; }
        if (!buf_is_bounds_query(c) && layout == 0 && c->dimensions == 3) {
            if (!I) I = c->dim[0].extent; if (!J) J = c->dim[1].extent; if (!Kn) Kn = c->dim[2].extent;
        }
        if (buf_is_bounds_query(a)) { int e3[3] = {L, I, J}; fill_query(a, kF32, 3, e3); }
        if (buf_is_bounds_query(b)) { int e2[2] = {L, Kn}; fill_query(b, kF32, 2, e2); }
        if (buf_is_bounds_query(c) && layout == 0) { int e3[3] = {I, J, Kn}; fill_query(c, kF32, 3, e3); }
        return 0;
    }
    for (auto& x : args)
        if (int e = check_type_dims(x, kF32)) return e;
    for (auto& x : args)
        if (int e = check_extents_nonneg(x)) return e;
    const int L = a->dim[0].extent, I = a->dim[1].extent, J = a->dim[2].extent, Kn = b->dim[1].extent;
    if (b->dim[0].extent != L) return constraint("b.extent.0", b->dim[0].extent, "a.extent.0", L);
    int III = 1, II = 1, JJJ = 1, JJ = 1, KKK = 1, KK = 1;
    if (layout == 0) {
        if (int e = check_covers(args[2], 0, I)) return e;
        if (int e = check_covers(args[2], 1, J)) return e;
        if (int e = check_covers(args[2], 2, Kn)) return e;
    } else {
        JJ = c->dim[0].extent; KK = c->dim[1].extent; II = c->dim[2].extent;
        KKK = c->dim[3].extent; JJJ = c->dim[4].extent; III = c->dim[5].extent;
        if (JJ <= 0 || KK <= 0 || II <= 0 || KKK <= 0 || JJJ <= 0 || III <= 0) return constraint("c.tile.extent", 0, "positive", 1);
        if (I % (III * II)) return constraint("a.extent.1", I, "multiple of III*II", III * II);
        if (J % (JJJ * JJ)) return constraint("a.extent.2", J, "multiple of JJJ*JJ", JJJ * JJ);
        if (Kn % (KKK * KK)) return constraint("b.extent.1", Kn, "multiple of KKK*KK", KKK * KK);
        if (int e = check_covers(args[2], 6, Kn / (KKK * KK))) return e;
        if (int e = check_covers(args[2], 7, J / (JJJ * JJ))) return e;
        if (int e = check_covers(args[2], 8, I / (III * II))) return e;
    }
    for (auto& x : args)
        if (int e = check_stride0(x)) return e;
    for (auto& x : args)
        if (int e = check_sizes(x)) return e;
    for (auto& x : args)
        if (int e = check_host(x)) return e;
    const int64_t Mrows = int64_t(I) * J;
    if (Mrows == 0 || Kn == 0) return 0;
    if (Mrows >= (int64_t(1) << 31)) return halide_error_buffer_extents_too_large(nullptr, "a", Mrows, (int64_t(1) << 31) - 1);
    if (J > 1 && int64_t(a->dim[2].stride) != int64_t(I) * a->dim[1].stride) {
        fprintf(stderr, "t2sp_b200: ttm: a must be dense across (i, j): a.stride.2 == a.extent.1 * a.stride.1\n");
        return constraint("a.stride.2", a->dim[2].stride, "a.extent.1*a.stride.1", I * a->dim[1].stride);
    }

    if (int e = rt_ensure_device()) return e;
    const bool resident = all_resident({a, b, c});
    const bool sync_after = !(resident && tls().async);
    Views vw;
    if (int e = rt_input_view(a, "a", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(b, "b", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_output_view(c, "c", &vw.v[vw.n])) return e;
    vw.n++;
    char* pa = static_cast<char*>(vw.v[0].ptr) + origin_offset(a) * 4;
    char* pb = static_cast<char*>(vw.v[1].ptr) + origin_offset(b) * 4;
    uint32_t* pc = static_cast<uint32_t*>(vw.v[2].ptr) + origin_offset(c);
    if (L == 0) {
        rt_zero_region(c, vw.v[2].ptr);
    } else {
        const int prec = resolve_precision(desc ? desc->precision : 0);
        const int M = static_cast<int>(Mrows), N = Kn;
        const bool tm128 = !rt_env().no_tm128 && N == 128 && presplit_worthwhile(128, prec, M, int64_t(L) * N * 4);
        const int x3un = x3_pair_width(M, N, kBlockM, (L + 31) / 32, tm128);
        const int bn = x3un ? x3un : core_pick_bn(AR_TF32X3, OP_TTM, N, M);
        int64_t lda = int64_t(a->dim[1].stride) * 4, ldb = int64_t(b->dim[1].stride) * 4;
        if (int e = repack_if_unaligned(vw, pa, lda, int64_t(L) * 4, M)) return e;
        if (int e = repack_if_unaligned(vw, pb, ldb, int64_t(L) * 4, N)) return e;
        if (!tma_ok(pa, {lda})) return tma_unsupported("a");
        if (!tma_ok(pb, {ldb})) return tma_unsupported("b");
        CoreParams p;
        memset(&p, 0, sizeof(p));
        {
            uint64_t dims[2] = {uint64_t(L), uint64_t(M)}, str[2] = {4, uint64_t(lda)};
            uint32_t box[2] = {32, uint32_t(kBlockM)};
            if (!rt_encode_tmap(&p.mapA[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, pa, dims, str, box)) return tma_unsupported("a");
        }
        {
            uint64_t dims[2] = {uint64_t(L), uint64_t(N)}, str[2] = {4, uint64_t(ldb)};
            uint32_t box[2] = {32, uint32_t(x3un ? bn / 2 : bn)};
            if (!rt_encode_tmap(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, pb, dims, str, box)) return tma_unsupported("b");
            if (presplit_worthwhile(x3un, prec, M, int64_t(N) * ldb)) {
                BImageParams q{reinterpret_cast<const float*>(pb), 1, ldb / 4, L, N, (L + 31) / 32};
                prepack_b(vw, p, q, x3un, N);
            }
        }
        p.M = M; p.N = N; p.tile_rows = kBlockM; p.a_tx_bytes = kBlockM * 128;
        p.single_pass = prec == T2SP_PRECISION_TF32;
        p.num_kb = (L + 31) / 32; p.total_kb = p.num_kb;
        p.tiles_m = (M + kBlockM - 1) / kBlockM; p.tiles_n = (N + bn - 1) / bn;
        p.idesc = idesc_for(AR_TF32X3, kF32, false, bn);
        if (x3un) {
            p.tiles_m = (M + 255) / 256;
            p.idesc = make_instr_desc(1, 2, false, false, 256, bn);
        }
        p.out = pc;
        if (layout == 0) {
            if (c->dim[0].stride == 1 && (J == 1 || c->dim[1].stride == I)) {
                set_colmajor_epilogue(p, pc, M, N, c->dim[2].stride);  // rows (i + I*j) are contiguous in the output
            } else {
                p.epi = EPI_SCATTER;
                add_digit(p.dm, 1, I, c->dim[0].stride);
                add_digit(p.dm, I, 1 << 30, c->dim[1].stride);
                add_digit(p.dn, 1, 1 << 30, c->dim[2].stride);
            }
        } else {
            p.epi = EPI_SCATTER;
            add_digit(p.dm, 1, III, c->dim[5].stride);
            add_digit(p.dm, III, II, c->dim[2].stride);
            add_digit(p.dm, III * II, I / (III * II), c->dim[8].stride);
            add_digit(p.dm, I, JJJ, c->dim[4].stride);
            add_digit(p.dm, I * JJJ, JJ, c->dim[0].stride);
            add_digit(p.dm, I * JJJ * JJ, 1 << 30, c->dim[7].stride);
            add_digit(p.dn, 1, KKK, c->dim[3].stride);
            add_digit(p.dn, KKK, KK, c->dim[1].stride);
            add_digit(p.dn, KKK * KK, 1 << 30, c->dim[6].stride);
        }
        if (int e = run_core("ttm", AR_TF32X3, OP_TTM, bn, p, sync_after, x3un != 0)) return e;
    }
    if (int e = rt_finish_output(c, "c", &vw.v[2])) return e;
    return finish_call("ttm", "kernel_unloader", sync_after);
}

// ======================================================================================= CONV
extern "C" int t2sp_b200_conv(halide_buffer_t* I, halide_buffer_t* K, halide_buffer_t* O,
                              const t2sp_conv_desc* desc) {
    if (!desc) {
        fprintf(stderr, "t2sp_b200: conv needs a descriptor (CI, CO, KY, KX, OY, OX cannot be read off the flattened buffers)\n");
        return halide_error_code_generic_error;
    }
    const int layout = desc->layout;
    Arg args[3] = {{I, "I", false, 2}, {K, "K", false, 2}, {O, "O", true, layout ? 10 : 2}};
    if (int e = check_null(args, 3)) return e;
    const int CI = desc->CI, CO = desc->CO, KY = desc->KY, KX = desc->KX, OY = desc->OY, OX = desc->OX;
    if (CI <= 0 || CO <= 0 || KY <= 0 || KX <= 0 || OY <= 0 || OX <= 0) return constraint("conv.desc", 0, "positive", 1);
    const int IY = OY + KY - 1, IX = OX + KX - 1;
    if (buf_is_bounds_query(I) || buf_is_bounds_query(K) || buf_is_bounds_query(O)) {
        int N = 0;
        if (!buf_is_bounds_query(I) && I->dimensions == 2) N = I->dim[0].extent / CI;
        else if (!buf_is_bounds_query(O) && layout == 0 && O->dimensions == 2) N = O->dim[0].extent / CO;
        else if (!buf_is_bounds_query(O) && layout == 1 && O->dimensions == 10) N = O->dim[9].extent;
        if (buf_is_bounds_query(I)) { int e2[2] = {CI * N, IY * IX}; fill_query(I, kF32, 2, e2); }
        if (buf_is_bounds_query(K)) { int e2[2] = {CO * KX, CI * KY}; fill_query(K, kF32, 2, e2); }
        if (buf_is_bounds_query(O)) {
            if (layout == 0) { int e2[2] = {CO * N, OY * OX}; fill_query(O, kF32, 2, e2); }
            else {
                const int den = std::max(1, desc->COOO * desc->COO);
                int e10[10] = {desc->COOO, desc->YYY, desc->XXX, desc->COO, desc->YY, desc->XX, desc->Y, desc->X, CO / den, N};
                fill_query(O, kF32, 10, e10);
            }
        }
        return 0;
    }
    for (auto& x : args)
        if (int e = check_type_dims(x, kF32)) return e;
    for (auto& x : args)
        if (int e = check_extents_nonneg(x)) return e;
    if (I->dim[0].extent % CI) return constraint("I.extent.0", I->dim[0].extent, "multiple of CI", CI);
    const int N = I->dim[0].extent / CI;
    if (I->dim[1].extent != IY * IX) return constraint("I.extent.1", I->dim[1].extent, "IY*IX", IY * IX);
    if (K->dim[0].extent != CO * KX) return constraint("K.extent.0", K->dim[0].extent, "CO*KX", CO * KX);
    if (K->dim[1].extent != CI * KY) return constraint("K.extent.1", K->dim[1].extent, "CI*KY", CI * KY);
    if (layout == 0) {
        if (int e = check_covers(args[2], 0, CO * N)) return e;
        if (int e = check_covers(args[2], 1, OY * OX)) return e;
    } else {
        if (desc->COOO <= 0 || desc->COO <= 0 || desc->YYY <= 0 || desc->YY <= 0 || desc->Y <= 0 || desc->XXX <= 0 ||
            desc->XX <= 0 || desc->X <= 0)
            return constraint("conv.desc.tile", 0, "positive", 1);
        if (desc->YYY * desc->YY * desc->Y != OY) return constraint("YYY*YY*Y", desc->YYY * desc->YY * desc->Y, "OY", OY);
        if (desc->XXX * desc->XX * desc->X != OX) return constraint("XXX*XX*X", desc->XXX * desc->XX * desc->X, "OX", OX);
        if (CO % (desc->COOO * desc->COO)) return constraint("CO", CO, "multiple of COOO*COO", desc->COOO * desc->COO);
        const int need[10] = {desc->COOO, desc->YYY, desc->XXX, desc->COO, desc->YY, desc->XX, desc->Y, desc->X,
                              CO / (desc->COOO * desc->COO), N};
        for (int d = 0; d < 10; ++d)
            if (int e = check_covers(args[2], d, need[d])) return e;
    }
    for (auto& x : args)
        if (int e = check_stride0(x)) return e;
    for (auto& x : args)
        if (int e = check_sizes(x)) return e;
    for (auto& x : args)
        if (int e = check_host(x)) return e;
    if (N == 0) return 0;
    const int64_t Mrows = int64_t(N) * OY * OX;
    if (Mrows >= (int64_t(1) << 31)) return halide_error_buffer_extents_too_large(nullptr, "O", Mrows, (int64_t(1) << 31) - 1);

    if (int e = rt_ensure_device()) return e;
    const bool resident = all_resident({I, K, O});
    const bool sync_after = !(resident && tls().async);
    Views vw;
    if (int e = rt_input_view(I, "I", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(K, "K", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_output_view(O, "O", &vw.v[vw.n])) return e;
    vw.n++;
    char* pi = static_cast<char*>(vw.v[0].ptr) + origin_offset(I) * 4;
    char* pk = static_cast<char*>(vw.v[1].ptr) + origin_offset(K) * 4;
    uint32_t* po = static_cast<uint32_t*>(vw.v[2].ptr) + origin_offset(O);
    const int prec = resolve_precision(desc->precision);

    int bn = core_pick_bn(AR_TF32X3, OP_CONV, CO, Mrows);
    const int64_t s1 = int64_t(I->dim[1].stride) * 4, t1 = int64_t(K->dim[1].stride) * 4;
    if (!tma_ok(pi, {int64_t(CI) * 4, s1})) return tma_unsupported("I");
    if (!tma_ok(pk, {int64_t(CO) * 4, t1})) return tma_unsupported("K");
    CoreParams p;
    memset(&p, 0, sizeof(p));
    p.rows.nd = 3;
    p.rows.ext[0] = N; p.rows.ext[1] = OY; p.rows.ext[2] = OX; p.rows.ext[3] = 1;
    int rbox[4] = {1, 1, 1, 1};
    plan_rows(p.rows, rbox);
    {
        // input as (ci, n, iy, ix)
        uint64_t dims[4] = {uint64_t(CI), uint64_t(N), uint64_t(IY), uint64_t(IX)};
        uint64_t str[4] = {4, uint64_t(CI) * 4, uint64_t(s1), uint64_t(IY) * uint64_t(s1)};
        uint32_t box[4] = {32, uint32_t(rbox[0]), uint32_t(rbox[1]), uint32_t(rbox[2])};
        if (!rt_encode_tmap(&p.mapA[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, pi, dims, str, box)) return tma_unsupported("I");
    }
    {
        // weights as (co, kx, ci, ky)
        uint64_t dims[4] = {uint64_t(CO), uint64_t(KX), uint64_t(CI), uint64_t(KY)};
        uint64_t str[4] = {4, uint64_t(CO) * 4, uint64_t(t1), uint64_t(CI) * uint64_t(t1)};
        uint32_t box[4] = {32, 1, 32, 1};
        if (!rt_encode_tmap(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, pk, dims, str, box, true)) return tma_unsupported("K");
    }
    p.M = static_cast<int>(Mrows); p.N = CO;
    p.tile_rows = p.rows.rows_per_box * p.rows.boxes_per_tile;
    p.a_tx_bytes = p.tile_rows * 128;
    p.single_pass = prec == T2SP_PRECISION_TF32;
    p.cblks = (CI + 31) / 32; p.KY = KY; p.KX = KX; p.stride = 1;
    p.num_kb = KY * KX * p.cblks; p.total_kb = p.num_kb;
    const bool tm128c = !rt_env().no_tm128 && CO == 128 && presplit_worthwhile(128, prec, p.M, int64_t(CI) * KY * t1);
    const int x3un = x3_pair_width(p.M, CO, p.tile_rows, p.num_kb, tm128c);
    if (x3un) bn = x3un;
    if (presplit_worthwhile(x3un, prec, p.M, int64_t(CI) * KY * t1)) {
        BImageParams q{reinterpret_cast<const float*>(pk), 2, t1 / 4, CI, CO, p.num_kb, 0, p.cblks, KY};
        prepack_b(vw, p, q, x3un, CO);
    }
    p.tiles_m = x3un ? (p.M + 255) / 256 : (p.M + p.tile_rows - 1) / p.tile_rows; p.tiles_n = (CO + bn - 1) / bn;
    p.idesc = x3un ? make_instr_desc(1, 2, false, true, 256, bn) : idesc_for(AR_TF32X3, kF32, true, bn);
    p.out = po;
    if (layout == 0) {
        const int64_t so = O->dim[1].stride;
        if (so == int64_t(CO) * N) {
            set_rowmajor_epilogue(p, po, p.M, CO, CO);
        } else {
            p.epi = EPI_SCATTER;
            add_digit(p.dm, 1, N, CO);
            add_digit(p.dm, N, 1 << 30, so);
            add_digit(p.dn, 1, 1 << 30, 1);
        }
    } else {
        p.epi = EPI_SCATTER;
        const halide_dimension_t* d = O->dim;
        add_digit(p.dm, 1, N, d[9].stride);
        add_digit(p.dm, N, desc->YYY, d[1].stride);
        add_digit(p.dm, N * desc->YYY, desc->YY, d[4].stride);
        add_digit(p.dm, N * desc->YYY * desc->YY, desc->Y, d[6].stride);
        add_digit(p.dm, N * OY, desc->XXX, d[2].stride);
        add_digit(p.dm, N * OY * desc->XXX, desc->XX, d[5].stride);
        add_digit(p.dm, N * OY * desc->XXX * desc->XX, 1 << 30, d[7].stride);
        add_digit(p.dn, 1, desc->COOO, d[0].stride);
        add_digit(p.dn, desc->COOO, desc->COO, d[3].stride);
        add_digit(p.dn, desc->COOO * desc->COO, 1 << 30, d[8].stride);
    }
    if (int e = run_core("conv", AR_TF32X3, OP_CONV, bn, p, sync_after, x3un != 0)) return e;
    if (int e = rt_finish_output(O, "O", &vw.v[2])) return e;
    return finish_call("conv", "kernel_unloader", sync_after);
}

// ======================================================================================= CAPSULE
extern "C" int t2sp_b200_capsule(halide_buffer_t* P, halide_buffer_t* W, halide_buffer_t* V,
                                 const t2sp_capsule_desc* desc) {
    if (!desc) {
        fprintf(stderr, "t2sp_b200: capsule needs a descriptor (the flattened buffers do not carry CI, CII, CO, ...)\n");
        return halide_error_code_generic_error;
    }
    const int layout = desc->layout;
    Arg args[3] = {{P, "P", false, 2}, {W, "W", false, 2}, {V, "V", true, layout ? 10 : 2}};
    if (int e = check_null(args, 3)) return e;
    const int CI = desc->CI, CII = desc->CII, CO = desc->CO, KY = desc->KY, KX = desc->KX, OY = desc->OY, OX = desc->OX;
    const int MY = desc->MY, MX = desc->MX, MK = desc->MK, NN = desc->NN, s = desc->stride;
    if (CI <= 0 || CII <= 0 || CO <= 0 || KY <= 0 || KX <= 0 || OY <= 0 || OX <= 0 || MY <= 0 || MX <= 0 || MK <= 0 || NN <= 0)
        return constraint("capsule.desc", 0, "positive", 1);
    if (s != 1 && s != 2) return constraint("capsule.desc.stride", s, "1 or 2", 2);
    if (CI % CII) return constraint("CI", CI, "multiple of CII", CII);
    const int IY = s * OY + KY - s, IX = s * OX + KX - s;
    const int Q = MX * NN, NW = CO * MY, CP = CI * MK;
    if (buf_is_bounds_query(P) || buf_is_bounds_query(W) || buf_is_bounds_query(V)) {
        int N = 0;
        if (!buf_is_bounds_query(P) && P->dimensions == 2) N = P->dim[1].extent / (IY * IX);
        else if (!buf_is_bounds_query(V) && layout == 0 && V->dimensions == 2) N = V->dim[1].extent / (OY * OX);
        else if (!buf_is_bounds_query(V) && layout == 1 && V->dimensions == 10) N = V->dim[9].extent;
        if (buf_is_bounds_query(P)) { int e2[2] = {CP * Q, IY * IX * N}; fill_query(P, kF32, 2, e2); }
        if (buf_is_bounds_query(W)) { int e2[2] = {NW, CI * KY * KX * MK}; fill_query(W, kF32, 2, e2); }
        if (buf_is_bounds_query(V)) {
            if (layout == 0) { int e2[2] = {NW * Q, OY * OX * N}; fill_query(V, kF32, 2, e2); }
            else {
                const int den = std::max(1, desc->COOO * desc->COO);
                int e10[10] = {desc->COOO, desc->YYY_XXX, desc->YY_XX, desc->Y_X, MY, MX, desc->COO, NN, CO / den, N};
                fill_query(V, kF32, 10, e10);
            }
        }
        return 0;
    }
    for (auto& x : args)
        if (int e = check_type_dims(x, kF32)) return e;
    for (auto& x : args)
        if (int e = check_extents_nonneg(x)) return e;
    if (P->dim[0].extent != CP * Q) return constraint("P.extent.0", P->dim[0].extent, "CI*MK*MX*NN", CP * Q);
    if (P->dim[1].extent % (IY * IX)) return constraint("P.extent.1", P->dim[1].extent, "multiple of IY*IX", IY * IX);
    const int N = P->dim[1].extent / (IY * IX);
    if (W->dim[0].extent != NW) return constraint("W.extent.0", W->dim[0].extent, "CO*MY", NW);
    if (W->dim[1].extent != CI * KY * KX * MK) return constraint("W.extent.1", W->dim[1].extent, "CI*KY*KX*MK", CI * KY * KX * MK);
    int slots = OY * OX;
    if (layout == 0) {
        if (int e = check_covers(args[2], 0, NW * Q)) return e;
        if (int e = check_covers(args[2], 1, OY * OX * N)) return e;
    } else {
        if (desc->COOO <= 0 || desc->COO <= 0 || desc->YYY_XXX <= 0 || desc->YY_XX <= 0 || desc->Y_X <= 0)
            return constraint("capsule.desc.tile", 0, "positive", 1);
        slots = desc->YYY_XXX * desc->YY_XX * desc->Y_X;
        if (slots < OY * OX) return constraint("YYY_XXX*YY_XX*Y_X", slots, "at least OY*OX", OY * OX);
        if (CO % (desc->COOO * desc->COO)) return constraint("CO", CO, "multiple of COOO*COO", desc->COOO * desc->COO);
        const int need[10] = {desc->COOO, desc->YYY_XXX, desc->YY_XX, desc->Y_X, MY, MX, desc->COO, NN,
                              CO / (desc->COOO * desc->COO), N};
        for (int d = 0; d < 10; ++d)
            if (int e = check_covers(args[2], d, need[d])) return e;
    }
    for (auto& x : args)
        if (int e = check_stride0(x)) return e;
    for (auto& x : args)
        if (int e = check_sizes(x)) return e;
    for (auto& x : args)
        if (int e = check_host(x)) return e;
    if (N == 0) return 0;
    const int64_t Mrows = int64_t(Q) * OY * OX * N;
    if (Mrows >= (int64_t(1) << 31)) return halide_error_buffer_extents_too_large(nullptr, "V", Mrows, (int64_t(1) << 31) - 1);
    // weight box walk: 32 consecutive c' = ci + CI*mk values per k-block
    int bcii, bcio, bmk;
    if (CII % 32 == 0) { bcii = 32; bcio = 1; bmk = 1; }
    else if (CI % 32 == 0 && 32 % CII == 0) { bcii = CII; bcio = 32 / CII; bmk = 1; }
    else if (32 % CI == 0) { bcii = CII; bcio = CI / CII; bmk = std::min(MK, 32 / CI); }
    else {
        fprintf(stderr, "t2sp_b200: capsule: CI=%d CII=%d is not supported (need CII%%32==0, or CI%%32==0 with 32%%CII==0, or 32%%CI==0)\n", CI, CII);
        return halide_error_code_constraint_violated;
    }

    if (int e = rt_ensure_device()) return e;
    const bool resident = all_resident({P, W, V});
    const bool sync_after = !(resident && tls().async);
    Views vw;
    if (int e = rt_input_view(P, "P", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(W, "W", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_output_view(V, "V", &vw.v[vw.n])) return e;
    vw.n++;
    char* pp = static_cast<char*>(vw.v[0].ptr) + origin_offset(P) * 4;
    char* pw = static_cast<char*>(vw.v[1].ptr) + origin_offset(W) * 4;
    uint32_t* pv = static_cast<uint32_t*>(vw.v[2].ptr) + origin_offset(V);
    const int prec = resolve_precision(desc->precision);

    int bn = core_pick_bn(AR_TF32X3, OP_CAPSULE, NW, Mrows);
    const int64_t s1 = int64_t(P->dim[1].stride) * 4, t1 = int64_t(W->dim[1].stride) * 4;
    if (!tma_ok(pp, {int64_t(CP) * 4, s1})) return tma_unsupported("P");
    if (!tma_ok(pw, {t1})) return tma_unsupported("W");
    CoreParams p;
    memset(&p, 0, sizeof(p));
    p.rows.nd = 4;
    p.rows.ext[0] = Q; p.rows.ext[1] = OY; p.rows.ext[2] = OX; p.rows.ext[3] = N;
    int rbox[4] = {1, 1, 1, 1};
    plan_rows(p.rows, rbox);
    for (int py = 0; py < s; ++py)
        for (int px = 0; px < s; ++px) {
            // input of one stride parity as (c', q, iy', ix', n), iy = s*iy' + py, ix = s*ix' + px
            const int ey = (IY - py + s - 1) / s, ex = (IX - px + s - 1) / s;
            uint64_t dims[5] = {uint64_t(CP), uint64_t(Q), uint64_t(ey), uint64_t(ex), uint64_t(N)};
            uint64_t str[5] = {4, uint64_t(CP) * 4, uint64_t(s) * uint64_t(s1), uint64_t(s) * uint64_t(IY) * uint64_t(s1),
                               uint64_t(IY) * uint64_t(IX) * uint64_t(s1)};
            uint32_t box[5] = {32, uint32_t(rbox[0]), uint32_t(rbox[1]), uint32_t(rbox[2]), uint32_t(rbox[3])};
            char* base = pp + (int64_t(py) + int64_t(px) * IY) * s1;
            if (!rt_encode_tmap(&p.mapA[py + 2 * px], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, base, dims, str, box))
                return tma_unsupported("P");
        }
    {
        // weights as (n = co + CO*my, cii, tap = ky + KY*kx, ci_outer, mk)
        uint64_t dims[5] = {uint64_t(NW), uint64_t(CII), uint64_t(KY) * uint64_t(KX), uint64_t(CI / CII), uint64_t(MK)};
        uint64_t str[5] = {4, uint64_t(t1), uint64_t(CII) * uint64_t(t1), uint64_t(CII) * KY * KX * uint64_t(t1),
                           uint64_t(CI) * KY * KX * uint64_t(t1)};
        uint32_t box[5] = {32, uint32_t(bcii), 1, uint32_t(bcio), uint32_t(bmk)};
        if (!rt_encode_tmap(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, pw, dims, str, box, true)) return tma_unsupported("W");
    }
    p.M = static_cast<int>(Mrows); p.N = NW;
    p.tile_rows = p.rows.rows_per_box * p.rows.boxes_per_tile;
    p.a_tx_bytes = p.tile_rows * 128;
    p.single_pass = prec == T2SP_PRECISION_TF32;
    p.cblks = (CP + 31) / 32; p.KY = KY; p.KX = KX; p.stride = s; p.CI = CI; p.CII = CII;
    p.num_kb = KY * KX * p.cblks; p.total_kb = p.num_kb;
    const bool tm128 = !rt_env().no_tm128 && NW == 128 && presplit_worthwhile(128, prec, p.M, int64_t(CI) * KY * KX * MK * t1);
    const int x3un = x3_pair_width(p.M, NW, p.tile_rows, p.num_kb, tm128);
    if (x3un) bn = x3un;
    if (presplit_worthwhile(x3un, prec, p.M, int64_t(CI) * KY * KX * MK * t1) && (x3un == 256 || tm128)) {
        BImageParams q{reinterpret_cast<const float*>(pw), 3, t1 / 4, CP, NW, p.num_kb, 0, p.cblks, KY, 0, CI, CII, KY * KX};
        prepack_b(vw, p, q, x3un, NW);
    }
    p.tiles_m = x3un ? (p.M + 255) / 256 : (p.M + p.tile_rows - 1) / p.tile_rows; p.tiles_n = (NW + bn - 1) / bn;
    p.idesc = x3un ? make_instr_desc(1, 2, false, true, 256, bn) : idesc_for(AR_TF32X3, kF32, true, bn);
    p.out = pv;
    if (layout == 0) {
        const int64_t so = V->dim[1].stride;
        if (so == int64_t(NW) * Q) {
            set_rowmajor_epilogue(p, pv, p.M, NW, NW);
        } else {
            p.epi = EPI_SCATTER;
            add_digit(p.dm, 1, Q, NW);
            add_digit(p.dm, Q, 1 << 30, so);
            add_digit(p.dn, 1, 1 << 30, 1);
        }
    } else {
        if (slots > OY * OX) rt_zero_region(V, vw.v[2].ptr);
        p.epi = EPI_SCATTER;
        const halide_dimension_t* d = V->dim;
        add_digit(p.dm, 1, MX, d[5].stride);
        add_digit(p.dm, MX, NN, d[7].stride);
        // pixel number pix = (m / Q) % (OY*OX), then its three tile digits
        const int PX = OY * OX;
        add_digit2(p.dm, Q, PX, 1, desc->YYY_XXX, d[1].stride);
        add_digit2(p.dm, Q, PX, desc->YYY_XXX, desc->YY_XX, d[2].stride);
        add_digit2(p.dm, Q, PX, desc->YYY_XXX * desc->YY_XX, 1 << 30, d[3].stride);
        add_digit(p.dm, Q * PX, 1 << 30, d[9].stride);
        add_digit(p.dn, 1, desc->COOO, d[0].stride);
        add_digit(p.dn, desc->COOO, desc->COO, d[6].stride);
        add_digit(p.dn, desc->COOO * desc->COO, CO / (desc->COOO * desc->COO), d[8].stride);
        add_digit(p.dn, CO, 1 << 30, d[4].stride);
    }
    if (int e = run_core("capsule", AR_TF32X3, OP_CAPSULE, bn, p, sync_after, x3un != 0)) return e;
    if (int e = rt_finish_output(V, "V", &vw.v[2])) return e;
    return finish_call("capsule", "kernel_unloader", sync_after);
}

// ======================================================================================= MTTKRP
namespace t2sp {
// Lowers and launches the split-K MTTKRP into caller-provided partial-sum scratch
// (splits * I * R floats) followed by the ordered reduction. Shared by the allocating entry.
int mttkrp_launch(const char* who, float* pa, int64_t lda1, int64_t lda2, const float* pb, int64_t ldb,
                  const float* pc, int64_t ldc, float* pd, int64_t ldd, int L, int I, int Kd, int R, int splits,
                  int num_kb, float* scratch, bool sync_after, bool single_pass) {
    const int bn = core_pick_bn(AR_TF32X3, OP_MTTKRP, R);
    if (bn == 0) return constraint("d.extent.1", R, "at most", 128);
    if (!tma_ok(pa, {lda1 * 4, lda2 * 4})) return tma_unsupported("a");
    CoreParams p;
    memset(&p, 0, sizeof(p));
    {
        uint64_t dims[3] = {uint64_t(L), uint64_t(I), uint64_t(Kd)};
        uint64_t str[3] = {4, uint64_t(lda1) * 4, uint64_t(lda2) * 4};
        uint32_t box[3] = {32, uint32_t(kBlockM), 1};
        if (!rt_encode_tmap(&p.mapA[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, pa, dims, str, box)) return tma_unsupported("a");
    }
    {
        // factor c(l, r): one box = 32 consecutive l of every column r, i.e. one K-major B tile
        if (!tma_ok(pc, {ldc * 4})) return tma_unsupported("c");
        uint64_t dims[2] = {uint64_t(L), uint64_t(R)};
        uint64_t str[2] = {4, uint64_t(ldc) * 4};
        uint32_t box[2] = {32, uint32_t(bn)};
        if (!rt_encode_tmap(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(pc), dims, str, box)) return tma_unsupported("c");
    }
    const int lblks = (L + 31) / 32;
    p.M = I; p.N = R; p.tile_rows = kBlockM; p.a_tx_bytes = kBlockM * 128;
    p.total_kb = lblks * Kd;
    p.num_kb = num_kb;
    p.tiles_m = (I + kBlockM - 1) / kBlockM;
    p.tiles_n = splits; p.splits = splits; p.lblks = lblks;
    p.idesc = idesc_for(AR_TF32X3, kF32, false, bn);
    p.epi = EPI_COLMAJOR;      // partial[split][r][i], i fastest
    p.ldo = I;
    p.out = scratch;
    p.fc = pc; p.fb = pb; p.ldfc = ldc; p.ldfb = ldb;
    p.L = L; p.Kdim = Kd; p.R = R;
    p.single_pass = single_pass;
    if (int e = run_core(who, AR_TF32X3, OP_MTTKRP, bn, p, sync_after)) return e;
    if (reduce_partials_launch(scratch, pd, I, R, ldd, splits, rt_stream()) != cudaSuccess)
        return halide_error_code_device_run_failed;
    rt_count_launch(1);
    if (sync_after) cudaEventRecord(rt_event(1), rt_stream());
    return 0;
}

// The accumulate-then-scale kernel (umma_mttkrp.cuh), for R <= 64: work items are (row tile, up to 4 l-blocks,
// up to 64 k values); as many k-ranges as fill the SMs once. `want_slabs` > 0 asks for about that many partial
// slabs instead (tests). Returns the number of partial slabs (l-ranges x k-ranges).
int mttkrp2_plan(int L, int I, int Kd, int want_slabs, CoreParams* p) {
    const int lblks = (L + 31) / 32, tiles_m = (I + kBlockM - 1) / kBlockM;
    const int lb_per = std::min(4, lblks), lranges = (lblks + lb_per - 1) / lb_per;
    int kranges = want_slabs > 0 ? std::max(1, (want_slabs + lranges / 2) / lranges)
                                 : std::max(1, core_sm_count() / std::max(1, tiles_m * lranges));
    kranges = std::max(1, std::min(kranges, Kd));
    int k_per = std::min(64, (Kd + kranges - 1) / kranges);
    kranges = (Kd + k_per - 1) / k_per;
    p->tiles_m = tiles_m; p->lblks = lblks;
    p->mt_lb_per = lb_per; p->mt_lranges = lranges; p->mt_k_per = k_per; p->mt_kranges = kranges;
    return lranges * kranges;
}

int mttkrp2_run(const char* who, float* pa, int64_t lda1, int64_t lda2, const float* pb, int64_t ldb, const float* pc,
                int64_t ldc, float* pd, int64_t ldd, int L, int I, int Kd, int R, int want_slabs, bool sync_after,
                bool single_pass) {
    if (!tma_ok(pa, {lda1 * 4, lda2 * 4})) return tma_unsupported("a");
    if (!tma_ok(pc, {ldc * 4})) return tma_unsupported("c");
    CoreParams p;
    memset(&p, 0, sizeof(p));
    const int slabs = mttkrp2_plan(L, I, Kd, want_slabs, &p);
    {
        uint64_t dims[3] = {uint64_t(L), uint64_t(I), uint64_t(Kd)};
        uint64_t str[3] = {4, uint64_t(lda1) * 4, uint64_t(lda2) * 4};
        uint32_t box[3] = {32, uint32_t(kBlockM), 1};
        if (!rt_encode_tmap(&p.mapA[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, pa, dims, str, box)) return tma_unsupported("a");
    }
    {
        // factor c(l, r): one box = 32 consecutive l of 64 columns r (columns beyond R read as zero), a K-major B tile
        uint64_t dims[2] = {uint64_t(L), uint64_t(R)};
        uint64_t str[2] = {4, uint64_t(ldc) * 4};
        uint32_t box[2] = {32, 64};
        if (!rt_encode_tmap(&p.mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(pc), dims, str, box)) return tma_unsupported("c");
    }
    float* scratch = static_cast<float*>(rt_alloc(size_t(slabs) * I * R * sizeof(float)));
    if (!scratch) return halide_error_code_device_malloc_failed;
    p.M = I; p.N = R; p.R = R; p.L = L; p.Kdim = Kd;
    p.fb = pb; p.ldfb = ldb;
    p.out = scratch;
    p.single_pass = single_pass;
    p.status = rt_status_word();
    p.wait_cycles = rt_env().wait_cycles;
    cudaStream_t s = rt_stream();
    const int items = p.tiles_m * slabs;
#ifdef T2SP_DEBUG_KNOBS
    static long long* trace_dev = nullptr;
    const char* trace_path = getenv("T2SP_B200_TRACE");
    if (trace_path) {
        if (!trace_dev) cudaMalloc(&trace_dev, 48 * 1024 * sizeof(long long));
        cudaMemsetAsync(trace_dev, 0, 48 * 1024 * sizeof(long long), s);
        p.trace = trace_dev;
    }
#endif
    if (sync_after) cudaEventRecord(rt_event(0), s);
    cudaError_t e = mttkrp2_launch(p, std::max(1, std::min(items, core_sm_count())), s);
    if (e == cudaSuccess) e = reduce_partials_launch(scratch, pd, I, R, ldd, slabs, s);
    rt_free(scratch);  // whoever takes the block over on another stream waits for this stream's work so far
    if (e != cudaSuccess) {
        fprintf(stderr, "t2sp_b200: %s: kernel launch failed: %s\n", who, cudaGetErrorString(e));
        return halide_error_code_device_run_failed;
    }
    rt_count_launch(2);
    if (sync_after) cudaEventRecord(rt_event(1), s);
#ifdef T2SP_DEBUG_KNOBS
    static int trace_calls = 0;
    const char* trace_at = getenv("T2SP_B200_TRACE_AT");
    if (trace_path && (!trace_at || ++trace_calls == atoi(trace_at))) {
        std::vector<long long> host(48 * 1024);
        cudaStreamSynchronize(s);
        cudaMemcpy(host.data(), trace_dev, host.size() * sizeof(long long), cudaMemcpyDeviceToHost);
        if (FILE* f = fopen(trace_path, "wb")) { fwrite(host.data(), sizeof(long long), host.size(), f); fclose(f); }
    }
#endif
    return 0;
}

// Split plan: enough (row tile, split) pairs to give every SM one CTA, never an empty split.
void mttkrp_plan(int L, int I, int Kd, int want_splits, int* splits, int* num_kb) {
    const int total_kb = ((L + 31) / 32) * Kd;
    const int tiles_m = (I + kBlockM - 1) / kBlockM;
    int s = want_splits > 0 ? want_splits : std::max(1, core_sm_count() / std::max(1, tiles_m));
    s = std::max(1, std::min(s, total_kb));
    const int per = (total_kb + s - 1) / s;
    *num_kb = per;
    *splits = (total_kb + per - 1) / per;
}
}  // namespace t2sp

extern "C" int t2sp_b200_mttkrp(halide_buffer_t* a, halide_buffer_t* b, halide_buffer_t* c, halide_buffer_t* d,
                                const t2sp_mttkrp_desc* desc) {
    Arg args[4] = {{a, "a", false, 3}, {b, "b", false, 2}, {c, "c", false, 2}, {d, "d", true, 2}};
    if (int e = check_null(args, 4)) return e;
    if (buf_is_bounds_query(a) || buf_is_bounds_query(b) || buf_is_bounds_query(c) || buf_is_bounds_query(d)) {
        int L = 0, I = 0, Kd = 0, R = 0;
        if (!buf_is_bounds_query(a) && a->dimensions == 3) { L = a->dim[0].extent; I = a->dim[1].extent; Kd = a->dim[2].extent; }
        if (!buf_is_bounds_query(b) && b->dimensions == 2) { if (!Kd) Kd = b->dim[0].extent; R = b->dim[1].extent; }
        if (!buf_is_bounds_query(c) && c->dimensions == 2) { if (!L) L = c->dim[0].extent; if (!R) R = c->dim[1].extent; }
        if (!buf_is_bounds_query(d) && d->dimensions == 2) { if (!I) I = d->dim[0].extent; if (!R) R = d->dim[1].extent; }
        if (buf_is_bounds_query(a)) { int e3[3] = {L, I, Kd}; fill_query(a, kF32, 3, e3); }
        if (buf_is_bounds_query(b)) { int e2[2] = {Kd, R}; fill_query(b, kF32, 2, e2); }
        if (buf_is_bounds_query(c)) { int e2[2] = {L, R}; fill_query(c, kF32, 2, e2); }
        if (buf_is_bounds_query(d)) { int e2[2] = {I, R}; fill_query(d, kF32, 2, e2); }
        return 0;
    }
    for (auto& x : args)
        if (int e = check_type_dims(x, kF32)) return e;
    for (auto& x : args)
        if (int e = check_extents_nonneg(x)) return e;
    const int L = a->dim[0].extent, I = a->dim[1].extent, Kd = a->dim[2].extent, R = b->dim[1].extent;
    if (b->dim[0].extent != Kd) return constraint("b.extent.0", b->dim[0].extent, "a.extent.2", Kd);
    if (c->dim[0].extent != L) return constraint("c.extent.0", c->dim[0].extent, "a.extent.0", L);
    if (c->dim[1].extent != R) return constraint("c.extent.1", c->dim[1].extent, "b.extent.1", R);
    if (int e = check_covers(args[3], 0, I)) return e;
    if (int e = check_covers(args[3], 1, R)) return e;
    for (auto& x : args)
        if (int e = check_stride0(x)) return e;
    for (auto& x : args)
        if (int e = check_sizes(x)) return e;
    for (auto& x : args)
        if (int e = check_host(x)) return e;
    if (I == 0 || R == 0) return 0;
    if (R > 128) return constraint("b.extent.1", R, "at most", 128);

    if (int e = rt_ensure_device()) return e;
    const bool resident = all_resident({a, b, c, d});
    const bool sync_after = !(resident && tls().async);
    Views vw;
    if (int e = rt_input_view(a, "a", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(b, "b", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_input_view(c, "c", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = rt_output_view(d, "d", &vw.v[vw.n])) return e;
    vw.n++;
    float* pa = static_cast<float*>(vw.v[0].ptr) + origin_offset(a);
    float* pb = static_cast<float*>(vw.v[1].ptr) + origin_offset(b);
    float* pc = static_cast<float*>(vw.v[2].ptr) + origin_offset(c);
    float* pd = static_cast<float*>(vw.v[3].ptr) + origin_offset(d);
    if (L == 0 || Kd == 0) {
        rt_zero_region(d, vw.v[3].ptr);
    } else {
        const int prec = resolve_precision(desc ? desc->precision : 0);
        if (R <= 64 && !rt_env().mttkrp_v1) {
            if (int rc = mttkrp2_run("mttkrp", pa, a->dim[1].stride, a->dim[2].stride, pb, b->dim[1].stride, pc, c->dim[1].stride, pd,
                                     d->dim[1].stride, L, I, Kd, R, desc ? desc->splits : 0, sync_after, prec == T2SP_PRECISION_TF32))
                return rc;
            if (int e = rt_finish_output(d, "d", &vw.v[3])) return e;
            return finish_call("mttkrp", "kernel_unloader", sync_after);
        }
        int splits = 0, num_kb = 0;
        mttkrp_plan(L, I, Kd, desc ? desc->splits : 0, &splits, &num_kb);
        float* scratch = static_cast<float*>(rt_alloc(size_t(splits) * I * R * sizeof(float)));
        if (!scratch) return halide_error_code_device_malloc_failed;
        int rc = mttkrp_launch("mttkrp", pa, a->dim[1].stride, a->dim[2].stride, pb, b->dim[1].stride, pc,
                               c->dim[1].stride, pd, d->dim[1].stride, L, I, Kd, R, splits, num_kb, scratch, sync_after,
                               prec == T2SP_PRECISION_TF32);
        // Stream order keeps the scratch block safe: a later call on this stream that reuses it
        // runs after this call's kernels.
        rt_free(scratch);
        if (rc) return rc;
    }
    if (int e = rt_finish_output(d, "d", &vw.v[3])) return e;
    return finish_call("mttkrp", "kernel_unloader", sync_after);
}

// ======================================================================================= N-D FRONTS
// The oneAPI flow of the reference passes convolution and capsule operands as N-D buffers with the
// spatial index innermost (oneapi-target-5-conv.cpp:58-62, oneapi-target-6-capsule.cpp:57-61) instead
// of the flattened channel-innermost 2-D buffers of the OpenCL flow. These entries re-lay the inputs
// out on the device (one gather kernel per operand, into scratch) and run the 2-D entries on the
// copies; every constant the 2-D entries take from a descriptor is read off the N-D extents.
namespace {

struct Scratch {
    void* p = nullptr;
    ~Scratch() { if (p) t2sp::rt_free(p); }  // stream order protects later users of the block
};

// A dense 2-D fp32 buffer that lives on this library's device.
void make_device_2d(halide_buffer_t* b, halide_dimension_t* dims, void* ptr, int e0, int e1) {
    memset(b, 0, sizeof(*b));
    b->type.code = 2; b->type.bits = 32; b->type.lanes = 1;
    b->dimensions = 2;
    b->dim = dims;
    dims[0].min = 0; dims[0].extent = e0; dims[0].stride = 1; dims[0].flags = 0;
    dims[1].min = 0; dims[1].extent = e1; dims[1].stride = e0; dims[1].flags = 0;
    t2sp_b200_wrap_device_ptr(b, reinterpret_cast<uint64_t>(ptr));
}

int nd_common_checks(Arg* args, int n) {
    if (int e = check_null(args, n)) return e;
    for (int i = 0; i < n; ++i) {
        if (buf_is_bounds_query(args[i].b))
            return halide_error_host_is_null(nullptr, args[i].role().c_str());  // shapes cannot be inferred from nothing
        if (int e = check_type_dims(args[i], kF32)) return e;
        if (int e = check_extents_nonneg(args[i])) return e;
        if (int e = check_sizes(args[i])) return e;
        if (int e = check_host(args[i])) return e;
    }
    return 0;
}

// Gathers input buffer `b` (N-D, any strides) into dense scratch laid out by `d` (d.sstride is
// filled in here from b's strides through `src_dim`: destination dimension i reads b's src_dim[i]).
int gather_to_scratch(halide_buffer_t* b, const char* name, t2sp::PermuteDesc d, const int* src_dim, size_t dst_elems,
                      Scratch* out, bool zero_fill = false) {
    t2sp::DeviceView v;
    if (int e = t2sp::rt_input_view(b, name, &v)) return e;
    out->p = t2sp::rt_alloc(dst_elems * 4);
    if (!out->p) { t2sp::rt_drop_view(&v); return halide_error_code_device_malloc_failed; }
    if (zero_fill) cudaMemsetAsync(out->p, 0, dst_elems * 4, t2sp::rt_stream());  // the copy leaves padding untouched
    for (int i = 0; i < d.nd; ++i) d.sstride[i] = b->dim[src_dim[i]].stride;
    const uint32_t* src = static_cast<const uint32_t*>(v.ptr) + origin_offset(b);
    const cudaError_t e = t2sp::permute_copy_launch(src, out->p, d, t2sp::rt_stream());
    t2sp::rt_count_launch(1);
    t2sp::rt_drop_view(&v);  // an uploaded copy goes back to the cache; stream order keeps it valid for the gather
    return e == cudaSuccess ? 0 : halide_error_code_device_run_failed;
}

}  // namespace

extern "C" int t2sp_b200_conv_nd(halide_buffer_t* I, halide_buffer_t* K, halide_buffer_t* O, int precision) {
    Arg args[3] = {{I, "I", false, 4}, {K, "K", false, 4}, {O, "O", true, 10}};
    if (int e = nd_common_checks(args, 3)) return e;
    const int IY = I->dim[0].extent, IX = I->dim[1].extent, CI = I->dim[2].extent, N = I->dim[3].extent;
    const int KY = K->dim[0].extent, KX = K->dim[1].extent, CO = K->dim[3].extent;
    if (K->dim[2].extent != CI) return constraint("K.extent.2", K->dim[2].extent, "I.extent.2", CI);
    t2sp_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.layout = 1;
    d.COOO = O->dim[0].extent; d.YYY = O->dim[1].extent; d.XXX = O->dim[2].extent; d.COO = O->dim[3].extent;
    d.YY = O->dim[4].extent; d.XX = O->dim[5].extent; d.Y = O->dim[6].extent; d.X = O->dim[7].extent;
    d.OY = d.YYY * d.YY * d.Y; d.OX = d.XXX * d.XX * d.X;
    d.KY = KY; d.KX = KX; d.CO = CO; d.precision = precision;
    if (IY != d.OY + KY - 1) return constraint("I.extent.0", IY, "OY+KY-1", d.OY + KY - 1);
    if (IX != d.OX + KX - 1) return constraint("I.extent.1", IX, "OX+KX-1", d.OX + KX - 1);
    if (d.COOO * d.COO * O->dim[8].extent != CO) return constraint("COOO*COO*CO", d.COOO * d.COO * O->dim[8].extent, "K.extent.3", CO);
    if (O->dim[9].extent != N) return constraint("O.extent.9", O->dim[9].extent, "I.extent.3", N);
    if (CO % 4) return constraint("K.extent.3", CO, "multiple of 4", (CO + 3) / 4 * 4);
    if (N == 0 || CO == 0 || d.OY == 0 || d.OX == 0) return 0;
    if (int e = t2sp::rt_ensure_device()) return e;
    const int CIp = (CI + 3) / 4 * 4;  // zero channels up to the 16-byte pitch TMA needs
    d.CI = CIp;
    Scratch si, sk;
    {
        // destination (ci, n, iy, ix). A dense input is one batched matrix transpose per image n:
        // rows = ci (pitch IY*IX), columns = pixels iy + IY*ix  ->  rows = pixels (pitch CIp*N), columns = ci
        const bool dense = I->dim[1].stride == IY && I->dim[2].stride == IY * IX && N <= 65535;
        if (dense && CIp == CI) {
            t2sp::DeviceView v;
            if (int e = t2sp::rt_input_view(I, "I", &v)) return e;
            si.p = t2sp::rt_alloc(size_t(CIp) * N * IY * IX * 4);
            if (!si.p) { t2sp::rt_drop_view(&v); return halide_error_code_device_malloc_failed; }
            const uint32_t* src = static_cast<const uint32_t*>(v.ptr) + origin_offset(I);
            const cudaError_t e = t2sp::transpose32_launch(src, (long long)IY * IX, si.p, (long long)CIp * N, CI, IY * IX,
                                                           t2sp::rt_stream(), N, I->dim[3].stride, CIp);
            t2sp::rt_count_launch(1);
            t2sp::rt_drop_view(&v);
            if (e != cudaSuccess) return halide_error_code_device_run_failed;
        } else {
            t2sp::PermuteDesc pd;
            memset(&pd, 0, sizeof(pd));
            pd.nd = 4;
            const int ext[4] = {CI, N, IY, IX}, src[4] = {2, 3, 0, 1};
            const long long ds[4] = {1, CIp, (long long)CIp * N, (long long)CIp * N * IY};
            for (int i = 0; i < 4; ++i) { pd.ext[i] = ext[i]; pd.dstride[i] = ds[i]; }
            if (int e = gather_to_scratch(I, "I", pd, src, size_t(CIp) * N * IY * IX, &si, CIp != CI)) return e;
        }
    }
    {
        t2sp::PermuteDesc pd;
        memset(&pd, 0, sizeof(pd));
        pd.nd = 4;  // destination order (co, kx, ci, ky)
        const int ext[4] = {CO, KX, CI, KY}, src[4] = {3, 1, 2, 0};
        const long long ds[4] = {1, CO, (long long)CO * KX, (long long)CO * KX * CIp};
        for (int i = 0; i < 4; ++i) { pd.ext[i] = ext[i]; pd.dstride[i] = ds[i]; }
        if (int e = gather_to_scratch(K, "K", pd, src, size_t(CO) * KX * CIp * KY, &sk, CIp != CI)) return e;
    }
    halide_buffer_t i2, k2;
    halide_dimension_t di[2], dk[2];
    make_device_2d(&i2, di, si.p, CIp * N, IY * IX);
    make_device_2d(&k2, dk, sk.p, CO * KX, CIp * KY);
    return t2sp_b200_conv(&i2, &k2, O, &d);
}

extern "C" int t2sp_b200_capsule_nd(halide_buffer_t* P, halide_buffer_t* W, halide_buffer_t* V, int precision) {
    Arg args[3] = {{P, "P", false, 6}, {W, "W", false, 6}, {V, "V", true, 9}};
    if (int e = nd_common_checks(args, 3)) return e;
    const int MK = P->dim[0].extent, MX = P->dim[1].extent, CI = P->dim[2].extent, IY = P->dim[3].extent,
              IX = P->dim[4].extent, N = P->dim[5].extent;
    const int MY = W->dim[0].extent, CO = W->dim[3].extent, KY = W->dim[4].extent, KX = W->dim[5].extent;
    if (W->dim[1].extent != MK) return constraint("W.extent.1", W->dim[1].extent, "P.extent.0", MK);
    if (W->dim[2].extent != CI) return constraint("W.extent.2", W->dim[2].extent, "P.extent.2", CI);
    t2sp_capsule_desc d;
    memset(&d, 0, sizeof(d));
    d.layout = 1;
    d.COOO = V->dim[0].extent; d.YYY_XXX = V->dim[1].extent; d.YY_XX = V->dim[2].extent; d.Y_X = V->dim[3].extent;
    d.COO = V->dim[6].extent;
    d.CI = CI; d.CII = CI; d.CO = CO; d.KY = KY; d.KX = KX; d.MY = MY; d.MX = MX; d.MK = MK; d.NN = 1;
    d.precision = precision;
    if (V->dim[4].extent != MY) return constraint("V.extent.4", V->dim[4].extent, "W.extent.0", MY);
    if (V->dim[5].extent != MX) return constraint("V.extent.5", V->dim[5].extent, "P.extent.1", MX);
    if (d.COOO * d.COO * V->dim[7].extent != CO) return constraint("COOO*COO*CO", d.COOO * d.COO * V->dim[7].extent, "W.extent.3", CO);
    if (V->dim[8].extent != N) return constraint("V.extent.8", V->dim[8].extent, "P.extent.5", N);
    // The reference's capsule layer strides by 2 (capsule.cpp:40-41); a stride-1 shape is accepted as well.
    // The stride is the one whose output size fits the pixel slots of V.
    const long long slots = (long long)d.YYY_XXX * d.YY_XX * d.Y_X;
    d.stride = 0;
    for (int s = 2; s >= 1 && !d.stride; --s) {
        const int oy = (IY - KY + s) / s, ox = (IX - KX + s) / s;
        if (oy > 0 && ox > 0 && (IY - KY) % s == 0 && (IX - KX) % s == 0 && (long long)oy * ox <= slots &&
            (long long)oy * ox > slots - d.YYY_XXX) {
            d.stride = s; d.OY = oy; d.OX = ox;
        }
    }
    if (!d.stride) return constraint("YYY_XXX*YY_XX*Y_X", (int)slots, "OY*OX", ((IY - KY + 2) / 2) * ((IX - KX + 2) / 2));
    if ((CI * MK) % 4) return constraint("P.extent.2*P.extent.0", CI * MK, "multiple of 4", (CI * MK + 3) / 4 * 4);
    if ((CO * MY) % 4) return constraint("W.extent.3*W.extent.0", CO * MY, "multiple of 4", (CO * MY + 3) / 4 * 4);
    if (N == 0 || CO == 0) return 0;
    if (int e = t2sp::rt_ensure_device()) return e;
    Scratch sp, sw;
    {
        t2sp::PermuteDesc pd;
        memset(&pd, 0, sizeof(pd));
        pd.nd = 6;  // destination order (ci, mk, mx, iy, ix, n)
        const int ext[6] = {CI, MK, MX, IY, IX, N}, src[6] = {2, 0, 1, 3, 4, 5};
        long long s = 1;
        for (int i = 0; i < 6; ++i) { pd.ext[i] = ext[i]; pd.dstride[i] = s; s *= ext[i]; }
        if (int e = gather_to_scratch(P, "P", pd, src, size_t(s), &sp)) return e;
    }
    {
        t2sp::PermuteDesc pd;
        memset(&pd, 0, sizeof(pd));
        pd.nd = 6;  // destination order (co, my, ci, ky, kx, mk): the 2-D layout with CII = CI
        const int ext[6] = {CO, MY, CI, KY, KX, MK}, src[6] = {3, 0, 2, 4, 5, 1};
        long long s = 1;
        for (int i = 0; i < 6; ++i) { pd.ext[i] = ext[i]; pd.dstride[i] = s; s *= ext[i]; }
        if (int e = gather_to_scratch(W, "W", pd, src, size_t(s), &sw)) return e;
    }
    halide_buffer_t p2, w2;
    halide_dimension_t dp[2], dw[2];
    make_device_2d(&p2, dp, sp.p, CI * MK * MX, IY * IX * N);
    make_device_2d(&w2, dw, sw.p, CO * MY, CI * KY * KX * MK);
    // V as the 10-D buffer of the OpenCL flow: a unit NN dimension goes in before CO
    halide_buffer_t v10 = *V;
    halide_dimension_t dv[10];
    for (int i = 0; i < 7; ++i) dv[i] = V->dim[i];
    dv[7].min = 0; dv[7].extent = 1; dv[7].stride = V->dim[7].stride; dv[7].flags = 0;
    dv[8] = V->dim[7];
    dv[9] = V->dim[8];
    v10.dimensions = 10;
    v10.dim = dv;
    const int rc = t2sp_b200_capsule(&p2, &w2, &v10, &d);
    V->flags = v10.flags;
    V->device = v10.device;
    V->device_interface = v10.device_interface;
    return rc;
}

// ======================================================================================= SYRK
// The generated SYRK interface of the PEPPERS BLAS layer
// (t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:12, specification
// t2s/tests/performance/syrk/syrk.cpp:52-73): A(K, N), symmetric C(N, N), and the folded 6-D output
// O(III, III, II, II, I+1, I) with N = III*II*I. The product R = A A^T runs as an fp32 GEMM whose B
// operand is A itself (both K-major) into scratch; a second kernel folds alpha R + beta C into O.
// OpA is accepted and, as in the specification (which never reads it), has no effect.
extern "C" int t2sp_b200_syrk(int32_t opa, float alpha, float beta, halide_buffer_t* A, halide_buffer_t* C,
                              halide_buffer_t* O) {
    (void)opa;
    Arg args[3] = {{A, "A", false, 2}, {C, "C", false, 2}, {O, "deserializer", true, 6}};
    if (int e = nd_common_checks(args, 3)) return e;
    const int K = A->dim[0].extent, N = A->dim[1].extent;
    const int III = O->dim[0].extent, II = O->dim[2].extent, I = O->dim[4].extent - 1;
    if (O->dim[1].extent != III) return constraint("deserializer.extent.1", O->dim[1].extent, "deserializer.extent.0", III);
    if (O->dim[3].extent != II) return constraint("deserializer.extent.3", O->dim[3].extent, "deserializer.extent.2", II);
    if (I < 0 || I % 2) return constraint("deserializer.extent.4 - 1", I, "even", I + 1);
    if (O->dim[5].extent < I / 2) return constraint("deserializer.extent.5", O->dim[5].extent, "I/2", I / 2);
    if (III * II * I != N) return constraint("III*II*I", III * II * I, "A.extent.1", N);
    if (C->dim[0].extent < N || C->dim[1].extent < N) return constraint("C.extent", std::min(C->dim[0].extent, C->dim[1].extent), "A.extent.1", N);
    for (int i = 0; i < 2; ++i)
        if (int e = check_stride0(args[i])) return e;
    if (N == 0) return 0;
    if (int e = t2sp::rt_ensure_device()) return e;
    Views vw;
    if (int e = t2sp::rt_input_view(A, "A", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = t2sp::rt_input_view(C, "C", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = t2sp::rt_output_view(O, "deserializer", &vw.v[vw.n])) return e;
    vw.n++;
    // The design writes rows i < I/2 of the folded buffer only; a host buffer comes back whole, so its
    // device copy starts from the host's content and the untouched elements keep their values.
    if (!vw.v[2].borrowed && O->host && vw.v[2].bytes &&
        cudaMemcpyAsync(vw.v[2].ptr, O->host, vw.v[2].bytes, cudaMemcpyHostToDevice, t2sp::rt_stream()) != cudaSuccess) {
        cudaGetLastError();
        return halide_error_code_copy_to_device_failed;
    }
    Scratch sr;
    sr.p = t2sp::rt_alloc(size_t(N) * N * 4);
    if (!sr.p) return halide_error_code_device_malloc_failed;
    // R(N, N) = A(K, N) x A(K, N)^T through the GEMM entry, on device-resident views
    halide_buffer_t a = *A, r;
    halide_dimension_t da[2] = {A->dim[0], A->dim[1]}, dr[2];
    a.dim = da;
    a.host = nullptr; a.flags = 0; a.device = 0; a.device_interface = nullptr;
    t2sp_b200_wrap_device_ptr(&a, reinterpret_cast<uint64_t>(static_cast<float*>(vw.v[0].ptr)));
    make_device_2d(&r, dr, sr.p, N, N);
    t2sp_gemm_desc gd;
    memset(&gd, 0, sizeof(gd));
    gd.trans_b = 1;
    ThreadState& ts = tls();
    const bool was_async = ts.async;
    ts.async = true;  // the fold below is ordered behind the GEMM on the stream; no host wait in between
    const int rc = K > 0 ? t2sp_b200_gemm(&a, &a, &r, &gd) : 0;
    ts.async = was_async;
    if (rc) return rc;
    if (K == 0) cudaMemsetAsync(sr.p, 0, size_t(N) * N * 4, t2sp::rt_stream());
    t2sp::SyrkFold f;
    f.III = III; f.II = II; f.I = I;
    for (int d = 0; d < 6; ++d) f.ostride[d] = O->dim[d].stride;
    f.ldr = N; f.ldc = C->dim[1].stride;
    f.alpha = alpha; f.beta = beta;
    const float* pc = static_cast<const float*>(vw.v[1].ptr) + origin_offset(C);
    float* po = static_cast<float*>(vw.v[2].ptr) + origin_offset(O);
    if (t2sp::syrk_fold_launch(static_cast<const float*>(sr.p), pc, po, f, t2sp::rt_stream()) != cudaSuccess)
        return halide_error_code_device_run_failed;
    t2sp::rt_count_launch(1);
    if (int e = t2sp::rt_finish_output(O, "deserializer", &vw.v[2])) return e;
    return t2sp::rt_check_status("syrk");
}

extern "C" int t2sp_b200_ger(halide_buffer_t* A, halide_buffer_t* X, halide_buffer_t* Y, halide_buffer_t* O) {
    Arg args[4] = {{A, "A", false, 2}, {X, "X", false, 1}, {Y, "Y", false, 1}, {O, "deserializer", true, 6}};
    if (int e = nd_common_checks(args, 4)) return e;
    const int TK = A->dim[0].extent, TI = A->dim[1].extent;
    const long long ok = 1ll * O->dim[0].extent * O->dim[3].extent * O->dim[4].extent;
    const long long oi = 1ll * O->dim[1].extent * O->dim[2].extent * O->dim[5].extent;
    if (ok != TK) return constraint("KKK*KK*K", static_cast<int>(ok), "A.extent.0", TK);
    if (oi != TI) return constraint("III*II*I", static_cast<int>(oi), "A.extent.1", TI);
    if (int e = check_covers(args[1], 0, TI)) return e;
    if (int e = check_covers(args[2], 0, TK)) return e;
    if (TK == 0 || TI == 0) return 0;
    if (int e = t2sp::rt_ensure_device()) return e;
    Views vw;
    if (int e = t2sp::rt_input_view(A, "A", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = t2sp::rt_input_view(X, "X", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = t2sp::rt_input_view(Y, "Y", &vw.v[vw.n])) return e;
    vw.n++;
    if (int e = t2sp::rt_output_view(O, "deserializer", &vw.v[vw.n])) return e;
    vw.n++;
    t2sp::GerDesc d;
    for (int i = 0; i < 6; ++i) { d.ext[i] = O->dim[i].extent; d.ostride[i] = O->dim[i].stride; }
    d.lda = A->dim[1].stride; d.sa0 = A->dim[0].stride; d.sx = X->dim[0].stride; d.sy = Y->dim[0].stride;
    // element 0 of the vectors is index 0 whatever the buffer's min (check_covers made sure it is covered)
    const float* pa = static_cast<const float*>(vw.v[0].ptr) + origin_offset(A);
    const float* px = static_cast<const float*>(vw.v[1].ptr) - 1ll * X->dim[0].min * X->dim[0].stride;
    const float* py = static_cast<const float*>(vw.v[2].ptr) - 1ll * Y->dim[0].min * Y->dim[0].stride;
    float* po = static_cast<float*>(vw.v[3].ptr) + origin_offset(O);
    if (t2sp::ger_launch(pa, px, py, po, d, t2sp::rt_stream()) != cudaSuccess) return halide_error_code_device_run_failed;
    t2sp::rt_count_launch(1);
    if (int e = t2sp::rt_finish_output(O, "deserializer", &vw.v[3])) return e;
    return t2sp::rt_check_status("ger");
}
