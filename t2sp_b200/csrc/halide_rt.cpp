// The rest of the entry points the reference's AOT runtime exports for generated host code and its
// callers (t2s/src/AOT-OpenCL-Runtime.cpp:70-72 device interface, :74-117 device malloc, :119-277 and
// :280-310 combined host/device allocation, :312-397 wait for kernels, :399-441 copies, :443-727 the
// remaining error reporters), under the same names and as weak symbols, over this library's device
// runtime. user_context and the device-interface argument are accepted and ignored: there is one
// device interface here (t2sp_b200_device_interface).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>

#include "t2sp_b200/runtime.h"

#define T2SP_WEAK __attribute__((weak))

extern "C" {
void halide_error(void*, const char*);
void* halide_malloc(void*, size_t);
void halide_free(void*, void*);
}

namespace {
int report(void* uc, const std::string& msg, int code) {
    halide_error(uc, msg.c_str());
    return code;
}
size_t span_bytes(const halide_buffer_t* b) {
    long long lo = 0, hi = 0;
    for (int d = 0; d < b->dimensions; ++d) {
        const long long reach = (long long)(b->dim[d].extent - 1) * b->dim[d].stride;
        if (b->dim[d].extent <= 0) return 0;
        if (reach > 0) hi += reach; else lo += reach;
    }
    return size_t(hi - lo + 1) * ((b->type.bits + 7) / 8);
}
}  // namespace

extern "C" {

T2SP_WEAK const struct halide_device_interface_t* halide_opencl_device_interface() {
    return static_cast<const halide_device_interface_t*>(t2sp_b200_device_interface());
}

T2SP_WEAK int halide_device_malloc(void* /*uc*/, halide_buffer_t* buf, const halide_device_interface_t* /*iface*/) {
    return t2sp_b200_device_malloc(buf);
}

T2SP_WEAK int32_t halide_device_and_host_malloc(void* uc, halide_buffer_t* buf, const halide_device_interface_t* /*iface*/) {
    if (!buf) return halide_error_code_buffer_argument_is_null;
    buf->host = static_cast<uint8_t*>(halide_malloc(uc, span_bytes(buf)));
    if (!buf->host) return halide_error_code_out_of_memory;
    const int rc = t2sp_b200_device_malloc(buf);
    if (rc != 0) {
        halide_free(uc, buf->host);
        buf->host = nullptr;
    }
    return rc;
}

T2SP_WEAK int32_t halide_device_and_host_free(void* uc, void* obj) {
    halide_buffer_t* buf = static_cast<halide_buffer_t*>(obj);
    if (!buf) return halide_error_code_buffer_argument_is_null;
    const int rc = t2sp_b200_device_free(buf);
    if (buf->host) {
        halide_free(uc, buf->host);
        buf->host = nullptr;
    }
    buf->flags &= ~uint64_t(3);  // neither copy is dirty any more
    return rc;
}

T2SP_WEAK void halide_device_and_host_free_as_destructor(void* /*uc*/, void* /*obj*/) {}
T2SP_WEAK void halide_device_host_nop_free(void* /*uc*/, void* /*obj*/) {}

// Returns once every kernel launched so far by the calling thread has finished.
T2SP_WEAK int32_t halide_opencl_wait_for_kernels_finish(void* /*uc*/) { return t2sp_b200_sync(); }

// Copies src to dst in whichever direction the buffers' state asks for: the source is the host copy
// when src has no device allocation or its host copy is the newer one.
T2SP_WEAK int halide_opencl_buffer_copy(void* /*uc*/, halide_buffer_t* src, halide_buffer_t* dst, bool to_host) {
    if (!src || !dst) return halide_error_code_buffer_argument_is_null;
    const bool from_host = src->device == 0 || ((src->flags & 1u) && src->host);
    if (!from_host && to_host) {
        if (src == dst) return t2sp_b200_copy_to_host(dst);
        uint8_t* keep = src->host;
        src->host = dst->host;
        const int rc = t2sp_b200_copy_to_host(src);
        src->host = keep;
        return rc;
    }
    if (from_host && !to_host) {
        if (src == dst) return t2sp_b200_copy_to_device(dst);
        uint8_t* keep = dst->host;
        dst->host = src->host;
        const int rc = t2sp_b200_copy_to_device(dst);
        dst->host = keep;
        return rc;
    }
    if (!from_host && !to_host) return halide_error_code_device_buffer_copy_failed;  // device to device: not offered
    if (dst->host != src->host && dst->host && src->host) memcpy(dst->host, src->host, span_bytes(src));
    return 0;
}

T2SP_WEAK int halide_copy_to_device(void* uc, halide_buffer_t* buf, const halide_device_interface_t* /*iface*/) {
    return halide_opencl_buffer_copy(uc, buf, buf, false);
}

T2SP_WEAK int halide_copy_to_host(void* uc, halide_buffer_t* buf) { return halide_opencl_buffer_copy(uc, buf, buf, true); }

// ---------------------------------------------------------------- remaining error reporters
T2SP_WEAK int halide_error_bounds_inference_call_failed(void* uc, const char* stage, int result) {
    return report(uc, "Bounds inference call to external stage " + std::string(stage) + " returned non-zero value: " + std::to_string(result), result);
}
T2SP_WEAK int halide_error_extern_stage_failed(void* uc, const char* stage, int result) {
    return report(uc, "Call to external stage " + std::string(stage) + " returned non-zero value: " + std::to_string(result), result);
}
T2SP_WEAK int halide_error_explicit_bounds_too_small(void* uc, const char* func, const char* var, int min_bound, int max_bound,
                                                     int min_required, int max_required) {
    return report(uc,
                  "Bounds given for " + std::string(var) + " in " + func + " (from " + std::to_string(min_bound) + " to " +
                      std::to_string(max_bound) + ") do not cover required region (from " + std::to_string(min_required) +
                      " to " + std::to_string(max_required) + ")",
                  halide_error_code_explicit_bounds_too_small);
}
T2SP_WEAK int halide_error_constraints_make_required_region_smaller(void* uc, const char* buffer, int dimension, int cmin,
                                                                    int cextent, int rmin, int rextent) {
    return report(uc,
                  "Applying the constraints on " + std::string(buffer) + " to the required region made it smaller in dimension " +
                      std::to_string(dimension) + ". Required size: " + std::to_string(rmin) + " to " +
                      std::to_string(rmin + rextent - 1) + ". Constrained size: " + std::to_string(cmin) + " to " +
                      std::to_string(cmin + cextent - 1) + ".",
                  halide_error_code_constraints_make_required_region_smaller);
}
#define T2SP_PARAM_REPORT(NAME, TYPE, WORD, CODE)                                                              \
    T2SP_WEAK int NAME(void* uc, const char* param, TYPE val, TYPE bound) {                                    \
        return report(uc, "Parameter " + std::string(param) + " is " + std::to_string(val) + " but must be at " WORD " " + \
                              std::to_string(bound), CODE);                                                   \
    }
T2SP_PARAM_REPORT(halide_error_param_too_small_i64, int64_t, "least", halide_error_code_param_too_small)
T2SP_PARAM_REPORT(halide_error_param_too_small_u64, uint64_t, "least", halide_error_code_param_too_small)
T2SP_PARAM_REPORT(halide_error_param_too_small_f64, double, "least", halide_error_code_param_too_small)
T2SP_PARAM_REPORT(halide_error_param_too_large_i64, int64_t, "most", halide_error_code_param_too_large)
T2SP_PARAM_REPORT(halide_error_param_too_large_u64, uint64_t, "most", halide_error_code_param_too_large)
T2SP_PARAM_REPORT(halide_error_param_too_large_f64, double, "most", halide_error_code_param_too_large)
#undef T2SP_PARAM_REPORT
T2SP_WEAK int halide_error_debug_to_file_failed(void* uc, const char* func, const char* filename, int error_code) {
    return report(uc, "Failed to dump function " + std::string(func) + " to file " + filename + " with error " + std::to_string(error_code),
                  halide_error_code_debug_to_file_failed);
}
T2SP_WEAK int halide_error_failed_to_upgrade_buffer_t(void* uc, const char* name, const char* reason) {
    return report(uc, "Failed to upgrade buffer_t to halide_buffer_t for " + std::string(name) + ": " + reason,
                  halide_error_code_failed_to_upgrade_buffer_t);
}
T2SP_WEAK int halide_error_failed_to_downgrade_buffer_t(void* uc, const char* name, const char* reason) {
    return report(uc, "Failed to downgrade halide_buffer_t to buffer_t for " + std::string(name) + ": " + reason,
                  halide_error_code_failed_to_downgrade_buffer_t);
}
T2SP_WEAK int halide_error_unaligned_host_ptr(void* uc, const char* func, int alignment) {
    return report(uc, "The host pointer of " + std::string(func) + " is not aligned to a " + std::to_string(alignment) + " bytes boundary.",
                  halide_error_code_unaligned_host_ptr);
}
T2SP_WEAK int halide_error_bad_fold(void* uc, const char* func, const char* var, const char* loop) {
    return report(uc, "The folded storage dimension " + std::string(var) + " of " + func + " was accessed out of order by loop " + loop + ".",
                  halide_error_code_bad_fold);
}
T2SP_WEAK int halide_error_bad_extern_fold(void* uc, const char* func, int dim, int min, int extent, int valid_min, int fold_factor) {
    return report(uc,
                  "The extern function " + std::string(func) + " accessed [" + std::to_string(min) + ", " + std::to_string(min + extent - 1) +
                      "] of folded dimension " + std::to_string(dim) + " (valid from " + std::to_string(valid_min) + ", fold factor " +
                      std::to_string(fold_factor) + ")",
                  halide_error_code_bad_extern_fold);
}
T2SP_WEAK int halide_error_fold_factor_too_small(void* uc, const char* func, const char* var, int fold_factor, const char* loop,
                                                 int required_extent) {
    return report(uc,
                  "The fold factor (" + std::to_string(fold_factor) + ") of dimension " + var + " of " + func + " is too small to store the required region accessed by loop " +
                      loop + " (" + std::to_string(required_extent) + ").",
                  halide_error_code_fold_factor_too_small);
}
T2SP_WEAK int halide_error_requirement_failed(void* uc, const char* condition, const char* message) {
    return report(uc, "Requirement Failed: (" + std::string(condition) + ") " + message, halide_error_code_requirement_failed);
}
T2SP_WEAK int halide_error_specialize_fail(void* uc, const char* message) {
    return report(uc, "A schedule specialized with specialize_fail() was chosen: " + std::string(message), halide_error_code_specialize_fail);
}
T2SP_WEAK int halide_error_no_device_interface(void* uc) {
    return report(uc, "Buffer has a non-zero device but no device interface.", halide_error_code_no_device_interface);
}
T2SP_WEAK int halide_error_host_and_device_dirty(void* uc) {
    return report(uc, "Buffer has both host and device dirty bits set.", halide_error_code_host_and_device_dirty);
}
T2SP_WEAK int halide_error_buffer_is_null(void* uc, const char* routine) {
    return report(uc, "Buffer pointer passed to " + std::string(routine) + " is null.", halide_error_code_buffer_is_null);
}
T2SP_WEAK int halide_error_integer_division_by_zero(void* uc) {
    return report(uc, "Integer division or modulo by zero.", halide_error_code_integer_division_by_zero);
}

}  // extern "C"
