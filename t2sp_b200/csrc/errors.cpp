// Halide-style error reporters: each prints a message through halide_error() and returns
// its halide_error_code_t. They are weak so a caller can supply its own, exactly as with the
// reference runtime (t2s/src/AOT-OpenCL-Runtime.cpp:22,56-72 for halide_error/malloc/free,
// :443-727 for the reporters; codes from HalideRuntime.h:957-1143).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>

#include "t2sp_b200/runtime.h"

#define T2SP_WEAK __attribute__((weak))

extern "C" {

T2SP_WEAK void* halide_malloc(void* /*user_context*/, size_t sz) {
    void* p = nullptr;
    if (posix_memalign(&p, 128, sz) != 0) return nullptr;
    return p;
}

T2SP_WEAK void halide_free(void* /*user_context*/, void* ptr) { free(ptr); }

T2SP_WEAK void halide_error(void* /*user_context*/, const char* msg) { fprintf(stderr, "%s\n", msg); }

static int report(void* uc, const std::string& msg, int code) {
    halide_error(uc, msg.c_str());
    return code;
}

T2SP_WEAK int halide_error_bad_type(void* uc, const char* func_name, uint32_t type_given_bits,
                                    uint32_t correct_type_bits) {
    halide_type_t given, correct;
    memcpy(&given, &type_given_bits, 4);
    memcpy(&correct, &correct_type_bits, 4);
    return report(uc,
                  std::string(func_name) + " has type code " + std::to_string(correct.code) + "/" +
                      std::to_string(correct.bits) + " bits but the buffer passed in has type code " +
                      std::to_string(given.code) + "/" + std::to_string(given.bits) + " bits",
                  halide_error_code_bad_type);
}

T2SP_WEAK int halide_error_bad_dimensions(void* uc, const char* func_name, int32_t dimensions_given,
                                          int32_t correct_dimensions) {
    return report(uc,
                  std::string(func_name) + " requires a buffer of exactly " + std::to_string(correct_dimensions) +
                      " dimensions, but the buffer passed in has " + std::to_string(dimensions_given) + " dimensions",
                  halide_error_code_bad_dimensions);
}

T2SP_WEAK int halide_error_access_out_of_bounds(void* uc, const char* func_name, int dimension, int min_touched,
                                                int max_touched, int min_valid, int max_valid) {
    std::string m = std::string(func_name);
    if (min_touched < min_valid)
        m += " is accessed at " + std::to_string(min_touched) + ", which is before the min (" +
             std::to_string(min_valid) + ") in dimension " + std::to_string(dimension);
    else
        m += " is accessed at " + std::to_string(max_touched) + ", which is beyond the max (" +
             std::to_string(max_valid) + ") in dimension " + std::to_string(dimension);
    return report(uc, m, halide_error_code_access_out_of_bounds);
}

T2SP_WEAK int halide_error_buffer_allocation_too_large(void* uc, const char* buffer_name, uint64_t allocation_size,
                                                       uint64_t max_size) {
    return report(uc,
                  "Total allocation for buffer " + std::string(buffer_name) + " is " + std::to_string(allocation_size) +
                      ", which exceeds the maximum size of " + std::to_string(max_size),
                  halide_error_code_buffer_allocation_too_large);
}

T2SP_WEAK int halide_error_buffer_extents_negative(void* uc, const char* buffer_name, int dimension, int extent) {
    return report(uc,
                  "The extents for buffer " + std::string(buffer_name) + " dimension " + std::to_string(dimension) +
                      " is negative (" + std::to_string(extent) + ")",
                  halide_error_code_buffer_extents_negative);
}

T2SP_WEAK int halide_error_buffer_extents_too_large(void* uc, const char* buffer_name, int64_t actual_size,
                                                    int64_t max_size) {
    return report(uc,
                  "Product of extents for buffer " + std::string(buffer_name) + " is " + std::to_string(actual_size) +
                      ", which exceeds the maximum size of " + std::to_string(max_size),
                  halide_error_code_buffer_extents_too_large);
}

T2SP_WEAK int halide_error_constraint_violated(void* uc, const char* var, int val, const char* constrained_var,
                                               int constrained_val) {
    return report(uc,
                  "Constraint violated: " + std::string(var) + " (" + std::to_string(val) + ") == " +
                      std::string(constrained_var) + " (" + std::to_string(constrained_val) + ")",
                  halide_error_code_constraint_violated);
}

T2SP_WEAK int halide_error_out_of_memory(void* uc) {
    return report(uc, "Out of memory (halide_malloc returned NULL)", halide_error_code_out_of_memory);
}

T2SP_WEAK int halide_error_buffer_argument_is_null(void* uc, const char* buffer_name) {
    return report(uc, "Buffer argument " + std::string(buffer_name) + " is NULL",
                  halide_error_code_buffer_argument_is_null);
}

T2SP_WEAK int halide_error_host_is_null(void* uc, const char* func_name) {
    return report(uc,
                  "The host pointer of " + std::string(func_name) +
                      " is null, but the pipeline will access it on the host.",
                  halide_error_code_host_is_null);
}

T2SP_WEAK int halide_error_device_interface_no_device(void* uc) {
    return report(uc, "Buffer has a non-null device_interface but device is 0.",
                  halide_error_code_device_interface_no_device);
}

}  // extern "C"
