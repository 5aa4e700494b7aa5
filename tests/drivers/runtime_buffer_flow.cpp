// A host program written the way the reference's callers are (Halide::Runtime::Buffer objects from
// the reference tree's header-only HalideBuffer.h), exercising this library's device interface table
// through the Buffer class itself: copy_to_device, device_malloc, copy_to_host, crops and slices of a
// device-resident buffer, a wrapped native pointer, device_sync, and the destructor's device_free
// (HalideBuffer.h:229-252, 388, 418, 1613-1713; table layout HalideRuntime.h:713-738).
// Built by oracle/build_ref_drivers.sh against libt2sp_b200.so; prints "Success" when all checks hold.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <utility>
#include <vector>

#include "HalideBuffer.h"
#include "t2sp_b200/runtime.h"

using Halide::Runtime::Buffer;

// declared by the reference's HalideRuntimeOpenCL.h; exported by the library under the same name
extern "C" const struct halide_device_interface_t* halide_opencl_device_interface();

static int fails = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::printf("FAILED line %d: %s\n", __LINE__, #cond);            \
            ++fails;                                                         \
        }                                                                    \
    } while (0)

int main() {
    const halide_device_interface_t* iface = t2sp_b200_device_interface();
    CHECK(iface && iface->device_malloc && iface->device_free && iface->copy_to_host && iface->copy_to_device &&
          iface->device_crop && iface->device_slice && iface->device_release_crop && iface->wrap_native &&
          iface->detach_native && iface->device_sync && iface->buffer_copy && iface->device_and_host_malloc &&
          iface->device_and_host_free && iface->compute_capability && iface->device_release);
    CHECK(halide_opencl_device_interface() == iface);
    int major = 0, minor = 0;
    CHECK(iface->compute_capability(nullptr, &major, &minor) == 0 && major == 10);

    const int M = 256, N = 192, K = 128;
    std::vector<double> want(size_t(M) * N);
    {
        Buffer<float> a(K, M), b(N, K), c(N, M);
        for (int i = 0; i < M; ++i)
            for (int k = 0; k < K; ++k) a(k, i) = float((i * 7 + k * 3) % 11 - 5) * 0.25f;
        for (int k = 0; k < K; ++k)
            for (int j = 0; j < N; ++j) b(j, k) = float((j * 5 + k) % 13 - 6) * 0.5f;
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j) {
                double s = 0;
                for (int k = 0; k < K; ++k) s += double(a(k, i)) * double(b(j, k));
                want[size_t(i) * N + j] = s;
                c(j, i) = -1.0f;
            }
        a.set_host_dirty();
        b.set_host_dirty();
        CHECK(a.copy_to_device(iface) == 0);                                       // through the table
        CHECK(halide_copy_to_device(nullptr, b.raw_buffer(), iface) == 0);         // under the reference runtime's name
        CHECK(a.has_device_allocation() && b.has_device_allocation() && !a.host_dirty() && !b.host_dirty());
        CHECK(c.device_malloc(iface) == 0);
        CHECK(t2sp_b200_gemm(a, b, c, nullptr) == 0);
        CHECK(c.device_dirty());
        const Buffer<float>& c_read = c;  // element access through a non-const Buffer marks the host copy dirty
        const float* c_host = c.data();   // and the class refuses element reads while the device copy is the newer one
        CHECK(c_host[0] == -1.0f);                                                 // the host copy is still the old one
        CHECK(c.device_sync() == 0);

        // a crop and a slice of the device-resident result: same allocation, shifted address
        Buffer<float> rows = c.cropped(1, 64, 32);                                 // rows 64..95
        CHECK(rows.has_device_allocation() && rows.raw_buffer()->device == c.raw_buffer()->device + size_t(64) * N * 4);
        Buffer<float> one = c.sliced(1, 100);                                      // row 100 as a 1-D buffer
        CHECK(one.dimensions() == 1 && one.raw_buffer()->device == c.raw_buffer()->device + size_t(100) * N * 4);
        rows.set_device_dirty();
        CHECK(rows.copy_to_host() == 0);
        const Buffer<float>& rows_read = rows;
        for (int i = 64; i < 96; ++i)
            for (int j = 0; j < N; ++j) CHECK(std::fabs(rows_read(j, i) - want[size_t(i) * N + j]) <= 1e-4);
        CHECK(c_host[0] == -1.0f && c_host[size_t(63) * N] == -1.0f && c_host[size_t(96) * N] == -1.0f);  // only the crop came back

        CHECK(c.copy_to_host() == 0);
        CHECK(!c.device_dirty());
        double worst = 0;
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j) worst = std::fmax(worst, std::fabs(c_read(j, i) - want[size_t(i) * N + j]));
        std::printf("gemm through Halide::Runtime::Buffer: max |diff| %.3e\n", worst);
        CHECK(worst <= 1e-4);

        // a second buffer wraps the same device memory, then lets go of it without freeing it
        Buffer<float> alias(nullptr, N, M);
        CHECK(alias.device_wrap_native(iface, c.raw_buffer()->device) == 0);
        CHECK(alias.raw_buffer()->device == c.raw_buffer()->device);
        CHECK(alias.device_detach_native() == 0 && !alias.has_device_allocation());

        // device -> host through buffer_copy into a fresh host buffer of the same shape
        Buffer<float> back(N, M);
        CHECK(iface->buffer_copy(nullptr, c.raw_buffer(), nullptr, back.raw_buffer()) == 0);
        CHECK(std::fabs(std::as_const(back)(5, 7) - want[size_t(7) * N + 5]) <= 1e-4);

        CHECK(a.device_free() == 0 && !a.has_device_allocation());
        // b, c, rows and one go out of scope here: the crops release, then the owners free through the table
    }
    {
        Buffer<float> both(nullptr, 64, 16);
        CHECK(both.device_and_host_malloc(iface) == 0 && both.data() != nullptr && both.has_device_allocation());
        CHECK(both.device_and_host_free(iface) == 0 && !both.has_device_allocation());
    }
    // the library is still in working order afterwards
    {
        Buffer<float> a(64, 128), b(128, 64), c(128, 128);
        a.fill(1.0f);
        b.fill(0.5f);
        CHECK(t2sp_b200_gemm(a, b, c, nullptr) == 0);
        CHECK(std::as_const(c)(3, 5) == 32.0f);
    }
    if (fails) {
        std::printf("FAILED: %d checks\n", fails);
        return 1;
    }
    std::printf("Success\n");
    return 0;
}
