// What sits behind include/l0/l0_rt_helpers.h and include/cm/cm_rt.h: images / surfaces as device buffers of this library and the launch
// of the operator a "kernel" names (the reference side: t2s/tests/performance/util/l0_rt_helpers.h:137-153,
// 326-346 over Level Zero).
#include <stdio.h>
#include <string.h>

#include "t2sp_b200/runtime.h"

namespace {
struct Image {
    halide_buffer_t buf;
    halide_dimension_t dims[2];
};
}  // namespace

extern "C" void* t2sp_l0_image_create(unsigned width, unsigned height, const void* data) {
    Image* im = new Image();
    memset(im, 0, sizeof(*im));
    const uint32_t f32 = 2u | (32u << 8) | (1u << 16);  // halide_type_t{float, 32 bits, 1 lane}
    memcpy(&im->buf.type, &f32, 4);
    im->buf.dimensions = 2;
    im->buf.dim = im->dims;
    im->dims[0].extent = int(width); im->dims[0].stride = 1;
    im->dims[1].extent = int(height); im->dims[1].stride = int(width);
    if (t2sp_b200_device_malloc(&im->buf) != 0) { delete im; return nullptr; }
    if (data) {
        im->buf.host = const_cast<uint8_t*>(static_cast<const uint8_t*>(data));
        im->buf.flags |= 1;  // host_dirty: the upload below takes the host copy
        const int rc = t2sp_b200_copy_to_device(&im->buf);
        im->buf.host = nullptr;
        if (rc != 0) { t2sp_b200_device_free(&im->buf); delete im; return nullptr; }
    }
    return im;
}

extern "C" int t2sp_l0_image_write(void* image, const void* src) {
    Image* im = static_cast<Image*>(image);
    im->buf.host = const_cast<uint8_t*>(static_cast<const uint8_t*>(src));
    im->buf.flags |= 1;
    const int rc = t2sp_b200_copy_to_device(&im->buf);
    im->buf.host = nullptr;
    return rc;
}

extern "C" double t2sp_l0_last_kernel_ns(void) { return t2sp_b200_last_kernel_ns(); }

extern "C" int t2sp_l0_image_read(void* image, void* dst) {
    Image* im = static_cast<Image*>(image);
    im->buf.host = static_cast<uint8_t*>(dst);
    im->buf.flags |= 2;  // device_dirty: the device holds the current data
    const int rc = t2sp_b200_copy_to_host(&im->buf);
    im->buf.host = nullptr;
    return rc;
}

extern "C" void t2sp_l0_image_destroy(void* image) {
    Image* im = static_cast<Image*>(image);
    if (!im) return;
    t2sp_b200_device_free(&im->buf);
    delete im;
}

extern "C" int t2sp_l0_run(int op, const int* d, void* const* images) {
    halide_buffer_t* in0 = &static_cast<Image*>(images[0])->buf;
    halide_buffer_t* in1 = &static_cast<Image*>(images[1])->buf;
    halide_buffer_t* out = &static_cast<Image*>(images[2])->buf;
    if (op == 0) return t2sp_b200_gemm(in0, in1, out, nullptr);  // plain C(total_j, total_i) (gemm.cpp:89)
    if (op == 1) {
        t2sp_conv_desc c;
        memset(&c, 0, sizeof(c));
        c.CI = d[0]; c.CO = d[1]; c.KY = d[2]; c.KX = d[3]; c.OY = d[4]; c.OX = d[5];
        return t2sp_b200_conv(in0, in1, out, &c);
    }
    t2sp_capsule_desc c;
    memset(&c, 0, sizeof(c));
    c.CI = d[0]; c.CII = d[1]; c.CO = d[2]; c.KY = d[3]; c.KX = d[4]; c.OY = d[5]; c.OX = d[6];
    c.MY = d[7]; c.MX = d[8]; c.MK = d[9]; c.NN = d[10]; c.stride = d[11];
    return t2sp_b200_capsule(in0, in1, out, &c);
}
