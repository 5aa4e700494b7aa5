// TEST INFRASTRUCTURE ONLY: stands in for the generated "capsule.generated_oneapi_header.h" when the
// reference's oneAPI driver is linked against the CPU oracle (oracle/ref_interface.cpp) to pin it.
#pragma once
#include "t2sp_b200/driver_prelude.h"
#ifndef T2SP_B200_SYCL_STANDINS
#define T2SP_B200_SYCL_STANDINS 1
namespace sycl { namespace ext { namespace intel {
struct fpga_selector {};
struct fpga_emulator_selector {};
}}}
#endif
extern "C" int oracle_pin_capsule_nd(struct halide_buffer_t*, struct halide_buffer_t*, struct halide_buffer_t*);
template <class DeviceSelector>
inline double capsule(DeviceSelector&, struct halide_buffer_t* a, struct halide_buffer_t* b, struct halide_buffer_t* c) {
    return oracle_pin_capsule_nd(a, b, c) == 0 ? 1.0 : -1.0;
}
