// Stand-in for the compiler's umbrella header, only for compiling the reference's test helper
// t2s/tests/correctness/util/util.h on a machine without libHalide: its golden loops
// (get_result_of_tmm :428-441, get_result_of_mttkrp :464-481) need nothing but a buffer class, which
// the header-only Halide::Runtime::Buffer of the reference tree provides. The one non-template
// function in that file (print_type :494-531) names a handful of IR node types through
// Expr::as<T>(); they are declared here as empty types so that it compiles, and are never used.
// Test infrastructure: nothing in the product includes this file.
#pragma once
#include "HalideBuffer.h"

namespace Halide {

template <typename T = void, int D = 4>
using Buffer = Halide::Runtime::Buffer<T, D>;

struct Expr {
    template <typename T>
    const T *as() const { return nullptr; }
};

namespace Internal {
struct StringImm {}; struct IntImm {}; struct FloatImm {}; struct Cast {}; struct Add {}; struct Sub {};
struct Mul {}; struct Div {}; struct Call {}; struct Select {}; struct Shuffle {}; struct Ramp {};
struct Load {}; struct Store {}; struct Broadcast {}; struct Let {}; struct Variable {};
}  // namespace Internal

}  // namespace Halide
