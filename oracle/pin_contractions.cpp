// Pins the oracle's TTM and MTTKRP restatements with the reference's own golden loops: compiled
// (by build_ref_drivers.sh) together with the reference's unmodified test helper
// t2s/tests/correctness/util/util.h, found in the mounted reference tree, it runs
// get_result_of_tmm (util.h:428-441) and get_result_of_mttkrp (util.h:464-481) on seeded random
// inputs and demands that oracle_ttm_f32 / oracle_mttkrp_f32 return the same bits (same loop
// order, unfused multiply-add on both sides), and that the fp64-accumulated variants agree to
// rounding. The MTTKRP helper's outer loop runs `i < K`, so the shapes here have I == K, where
// that bound and the intended `i < I` coincide. Test infrastructure only.
#include "util.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" {
void oracle_ttm_f32(const float* a, const float* b, float* c, int L, int I, int J, int K, int acc64);
void oracle_mttkrp_f32(const float* a, const float* b, const float* c, float* d, int L, int I, int K, int R, int acc64);
}

namespace {

uint64_t g_state = 0x9E3779B97F4A7C15ull;
float next_uniform() {  // uniform in [-1, 1), 24 random bits
    g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
    return static_cast<float>(static_cast<int64_t>(g_state >> 40) - (1 << 23)) / static_cast<float>(1 << 23);
}

template <typename B>
void fill(B& buf) {
    buf.for_each_value([](float& v) { v = next_uniform(); });
}

// Dense copy in Halide order (dimension 0 fastest), the layout the oracle takes.
template <typename B>
std::vector<float> dense(const B& buf) {
    std::vector<float> out(buf.number_of_elements());
    B tmp = buf.copy();
    std::memcpy(out.data(), tmp.data(), out.size() * sizeof(float));
    return out;
}

int compare(const char* what, const std::vector<float>& got, const std::vector<float>& want, bool exact, double tol) {
    double worst = 0, scale = 0;
    size_t bad = 0;
    for (size_t i = 0; i < want.size(); ++i) {
        scale = std::max(scale, std::fabs(static_cast<double>(want[i])));
        worst = std::max(worst, std::fabs(static_cast<double>(got[i]) - want[i]));
        if (exact && std::memcmp(&got[i], &want[i], 4) != 0) ++bad;
    }
    const bool ok = exact ? bad == 0 : worst <= tol * scale;
    std::printf("%s: %zu elements, max |diff| %.3e of %.3e, %zu differing bit patterns -> %s\n", what, want.size(), worst,
                scale, bad, ok ? "ok" : "MISMATCH");
    return ok ? 0 : 1;
}

template <int L, int I, int J, int K>
int pin_ttm() {
    Halide::Buffer<float> a(L, I, J), b(L, K);
    fill(a);
    fill(b);
    Halide::Buffer<float> c = get_result_of_tmm<float, L, I, J, K>(a, b);
    const std::vector<float> av = dense(a), bv = dense(b), want = dense(c);
    std::vector<float> got(want.size()), got64(want.size());
    oracle_ttm_f32(av.data(), bv.data(), got.data(), L, I, J, K, 0);
    oracle_ttm_f32(av.data(), bv.data(), got64.data(), L, I, J, K, 1);
    return compare("ttm spec order", got, want, true, 0) + compare("ttm fp64 accumulation", got64, want, false, 1e-5);
}

template <int L, int I, int R>
int pin_mttkrp() {
    constexpr int K = I;  // see the header comment
    Halide::Buffer<float> a(L, I, K), b(K, R), c(L, R);
    fill(a);
    fill(b);
    fill(c);
    Halide::Buffer<float> d = get_result_of_mttkrp<float, L, I, R, K>(a, b, c);
    const std::vector<float> av = dense(a), bv = dense(b), cv = dense(c), want = dense(d);
    std::vector<float> got(want.size()), got64(want.size());
    oracle_mttkrp_f32(av.data(), bv.data(), cv.data(), got.data(), L, I, K, R, 0);
    oracle_mttkrp_f32(av.data(), bv.data(), cv.data(), got64.data(), L, I, K, R, 1);
    return compare("mttkrp spec order", got, want, true, 0) + compare("mttkrp fp64 accumulation", got64, want, false, 1e-5);
}

}  // namespace

int main() {
    int bad = 0;
    bad += pin_ttm<8, 8, 8, 8>();       // the size of tmm_small.cpp
    bad += pin_ttm<40, 12, 7, 20>();
    bad += pin_ttm<96, 16, 5, 33>();
    bad += pin_mttkrp<8, 8, 8>();
    bad += pin_mttkrp<36, 24, 10>();
    bad += pin_mttkrp<64, 17, 40>();
    if (bad) {
        std::printf("FAILED: %d comparisons\n", bad);
        return 1;
    }
    std::printf("Success: the oracle's TTM and MTTKRP match get_result_of_tmm / get_result_of_mttkrp\n");
    return 0;
}
