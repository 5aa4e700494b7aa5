// Implementation of the reference's roofline helper API (t2s/src/Roofline.h:24-31: DSPs, FMax,
// ExecTime, roofline) for the B200, so that the reference's host drivers run unmodified in their
// performance mode too (e.g. t2s/tests/performance/gemm/gemm-run-fpga.cpp:88-108). The reference
// implementation (t2s/src/Roofline.cpp) parses an FPGA synthesis report for the DSP count and
// fmax, reads exec_time.txt next to the bitstream and shells out to a matplotlib script; here
//   * DSPs() and FMax() describe the fp32 ceiling of this library's 3xTF32 path in the driver's own
//     formula `compute_roof = 2 * DSPs() * FMax()` (MFLOP/s): FMax() is the SM clock in MHz and DSPs()
//     the fp32-equivalent multiply-add lanes, 148 SMs x 2048 TF32 MACs per clock / 3 MMAs per product;
//   * ExecTime() is the device time of the last call (nanoseconds, CUDA events), the figure the
//     runtime also writes to exec_time.txt;
//   * roofline() prints the same "GFlops" line and draws roofline.png itself (a small PNG writer,
//     no Python needed).
// Link this file instead of Roofline.cpp + SharedUtilsInC.cpp.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "t2sp_b200/runtime.h"

int DSPs();
double FMax();
double ExecTime(const char* kernel_name = 0);
void roofline(double mem_bandwidth, double compute_roof, double number_ops, double number_bytes, double exec_time);
int DSPs_oneapi();
double FMax_oneapi();

namespace {

int sm_count_and_clock(double* mhz) {
    int sms = 148, khz = 1965000;  // B200 figures, used when no device answers
    int s = 0, k = 0;
    if (t2sp_b200_device_info(&s, &k) == 0 && s > 0 && k > 0) { sms = s; khz = k; }
    if (mhz) *mhz = khz / 1000.0;
    return sms;
}

// ---- minimal PNG (8-bit RGB, zlib "stored" blocks)
uint32_t crc32_of(const uint8_t* p, size_t n, uint32_t crc = 0xFFFFFFFFu) {
    static uint32_t table[256];
    static bool init = false;
    if (!init) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            table[i] = c;
        }
        init = true;
    }
    for (size_t i = 0; i < n; ++i) crc = table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
    return crc;
}

void put32(std::vector<uint8_t>& v, uint32_t x) {
    for (int s = 24; s >= 0; s -= 8) v.push_back(uint8_t(x >> s));
}

void chunk(std::vector<uint8_t>& out, const char* type, const std::vector<uint8_t>& data) {
    put32(out, uint32_t(data.size()));
    std::vector<uint8_t> body(type, type + 4);
    body.insert(body.end(), data.begin(), data.end());
    out.insert(out.end(), body.begin(), body.end());
    put32(out, crc32_of(body.data(), body.size()) ^ 0xFFFFFFFFu);
}

bool write_png(const char* path, int w, int h, const std::vector<uint8_t>& rgb) {
    std::vector<uint8_t> raw;
    for (int y = 0; y < h; ++y) {
        raw.push_back(0);
        raw.insert(raw.end(), rgb.begin() + size_t(y) * w * 3, rgb.begin() + size_t(y + 1) * w * 3);
    }
    std::vector<uint8_t> z = {0x78, 0x01};
    uint32_t a = 1, b = 0;
    for (uint8_t c : raw) { a = (a + c) % 65521; b = (b + a) % 65521; }
    for (size_t pos = 0; pos < raw.size();) {
        const size_t n = std::min<size_t>(65535, raw.size() - pos);
        z.push_back(pos + n == raw.size() ? 1 : 0);
        z.push_back(uint8_t(n)); z.push_back(uint8_t(n >> 8));
        z.push_back(uint8_t(~n)); z.push_back(uint8_t((~n) >> 8));
        z.insert(z.end(), raw.begin() + pos, raw.begin() + pos + n);
        pos += n;
    }
    put32(z, (b << 16) | a);
    std::vector<uint8_t> out = {0x89, 'P', 'N', 'G', 0x0D, 0x0A, 0x1A, 0x0A};
    std::vector<uint8_t> ihdr;
    put32(ihdr, w); put32(ihdr, h);
    ihdr.insert(ihdr.end(), {8, 2, 0, 0, 0});
    chunk(out, "IHDR", ihdr);
    chunk(out, "IDAT", z);
    chunk(out, "IEND", {});
    FILE* f = fopen(path, "wb");
    if (!f) return false;
    const bool ok = fwrite(out.data(), 1, out.size(), f) == out.size();
    fclose(f);
    return ok;
}

struct Canvas {
    int w, h;
    std::vector<uint8_t> px;
    Canvas(int w_, int h_) : w(w_), h(h_), px(size_t(w_) * h_ * 3, 255) {}
    void dot(int x, int y, uint8_t r, uint8_t g, uint8_t b) {
        if (x < 0 || y < 0 || x >= w || y >= h) return;
        uint8_t* p = &px[(size_t(y) * w + x) * 3];
        p[0] = r; p[1] = g; p[2] = b;
    }
    void line(double x0, double y0, double x1, double y1, uint8_t r, uint8_t g, uint8_t b, bool dashed) {
        const int n = int(fmax(fabs(x1 - x0), fabs(y1 - y0))) + 1;
        for (int i = 0; i <= n; ++i) {
            if (dashed && (i / 6) % 2) continue;
            dot(int(lround(x0 + (x1 - x0) * i / n)), int(lround(y0 + (y1 - y0) * i / n)), r, g, b);
        }
    }
};

}  // namespace

int DSPs() {
    double mhz;
    return int(lround(sm_count_and_clock(&mhz) * 2048.0 / 3.0));
}

double FMax() {
    double mhz = 0;
    sm_count_and_clock(&mhz);
    return mhz;
}

int DSPs_oneapi() { return DSPs(); }
double FMax_oneapi() { return FMax(); }

double ExecTime(const char* kernel_name) {
    const double ns = t2sp_b200_last_kernel_ns();
    if (kernel_name) printf("kernel %s exec time: %lf\n", kernel_name, ns);
    return ns;
}

// Same figure as t2s/src/Roofline.py: x = FLOP/byte, y = GFLOP/s; the bandwidth roof y = bw * x
// (dashed blue), the compute roof y = compute_roof / 1000 (dashed orange), the measured point (triangle).
void roofline(double mem_bandwidth, double compute_roof, double number_ops, double number_bytes, double exec_time) {
    if (exec_time == 0 || compute_roof == 0) {
        printf("Roofline parameters Error!\n");
        return;
    }
    printf("GFlops: %lf\n", number_ops / exec_time);
    const double y0 = compute_roof * 0.001, x0 = y0 / mem_bandwidth;
    const double x1 = number_ops / number_bytes, y1 = number_ops / exec_time;
    const double xmax = fmax(5 * x0, 1.5 * x1), ymax = fmax(2 * y0, 1.2 * y1);
    const int W = 640, H = 480, L = 50, B = 40;
    Canvas c(W, H);
    auto X = [&](double x) { return L + x / xmax * (W - L - 10); };
    auto Y = [&](double y) { return (H - B) - y / ymax * (H - B - 10); };
    c.line(L, H - B, W - 10, H - B, 0, 0, 0, false);
    c.line(L, H - B, L, 10, 0, 0, 0, false);
    c.line(X(0), Y(0), X(fmin(xmax, ymax / mem_bandwidth)), Y(fmin(ymax, mem_bandwidth * xmax)), 100, 149, 237, true);
    c.line(X(0), Y(y0), X(xmax), Y(y0), 255, 165, 0, true);
    for (int dy = 0; dy < 12; ++dy)
        for (int dx = -dy / 2; dx <= dy / 2; ++dx) c.dot(int(X(x1)) + dx, int(Y(y1)) - 6 + dy, 31, 119, 180);
    if (!write_png("roofline.png", W, H, c.px)) printf("cannot write roofline.png\n");
    printf("Roofline: %g FLOP/B, %g GFLOPS measured; compute roof %g GFLOPS, memory roof %g GB/s\n", x1, y1, y0, mem_bandwidth);
}
