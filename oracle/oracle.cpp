// TEST INFRASTRUCTURE ONLY. CPU restatement of the T2SP specifications that the B200
// kernels are checked against. Nothing in the shipped library includes, links or calls
// this file; only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs do.
//
// Every function follows the reduction order of the reference specification it cites
// (fp32 multiply, then fp32 add into a running sum that starts at 0, no FMA contraction:
// build with -ffp-contract=off), or, with acc64 != 0, accumulates the exact fp32 products
// in double as the "truth" the tolerances are measured against.
//
// Pinning: the reference stores no golden files; its tests recompute goldens in the driver
// (gemm-run-fpga.cpp:72-86, conv-run-fpga.cpp:71-93, capsule-run-fpga.cpp:76-104,
// aot/gemm-run.cpp:64-83). oracle/ref_interface.cpp exposes these functions under the
// reference's interface symbols so that those unmodified drivers validate them
// (tests/test_oracle_pins.py), and tests/golden/ holds the reference's deterministic
// SEQUENTIAL fixtures evaluated in closed form. MTTKRP has no reference test at all
// (util.h:464-481 is dead code): its parity is unpinned beyond the fp64 variant here.
//
// All tensors are dense, dimension 0 fastest, as Halide::Runtime::Buffer lays them out.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <thread>
#include <vector>

// Runs fn(0..n-1) over all host threads (or $ORACLE_THREADS); chunks are handed out dynamically.
// Each index owns its outputs, so results do not depend on the thread count.
template <class F>
static void par_for(int n, F fn) {
    int nt = int(std::thread::hardware_concurrency());
    if (const char* e = getenv("ORACLE_THREADS")) nt = atoi(e);
    if (nt < 1) nt = 1;
    if (nt > n) nt = n;
    if (nt <= 1) {
        for (int i = 0; i < n; ++i) fn(i);
        return;
    }
    std::atomic<int> next{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&] {
            for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
        });
    for (auto& th : pool) th.join();
}

extern "C" {

// Threads par_for will use (reported next to CPU timings).
int oracle_threads(void) {
    int nt = int(std::thread::hardware_concurrency());
    if (const char* e = getenv("ORACLE_THREADS")) nt = atoi(e);
    return nt < 1 ? 1 : nt;
}

static inline float bf16_to_f32(uint16_t h) {
    uint32_t w = uint32_t(h) << 16;
    float f;
    memcpy(&f, &w, 4);
    return f;
}

static inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t w;
    if (exp == 0) {
        if (man == 0) w = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            w = sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        w = sign | 0x7F800000u | man << 13;
    } else {
        w = sign | (exp + 112) << 23 | man << 13;
    }
    float f;
    memcpy(&f, &w, 4);
    return f;
}

// fp32 -> bf16, round to nearest even (how the tests and the bench quantise their inputs).
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t w;
    memcpy(&w, &f, 4);
    if ((w & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((w >> 16) | 0x40u);
    w += 0x7FFFu + ((w >> 16) & 1u);
    return uint16_t(w >> 16);
}

// ------------------------------------------------------------------------------ GEMM
// C(j,i) = sum_{k ascending} A(k,i) * B(j,k)         t2s/tests/performance/gemm/gemm.cpp:58-63
// A: (K,M)  B: (N,K)  C: (N,M); golden loop gemm-run-fpga.cpp:82-84.
void oracle_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int acc64) {
    par_for(M, [&](int i) {
        if (acc64) {
            std::vector<double> row(N, 0.0);
            for (int k = 0; k < K; ++k) {
                const double a = A[size_t(i) * K + k];
                const float* b = B + size_t(k) * N;
                for (int j = 0; j < N; ++j) row[j] += a * double(b[j]);
            }
            for (int j = 0; j < N; ++j) C[size_t(i) * N + j] = float(row[j]);
        } else {
            float* row = C + size_t(i) * N;
            for (int j = 0; j < N; ++j) row[j] = 0.0f;
            for (int k = 0; k < K; ++k) {
                const float a = A[size_t(i) * K + k];
                const float* b = B + size_t(k) * N;
                for (int j = 0; j < N; ++j) row[j] = row[j] + a * b[j];
            }
        }
    });
}

// Same contraction on 16-bit inputs (kind 0: bf16, 1: f16); products are exact in fp32.
void oracle_gemm_h16(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K, int kind, int acc64) {
    std::vector<float> Bf(size_t(N) * K);
    for (size_t x = 0; x < Bf.size(); ++x) Bf[x] = kind ? f16_to_f32(B[x]) : bf16_to_f32(B[x]);
    par_for(M, [&](int i) {
        std::vector<double> row64(acc64 ? N : 0, 0.0);
        std::vector<float> row32(acc64 ? 0 : N, 0.0f);
        for (int k = 0; k < K; ++k) {
            const float a = kind ? f16_to_f32(A[size_t(i) * K + k]) : bf16_to_f32(A[size_t(i) * K + k]);
            const float* b = Bf.data() + size_t(k) * N;
            if (acc64) for (int j = 0; j < N; ++j) row64[j] += double(a) * double(b[j]);
            else for (int j = 0; j < N; ++j) row32[j] = row32[j] + a * b[j];
        }
        for (int j = 0; j < N; ++j) C[size_t(i) * N + j] = acc64 ? float(row64[j]) : row32[j];
    });
}

// int8 x int8 -> int32, exact (integer variant of the same recurrence; small int32 cases in
// t2s/tests/correctness/gemm/gemm2.cpp:36-37).
void oracle_gemm_i8(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
    par_for(M, [&](int i) {
        int32_t* row = C + size_t(i) * N;
        for (int j = 0; j < N; ++j) row[j] = 0;
        for (int k = 0; k < K; ++k) {
            const int32_t a = A[size_t(i) * K + k];
            const int8_t* b = B + size_t(k) * N;
            for (int j = 0; j < N; ++j) row[j] += a * int32_t(b[j]);
        }
    });
}

// Rows [i0, i0+rows) only: bounded CPU work for spot checks and timing samples at sizes
// where the full product would take minutes.
void oracle_gemm_h16_rows(const uint16_t* A, const uint16_t* B, float* Crows, int i0, int rows, int N, int K,
                          int kind, int acc64) {
    oracle_gemm_h16(A + size_t(i0) * K, B, Crows, rows, N, K, kind, acc64);
}
void oracle_gemm_i8_rows(const int8_t* A, const int8_t* B, int32_t* Crows, int i0, int rows, int N, int K) {
    oracle_gemm_i8(A + size_t(i0) * K, B, Crows, rows, N, K);
}

// Plain C(N,M) -> tiled c(JJJ,III,JJ,II,J,I): element (jjj,iii,jj,ii,j,i) holds
// C(jjj + JJJ*jj + JJJ*JJ*j, iii + III*ii + III*II*i)          gemm-run-fpga.cpp:69,80-85
void oracle_gemm_tile_layout(const float* C, float* c6, int JJJ, int III, int JJ, int II, int J, int I) {
    const int N = JJJ * JJ * J;
    size_t o = 0;
    for (int i = 0; i < I; ++i)
        for (int j = 0; j < J; ++j)
            for (int ii = 0; ii < II; ++ii)
                for (int jj = 0; jj < JJ; ++jj)
                    for (int iii = 0; iii < III; ++iii)
                        for (int jjj = 0; jjj < JJJ; ++jjj) {
                            const int ti = iii + III * ii + III * II * i, tj = jjj + JJJ * jj + JJJ * JJ * j;
                            c6[o++] = C[size_t(ti) * N + tj];
                        }
}

// ------------------------------------------------------------------------------ CONV
// O2(co + CO*n, oy + OY*ox) = sum I2(ci + CI*n, (oy+ky) + IY*(ox+kx)) * K2(co + CO*kx, ci + CI*ky)
// accumulation order (outer to inner): ci_outer, kx, ky, cii with ci = cii + CII*ci_outer
//                                                   t2s/tests/performance/conv/conv.cpp:52-65
// (the driver's golden loop, conv-run-fpga.cpp:83-91, runs the whole ci range outermost, which is
//  this order with CII == 1; the spec's dependence chain nests cii inside ky, so CII is a
//  parameter here.)
void oracle_conv_f32(const float* I2, const float* K2, float* O2, int N, int CI, int CO, int KY, int KX, int OY,
                     int OX, int CII, int acc64) {
    const int IY = OY + KY - 1;
    const size_t ld_i = size_t(CI) * N, ld_k = size_t(CO) * KX, ld_o = size_t(CO) * N;
    if (CII <= 0 || CI % CII) CII = CI;
    par_for(OX * OY, [&](int pix) {
        const int ox = pix / OY, oy = pix % OY;
            for (int n = 0; n < N; ++n) {
                std::vector<double> r64(acc64 ? CO : 0, 0.0);
                std::vector<float> r32(acc64 ? 0 : CO, 0.0f);
                for (int cio = 0; cio < CI / CII; ++cio)
                    for (int kx = 0; kx < KX; ++kx)
                        for (int ky = 0; ky < KY; ++ky)
                            for (int cii = 0; cii < CII; ++cii) {
                                const int ci = cii + CII * cio;
                                const float x = I2[(ci + size_t(CI) * n) + ld_i * ((oy + ky) + size_t(IY) * (ox + kx))];
                                const float* w = K2 + size_t(CO) * kx + ld_k * (ci + size_t(CI) * ky);
                                if (acc64) for (int co = 0; co < CO; ++co) r64[co] += double(x) * double(w[co]);
                                else for (int co = 0; co < CO; ++co) r32[co] = r32[co] + x * w[co];
                            }
                float* o = O2 + size_t(CO) * n + ld_o * (oy + size_t(OY) * ox);
                for (int co = 0; co < CO; ++co) o[co] = acc64 ? float(r64[co]) : r32[co];
            }
    });
}

// Plain O2 -> tiled o(COOO,YYY,XXX,COO,YY,XX,Y,X,CO_outer,N)          conv-run-fpga.cpp:68,73-93
void oracle_conv_tile_layout(const float* O2, float* o10, int N, int COOO, int YYY, int XXX, int COO, int YY, int XX,
                             int Y, int X, int COout) {
    const int CO = COOO * COO * COout, OY = YYY * YY * Y;
    const size_t ld_o = size_t(CO) * N;
    size_t o = 0;
    for (int n = 0; n < N; ++n)
        for (int co = 0; co < COout; ++co)
            for (int x = 0; x < X; ++x)
                for (int y = 0; y < Y; ++y)
                    for (int xx = 0; xx < XX; ++xx)
                        for (int yy = 0; yy < YY; ++yy)
                            for (int coo = 0; coo < COO; ++coo)
                                for (int xxx = 0; xxx < XXX; ++xxx)
                                    for (int yyy = 0; yyy < YYY; ++yyy)
                                        for (int cooo = 0; cooo < COOO; ++cooo) {
                                            const int oy = yyy + YYY * yy + YYY * YY * y;
                                            const int ox = xxx + XXX * xx + XXX * XX * x;
                                            const int c = cooo + COOO * coo + COOO * COO * co;
                                            o10[o++] = O2[(c + size_t(CO) * n) + ld_o * (oy + size_t(OY) * ox)];
                                        }
}

// ------------------------------------------------------------------------------ CAPSULE
// V2(co + CO*my + CO*MY*mx + CO*MY*MX*nn, oy + OY*ox + OY*OX*n) =
//   sum P2(ci + CI*mk + CI*MK*mx + CI*MK*MX*nn, (s*oy+ky) + IY*(s*ox+kx) + IY*IX*n)
//     * W2(co + CO*my, cii + CII*ky + CII*KY*kx + CII*KY*KX*ci_o + CI*KY*KX*mk)
// accumulation order (outer to inner): mk, ci_outer, kx, ky, cii
//                                         t2s/tests/performance/capsule/capsule.cpp:52-66
void oracle_capsule_f32(const float* P2, const float* W2, float* V2, int N, int NN, int CI, int CII, int CO, int KY,
                        int KX, int OY, int OX, int MY, int MX, int MK, int s, int acc64) {
    const int IY = s * OY + KY - s, IX = s * OX + KX - s;
    const size_t ld_p = size_t(CI) * MK * MX * NN, ld_w = size_t(CO) * MY, ld_v = size_t(CO) * MY * MX * NN;
    const int NW = CO * MY;
    par_for(N * OX, [&](int nx) {
        const int n = nx / OX, ox = nx % OX;
            for (int oy = 0; oy < OY; ++oy)
                for (int nn = 0; nn < NN; ++nn)
                    for (int mx = 0; mx < MX; ++mx) {
                        std::vector<double> r64(acc64 ? NW : 0, 0.0);
                        std::vector<float> r32(acc64 ? 0 : NW, 0.0f);
                        for (int mk = 0; mk < MK; ++mk)
                            for (int cio = 0; cio < CI / CII; ++cio)
                                for (int kx = 0; kx < KX; ++kx)
                                    for (int ky = 0; ky < KY; ++ky)
                                        for (int cii = 0; cii < CII; ++cii) {
                                            const int ci = cii + CII * cio;
                                            const size_t prow = ci + size_t(CI) * mk + size_t(CI) * MK * mx + size_t(CI) * MK * MX * nn;
                                            const size_t pcol = (s * oy + ky) + size_t(IY) * (s * ox + kx) + size_t(IY) * IX * n;
                                            const float x = P2[prow + ld_p * pcol];
                                            const size_t wcol = cii + size_t(CII) * ky + size_t(CII) * KY * kx +
                                                                size_t(CII) * KY * KX * cio + size_t(CI) * KY * KX * mk;
                                            const float* w = W2 + ld_w * wcol;
                                            if (acc64) for (int c = 0; c < NW; ++c) r64[c] += double(x) * double(w[c]);
                                            else for (int c = 0; c < NW; ++c) r32[c] = r32[c] + x * w[c];
                                        }
                        float* v = V2 + size_t(NW) * mx + size_t(NW) * MX * nn + ld_v * (oy + size_t(OY) * ox + size_t(OY) * OX * n);
                        for (int c = 0; c < NW; ++c) v[c] = acc64 ? float(r64[c]) : r32[c];
                    }
    });
}

// Plain V2 -> tiled V(COOO,YYY_XXX,YY_XX,Y_X,MY,MX,COO,NN,CO_outer,N); pixel slots beyond OY*OX hold 0.
//                                                                capsule-run-fpga.cpp:73,78-104
void oracle_capsule_tile_layout(const float* V2, float* v10, int N, int NN, int COOO, int COO, int COout, int YYY_XXX,
                                int YY_XX, int Y_X, int MY, int MX, int OY, int OX) {
    const int CO = COOO * COO * COout;
    const size_t ld_v = size_t(CO) * MY * MX * NN;
    size_t o = 0;
    for (int n = 0; n < N; ++n)
        for (int co = 0; co < COout; ++co)
            for (int nn = 0; nn < NN; ++nn)
                for (int coo = 0; coo < COO; ++coo)
                    for (int mx = 0; mx < MX; ++mx)
                        for (int my = 0; my < MY; ++my)
                            for (int y_x = 0; y_x < Y_X; ++y_x)
                                for (int yy_xx = 0; yy_xx < YY_XX; ++yy_xx)
                                    for (int yyy_xxx = 0; yyy_xxx < YYY_XXX; ++yyy_xxx)
                                        for (int cooo = 0; cooo < COOO; ++cooo) {
                                            const int pix = yyy_xxx + YYY_XXX * yy_xx + YYY_XXX * YY_XX * y_x;
                                            float val = 0.0f;
                                            if (pix < OY * OX) {
                                                const int oy = pix % OY, ox = pix / OY;
                                                const int c = cooo + COOO * coo + COOO * COO * co;
                                                val = V2[(c + size_t(CO) * my + size_t(CO) * MY * mx + size_t(CO) * MY * MX * nn) +
                                                         ld_v * (oy + size_t(OY) * ox + size_t(OY) * OX * n)];
                                            }
                                            v10[o++] = val;
                                        }
}

// ------------------------------------------------------------------------------ TTM
// c(i,j,k) = sum_{l ascending} a(l,i,j) * b(l,k)        t2s/tests/correctness/util/util.h:428-441,
// spec t2s/tests/correctness/buffer/tmm_small.cpp:60-64.   a: (L,I,J)  b: (L,K)  c: (I,J,K)
void oracle_ttm_f32(const float* a, const float* b, float* c, int L, int I, int J, int K, int acc64) {
    par_for(K * J, [&](int kj) {
        const int k = kj / J, j = kj % J;
            for (int i = 0; i < I; ++i) {
                const float* ar = a + size_t(L) * (i + size_t(I) * j);
                const float* br = b + size_t(L) * k;
                float s32 = 0.0f;
                double s64 = 0.0;
                if (acc64) for (int l = 0; l < L; ++l) s64 += double(ar[l]) * double(br[l]);
                else for (int l = 0; l < L; ++l) s32 = s32 + ar[l] * br[l];
                c[i + size_t(I) * (j + size_t(J) * k)] = acc64 ? float(s64) : s32;
            }
    });
}

// Plain c(I,J,K) -> tiled (JJ,KK,II,KKK,JJJ,III,OK,OJ,OI)                tmm_small.cpp:116-129,141-154
void oracle_ttm_tile_layout(const float* c, float* c9, int JJ, int KK, int II, int KKK, int JJJ, int III, int OK,
                            int OJ, int OI) {
    const int I = III * II * OI, J = JJJ * JJ * OJ;
    size_t o = 0;
    for (int oi = 0; oi < OI; ++oi)
        for (int oj = 0; oj < OJ; ++oj)
            for (int ok = 0; ok < OK; ++ok)
                for (int iii = 0; iii < III; ++iii)
                    for (int jjj = 0; jjj < JJJ; ++jjj)
                        for (int kkk = 0; kkk < KKK; ++kkk)
                            for (int ii = 0; ii < II; ++ii)
                                for (int kk = 0; kk < KK; ++kk)
                                    for (int jj = 0; jj < JJ; ++jj) {
                                        const int i = iii + III * ii + III * II * oi;
                                        const int j = jjj + JJJ * jj + JJJ * JJ * oj;
                                        const int k = kkk + KKK * kk + KKK * KK * ok;
                                        c9[o++] = c[i + size_t(I) * (j + size_t(J) * k)];
                                    }
}

// ------------------------------------------------------------------------------ MTTKRP
// d(i,r) = sum_{k ascending} ( sum_{l ascending} a(l,i,k) * c(l,r) ) * b(k,r)
// t2s/tests/correctness/util/util.h:464-481 with the outer bound `i < K` read as `i < I`.
// a: (L,I,K)  b: (K,R)  c: (L,R)  d: (I,R)
void oracle_mttkrp_f32(const float* a, const float* b, const float* c, float* d, int L, int I, int K, int R,
                       int acc64) {
    par_for(R * I, [&](int ri) {
        const int r = ri / I, i = ri % I;
        {
            float d32 = 0.0f;
            double d64 = 0.0;
            for (int k = 0; k < K; ++k) {
                const float* ar = a + size_t(L) * (i + size_t(I) * k);
                const float* cr = c + size_t(L) * r;
                if (acc64) {
                    double e = 0.0;
                    for (int l = 0; l < L; ++l) e += double(ar[l]) * double(cr[l]);
                    d64 += e * double(b[k + size_t(K) * r]);
                } else {
                    float e = 0.0f;
                    for (int l = 0; l < L; ++l) e = e + ar[l] * cr[l];
                    d32 = d32 + e * b[k + size_t(K) * r];
                }
            }
            d[i + size_t(I) * r] = acc64 ? float(d64) : d32;
        }
    });
}

// ------------------------------------------------------------------------------ comparison metrics
// max over elements of |got - ref| / max(|ref|, floor); with floor = 0 the strict elementwise
// relative error (0/0 counts as 0).
double oracle_max_rel_err(const float* got, const float* ref, size_t n, double floor_abs) {
    double worst = 0.0;
    for (size_t x = 0; x < n; ++x) {
        const double g = got[x], r = ref[x];
        const double den = fmax(fabs(r), floor_abs);
        const double e = den > 0 ? fabs(g - r) / den : (g == r ? 0.0 : INFINITY);
        if (!(e <= worst)) worst = e;
    }
    return worst;
}

double oracle_max_abs(const float* x, size_t n) {
    double m = 0.0;
    for (size_t i = 0; i < n; ++i) m = fmax(m, fabs(double(x[i])));
    return m;
}

// ------------------------------------------------------------------------------ SYRK (folded output)
// Out(jjj,iii,jj,ii,j,i) = Alpha * sum_{k ascending} A(k,r) * A(k,c) + Beta * C(c,r)
//                                                   t2s/tests/performance/syrk/syrk.cpp:38-73
// with ti = iii + III*ii + III*II*i, tj = jjj + III*jj + III*II*j, N = III*II*I and
//   (r, c) = (N-1-ti, N-1-tj) where i >= j ("is_bot"), (ti, tj - III*II) otherwise;
// loop bounds j in [0, I], i in [0, I/2) (syrk.cpp:80-86). A: (K,N) k innermost; C: (N,N), element
// C(x, y) at y*ldc + x; O dense (III,III,II,II,I+1,Irows), only rows i < I/2 are written.
// Golden loop: syrk-run-fpga.cpp:70-106.
void oracle_syrk_f32(const float* A, const float* C, float* O, int K, int III, int II, int I, int Irows, int ldc,
                     float alpha, float beta, int acc64) {
    const int t = III * II, N = t * I;
    par_for((I / 2) * (I + 1), [&](int ij) {
        const int i = ij / (I + 1), j = ij % (I + 1);
        for (int ii = 0; ii < II; ++ii)
            for (int jj = 0; jj < II; ++jj)
                for (int iii = 0; iii < III; ++iii)
                    for (int jjj = 0; jjj < III; ++jjj) {
                        const int ti = iii + III * ii + t * i, tj = jjj + III * jj + t * j;
                        const int r = i >= j ? N - 1 - ti : ti, c = i >= j ? N - 1 - tj : tj - t;
                        const float* ar = A + size_t(r) * K;
                        const float* ac = A + size_t(c) * K;
                        float v;
                        if (acc64) {
                            double z = 0.0;
                            for (int k = 0; k < K; ++k) z += double(ar[k]) * double(ac[k]);
                            v = float(double(alpha) * z + double(beta) * double(C[size_t(r) * ldc + c]));
                        } else {
                            float z = 0.f;
                            for (int k = 0; k < K; ++k) z = z + ar[k] * ac[k];
                            v = alpha * z + beta * C[size_t(r) * ldc + c];
                        }
                        const size_t off = jjj + size_t(III) * (iii + size_t(III) * (jj + size_t(II) * (ii + size_t(II) * (j + size_t(I + 1) * i))));
                        (void)Irows;
                        O[off] = v;
                    }
    });
}

// GER of t2s/tests/performance/ger/ger.cpp:34-62: Out(kkk,iii,ii,kk,k,i) = A(tk, ti) + X(ti) * Y(tk), one
// fp32 multiply and one fp32 add (this file is built with -ffp-contract=off). A: (TK, TI), k innermost
// with row pitch lda; O dense (KKK,III,II,KK,K,I). Golden loop: ger-run-fpga.cpp:70-82.
void oracle_ger_f32(const float* A, const float* X, const float* Y, float* O, int KKK, int III, int II, int KK, int K,
                    int I, int lda) {
    par_for(I * K, [&](int ik) {
        const int i = ik / K, k = ik % K;
        for (int kk = 0; kk < KK; ++kk)
            for (int ii = 0; ii < II; ++ii)
                for (int iii = 0; iii < III; ++iii)
                    for (int kkk = 0; kkk < KKK; ++kkk) {
                        const size_t ti = iii + size_t(III) * (ii + size_t(II) * i);
                        const size_t tk = kkk + size_t(KKK) * (kk + size_t(KK) * k);
                        const float prod = X[ti] * Y[tk];
                        const size_t off = kkk + size_t(KKK) * (iii + size_t(III) * (ii + size_t(II) * (kk + size_t(KK) * (k + size_t(K) * i))));
                        O[off] = A[ti * lda + tk] + prod;
                    }
    });
}

// ------------------------------------------------------------------------------ N-D operand layouts (oneAPI flow)
// conv:    I(iy, ix, ci, n), K(ky, kx, ci, co)      t2s/tests/correctness/oneapi-integration/oneapi-target-5-conv.cpp:58-62
// capsule: P(mk, mx, ci, iy, ix, n), W(my, mk, ci, co, ky, kx)                        oneapi-target-6-capsule.cpp:57-61
// Same sums and summation order as the 2-D specifications; these re-lay the operands out into the
// 2-D buffers of oracle_conv_f32 / oracle_capsule_f32 (CII = CI) on the CPU.
void oracle_conv_nd_to_2d(const float* I4, const float* K4, float* I2, float* K2, int N, int CI, int CO, int KY, int KX,
                          int IY, int IX) {
    for (int n = 0; n < N; ++n)
        for (int ci = 0; ci < CI; ++ci)
            for (int ix = 0; ix < IX; ++ix)
                for (int iy = 0; iy < IY; ++iy)
                    I2[(size_t(ci) + size_t(CI) * n) + size_t(CI) * N * (iy + size_t(IY) * ix)] =
                        I4[iy + size_t(IY) * (ix + size_t(IX) * (ci + size_t(CI) * n))];
    for (int co = 0; co < CO; ++co)
        for (int ci = 0; ci < CI; ++ci)
            for (int kx = 0; kx < KX; ++kx)
                for (int ky = 0; ky < KY; ++ky)
                    K2[(size_t(co) + size_t(CO) * kx) + size_t(CO) * KX * (ci + size_t(CI) * ky)] =
                        K4[ky + size_t(KY) * (kx + size_t(KX) * (ci + size_t(CI) * co))];
}

void oracle_capsule_nd_to_2d(const float* P6, const float* W6, float* P2, float* W2, int N, int CI, int CO, int KY, int KX,
                             int IY, int IX, int MY, int MX, int MK) {
    const size_t p0 = size_t(CI) * MK * MX;  // extent of dimension 0 of P2 (NN = 1)
    for (int n = 0; n < N; ++n)
        for (int ix = 0; ix < IX; ++ix)
            for (int iy = 0; iy < IY; ++iy)
                for (int ci = 0; ci < CI; ++ci)
                    for (int mx = 0; mx < MX; ++mx)
                        for (int mk = 0; mk < MK; ++mk)
                            P2[(ci + size_t(CI) * (mk + size_t(MK) * mx)) + p0 * (iy + size_t(IY) * (ix + size_t(IX) * n))] =
                                P6[mk + size_t(MK) * (mx + size_t(MX) * (ci + size_t(CI) * (iy + size_t(IY) * (ix + size_t(IX) * n))))];
    const size_t w0 = size_t(CO) * MY;
    for (int kx = 0; kx < KX; ++kx)
        for (int ky = 0; ky < KY; ++ky)
            for (int co = 0; co < CO; ++co)
                for (int ci = 0; ci < CI; ++ci)
                    for (int mk = 0; mk < MK; ++mk)
                        for (int my = 0; my < MY; ++my)
                            W2[(co + size_t(CO) * my) + w0 * (ci + size_t(CI) * (ky + size_t(KY) * (kx + size_t(KX) * mk)))] =
                                W6[my + size_t(MY) * (mk + size_t(MK) * (ci + size_t(CI) * (co + size_t(CO) * (ky + size_t(KY) * kx))))];
}

}  // extern "C"
