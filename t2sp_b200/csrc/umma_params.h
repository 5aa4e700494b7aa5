// Parameter block shared by the host lowering code and the contraction kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace t2sp {

enum : int { AR_F16 = 0, AR_TF32X3 = 1, AR_I8 = 2 };
enum : int { OP_GEMM = 0, OP_TTM = 1, OP_CONV = 2, OP_CAPSULE = 3, OP_MTTKRP = 4 };
enum : int { EPI_ROWMAJOR = 0, EPI_COLMAJOR = 1, EPI_SCATTER = 2, EPI_TMA = 3 };

// Status bits written by a kernel whose wait ran out (which role gave up).
enum : unsigned {
    ST_TIMEOUT_PRODUCER = 1u,
    ST_TIMEOUT_MMA = 2u,
    ST_TIMEOUT_EPILOGUE = 4u,
    ST_TIMEOUT_SPLITTER = 8u,
};

constexpr long long kWaitTimeoutCycles = 4000000000ll;  // SM cycles: 2 s at 1965 MHz, 4 s at 1 GHz
constexpr int kBlockM = 128;
constexpr int kMaxDigits = 8;
constexpr int kCStageBytes = 4 * 4096;  // EPI_TMA: one 32 x 32 fp32 staging tile per epilogue warp

// offset(x) = sum_i ((((x / div[i]) % mod[i]) / div2[i]) % mod2[i]) * stride[i]
// (the second stage lets a digit be taken of a sub-index such as the pixel number inside a row index)
struct Digits {
    int n;
    int div[kMaxDigits];
    int mod[kMaxDigits];
    int div2[kMaxDigits];
    int mod2[kMaxDigits];
    long long stride[kMaxDigits];
};

// 32-bit tcgen05 instruction descriptor for kind::f16 / kind::tf32 / kind::i8:
//   [4,6) D format (0 f16, 1 f32, 2 s32)   [7,10) A format   [10,13) B format
//   (f16 kind: 0 f16, 1 bf16; tf32 kind: 2; i8 kind: 0 u8, 1 s8)
//   [15] A is MN-major   [16] B is MN-major   [17,23) N>>3   [24,29) M>>4
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t d_fmt, uint32_t ab_fmt, bool a_mn_major, bool b_mn_major, uint32_t m,
                                   uint32_t n) {
    return (d_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | (uint32_t(a_mn_major) << 15) |
           (uint32_t(b_mn_major) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// How the GEMM row index decomposes into up to four nested tensor coordinates
// (ext[0] fastest) and how a 128-row tile is cut into TMA boxes.
struct RowSpace {
    int nd;
    int ext[4];
    int rows_per_box;    // rows one TMA box brings (divides 128, or the whole row space if smaller)
    int boxes_per_tile;  // boxes issued per 128-row tile
};

struct CoreParams {
    CUtensorMap mapA[4];
    CUtensorMap mapB;
    CUtensorMap mapC;  // EPI_TMA: row-major output as (N, M), box 32 columns x 32 rows, 128-byte swizzle; with tma_t (M, N), 32 rows x 32 columns, no swizzle
    int M, N;         // GEMM-view extents of the output
    int tile_rows;    // output rows per tile (128 unless the row boxes cannot fill a tile)
    int a_tx_bytes;   // bytes the A-operand TMA boxes of one stage deliver (tile_rows * 128, or 16384)
    int num_kb;       // k-blocks per output tile (per split for MTTKRP)
    int total_kb;     // MTTKRP: k-blocks over all splits (the last split may get fewer)
    int tiles_m, tiles_n;
    int group_m;      // row-blocks per rasterisation group (tile order, L2 reuse)
    uint32_t idesc;   // tcgen05 instruction descriptor
    int epi;          // EPI_*
    int b_pre;        // fp32 pair kernel: B comes as the 32 KB slot images a pre-pass wrote (b_images), not through mapB
    int b_halves;     // 128-column half tiles per k-block in b_images (2 x tiles_n)
    const void* b_images;  // [k-block][half tile][raw fp32 tile 16 KB | bf16(b), bf16(lo_b) tile 16 KB]
    int tma_t;        // EPI_TMA on a column-major output: mapC is (M, N) with m innermost, the staged tile is transposed
    void* out;        // fp32 or int32 elements
    long long ldo;    // EPI_ROWMAJOR: row pitch; EPI_COLMAJOR: column pitch (elements)
    Digits dm, dn;    // EPI_SCATTER
    RowSpace rows;    // OP_CONV / OP_CAPSULE
    // convolution-style k-block walk: kb -> (tap, channel block)
    int cblks;        // channel blocks per filter tap
    int KY, KX;       // filter taps (tap = ky + KY*kx)
    int stride;       // capsule spatial stride (1 or 2)
    // capsule weight box walk: channel block -> (cii0, cio0, mk0)
    int CI, CII;
    // MTTKRP
    int splits;       // split-K factor (tiles_n is reused for it)
    int lblks;        // l-blocks per k slice
    const float* fc;  // c(l,r), l fastest, column pitch ldfc
    const float* fb;  // b(k,r), k fastest, column pitch ldfb
    long long ldfc, ldfb;
    int L, Kdim, R;
    // MTTKRP, accumulate-then-scale kernel: work item = (row tile, range of l-blocks, range of k)
    int mt_lb_per, mt_lranges;  // l-blocks per l-range (at most 4), number of l-ranges
    int mt_k_per, mt_kranges;   // k values per k-range (at most 64), number of k-ranges
    int slab_rows;    // fp32 pair kernel, splits > 1: rows between the partial tiles of successive k-ranges
    int use_ab;       // EPI_ROWMAJOR, fp32: out = alpha * acc + beta * out
    float alpha, beta;
    int single_pass;  // fp32 data: 1 = one TF32 MMA per product (raw tiles, no hi/lo split)
    long long wait_cycles;  // limit of every mbarrier wait in SM cycles (kWaitTimeoutCycles unless a test shortens it)
    int skip_stage;   // test hook for the bounded waits: the producer leaves out the copies of this k-block (1-based; 0 = none)
    unsigned* status;
#ifdef T2SP_DEBUG_KNOBS
    long long* trace;  // per-role cycle stamps of CTAs 0 and 1 (timing experiments), or null
#endif
};

#ifdef T2SP_DEBUG_KNOBS
#define T2SP_TRACE(p, role, idx) \
    do { if ((p).trace && blockIdx.x < 2 && (idx) < 1024) (p).trace[((role) + 24 * blockIdx.x) * 1024 + (idx)] = clock64(); } while (0)
// Pair of (SM cycle counter, nanosecond timer) stamps: their differences between two points give the
// SM clock the kernel actually ran at.
#define T2SP_TRACE_CLOCK(p, idx) \
    do { if ((p).trace && blockIdx.x == 0) { (p).trace[23 * 1024 + 2 * (idx)] = clock64(); \
         unsigned long long t2sp_ns_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t2sp_ns_)); \
         (p).trace[23 * 1024 + 2 * (idx) + 1] = static_cast<long long>(t2sp_ns_); } } while (0)
#else
#define T2SP_TRACE(p, role, idx) do { } while (0)
#define T2SP_TRACE_CLOCK(p, idx) do { } while (0)
#endif

}  // namespace t2sp
