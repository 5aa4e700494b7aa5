// Host entry to the contraction kernel family (definitions in umma_launch.cu).
#pragma once
#include <cuda_runtime.h>

#include "umma_params.h"

namespace t2sp {

// Column-tile widths compiled for each arithmetic/operator pair; 0 terminates.
// Returns the tile width to use for an N-extent (narrower tiles when the wide ones would leave
// SMs without work for the given M-extent), or 0 when the pair is not compiled.
int core_pick_bn(int arith, int op, int n_extent, long long m_extent = 1 << 30);

// Launches umma_contract_kernel<arith, op, bn, stages> with `grid` persistent CTAs.
// Returns cudaSuccess or the launch error.
cudaError_t core_launch(int arith, int op, int bn, const CoreParams& p, int grid, cudaStream_t stream);

// Launches the two-CTA (cluster of 2, 256 x 256 tiles) GEMM kernel for the 16-bit and 8-bit
// arithmetics; `grid` must be even. p.tiles_m / p.tiles_n count 256 x 256 tiles and p.idesc
// describes a 256 x 256 MMA. B is MN-major for OP_GEMM and K-major for OP_TTM.
cudaError_t pair_launch(int arith, int op, const CoreParams& p, int grid, cudaStream_t stream);

// Same with 512 x 256 tiles (each CTA owns two 128-row sub-tiles); p.tiles_m counts 512-row tiles.
cudaError_t pair2_launch(int arith, int op, const CoreParams& p, int grid, cudaStream_t stream);

// Launches the two-CTA 3xTF32 kernel (fp32 data, 256 x `un` tiles, un = 256 or 128) for
// OP_GEMM / OP_TTM / OP_CONV / OP_CAPSULE; `grid` must be even, tiles count 256 x un tiles and
// p.idesc describes a 256 x un TF32 MMA.
cudaError_t x3pair_launch(int op, int un, const CoreParams& p, int grid, cudaStream_t stream);
// The 256-column pair tile with the A operand in tensor memory, B pre-packed by b_images_launch (p.b_pre) and the
// cross terms as bf16 MMAs (umma_x3tm.cuh); pair tiles of 256 x un, un = 256 or 128.
cudaError_t x3tm_launch(int op, int un, const CoreParams& p, int grid, cudaStream_t stream);

// Launches the accumulate-then-scale MTTKRP kernel (umma_mttkrp.cuh; R <= 64) with `grid` persistent CTAs over the
// work items that p.tiles_m, p.mt_lranges and p.mt_kranges describe; partial slabs go to p.out.
cudaError_t mttkrp2_launch(const CoreParams& p, int grid, cudaStream_t stream);

// dst[z][c][r] = src[z][r][c] for `batch` rows x cols matrices of 32-bit elements (pitches and batch
// strides in elements; batch <= 65535).
cudaError_t transpose32_launch(const void* src, long long ld_src, void* dst, long long ld_dst, int rows, int cols,
                               cudaStream_t stream, int batch = 1, long long bs_src = 0, long long bs_dst = 0);

// Pre-pass of the fp32 pair kernel with its A operand in tensor memory (umma_x3tm.cuh): the slot images of B,
// [k-block][half tile of 128 or 64 columns][raw fp32 tile | bf16(b), bf16(lo_b) tile], for an operand many row tiles re-read.
struct BImageParams {
    const float* src;
    int mode;        // 0: MN-major B[k][n]; 1: K-major B[n][k]; 2: conv weights (co, kx, ci, ky); 3: capsule weights
                     //    (n = co + CO * my, cii, tap = ky + KY * kx, ci / CII, mk)
    long long ld;    // elements between rows (mode 0: k rows, mode 1: n rows, modes 2 and 3: between channels)
    int K, N;        // contraction extent (mode 2: CI per tap, mode 3: CI * MK per tap) and columns
    int num_kb, halves;
    int cblks, KY;   // modes 2 and 3: k-block = tap * cblks + channel block; mode 2: tap = ky + KY * kx
    int half_cols;   // columns of a half tile: 128 (256-column pair tiles) or 64
    int CI, CII, taps;  // mode 3: capsule channels, inner channel extent, KY * KX
};
cudaError_t b_images_launch(const BImageParams& q, void* dst, cudaStream_t stream);

// Number of SMs of the current device (cached).
int core_sm_count();

// Sums `splits` dense partial slabs [split][col][row] (rows * cols fp32 values each, row fastest) in
// slab order (deterministic) into out[col * ld_out + row]; used by the split-K MTTKRP.
cudaError_t reduce_partials_launch(const float* partials, float* out, int rows, int cols, long long ld_out, int splits,
                                   cudaStream_t stream);

// Split-K epilogue of the fp32 pair kernel: sums the `splits` partial tiles (row-major slabs of
// `slab_rows` rows with pitch `ld_part`, slab after slab) in slab order and writes the M x N result
// through the epilogue `final_p` describes (row-major with optional alpha/beta, column-major, or the
// mixed-radix scatter of the tiled layouts).
cudaError_t splitk_finalize_launch(const float* partials, long long ld_part, int slab_rows, int splits,
                                   const CoreParams& final_p, cudaStream_t stream);

// Copies a tensor of up to 6 dimensions of 32-bit elements between two layouts: element
// (c0..c5) moves from src[sum c_d * sstride[d]] to dst[sum c_d * dstride[d]] (strides in elements).
// Dimension 0 should be the destination's innermost so that the writes coalesce.
struct PermuteDesc {
    int nd;
    int ext[6];
    long long sstride[6];
    long long dstride[6];
};
cudaError_t permute_copy_launch(const void* src, void* dst, const PermuteDesc& d, cudaStream_t stream);

// Folded output of the reference's SYRK design (t2s/tests/performance/syrk/syrk.cpp:38-73): element
// (jjj,iii,jj,ii,j,i) of the 6-D buffer, i < I/2, j <= I, holds alpha * R[r][c] + beta * C[r][c] with
//   (r, c) = (N-1-ti, N-1-tj)        when i >= j   ("bottom" half of the upper triangle, mirrored)
//   (r, c) = (ti, tj - III*II)       otherwise
// ti = iii + III*ii + III*II*i, tj = jjj + III*jj + III*II*j, N = III*II*I. R is the N x N product
// (pitch ldr), C the caller's matrix (pitch ldc); ostride are the element strides of the six dimensions.
struct SyrkFold {
    int III, II, I;
    long long ostride[6];
    long long ldr, ldc;
    float alpha, beta;
};
cudaError_t syrk_fold_launch(const float* R, const float* C, float* O, const SyrkFold& f, cudaStream_t stream);

// Tiled output of the reference's GER design (t2s/tests/performance/ger/ger.cpp:34-62): element
// (kkk,iii,ii,kk,k,i) of the 6-D buffer holds a(tk, ti) + x(ti) * y(tk) with ti = iii + III*ii + III*II*i,
// tk = kkk + KKK*kk + KKK*KK*k. a is addressed as a[ti * lda + tk * sa0]; x, y with their own strides.
struct GerDesc {
    int ext[6];            // KKK, III, II, KK, K, I
    long long ostride[6];  // element strides of the six output dimensions
    long long lda, sa0, sx, sy;
};
cudaError_t ger_launch(const float* a, const float* x, const float* y, float* o, const GerDesc& d, cudaStream_t stream);

}  // namespace t2sp
