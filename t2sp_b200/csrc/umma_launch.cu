// The small kernels around the contraction kernels (split-K sums, layout changes, SYRK fold, GER) and
// their launchers; the contraction kernels themselves are instantiated in launch_*.cu.
#include "launch_util.cuh"
#include "umma_core.cuh"
#include <cuda_bf16.h>

#include "umma_launch.h"

namespace t2sp {

namespace {

// Partial slabs [split][col][row] (dense, `rows` fastest) summed into out[col * ld_out + row]. Four neighbouring
// lanes share an element: lane part p adds slabs p, p + 4, p + 8, ... in that order, then the four sums are added
// as (s0 + s1) + (s2 + s3): a fixed order whatever the launch, so the result is reproducible bit for bit.
__global__ void reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out, int rows, int cols,
                                       long long ld_out, int splits) {
    const long long elems = static_cast<long long>(rows) * cols;
    const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long idx = tid >> 2;
    const int part = static_cast<int>(tid & 3);
    ptx::grid_dep_wait();  // launched while the kernel that writes the partial slabs may still be running
    float acc = 0.f;
    if (idx < elems)
        for (int s = part; s < splits; s += 4) acc += partials[s * elems + idx];
    const float other = __shfl_xor_sync(0xffffffffu, acc, 1);
    const float pair = (part & 1) ? other + acc : acc + other;   // (s0 + s1) resp. (s2 + s3), same operand order in both lanes
    const float far = __shfl_xor_sync(0xffffffffu, pair, 2);
    if (idx < elems && part == 0) out[(idx / rows) * ld_out + idx % rows] = pair + far;
}

// Pre-pass of the fp32 pair kernel with its A operand in tensor memory: the bf16 operands of the cross-term MMAs,
// bf16(x) and bf16(x - trunc_tf32(x)), of an operand that many row tiles re-read.
__device__ __forceinline__ float presplit_lo(float v) { return v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }
__device__ __forceinline__ uint32_t presplit_pack(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// Writes, for every k-block and every half tile of B (128 or 64 columns), the image of the kernel's B slot: the raw
// fp32 tile as TMA would have laid it out followed by the bf16 tile [bf16(b) | bf16(lo_b)] of the same size. One
// thread per 16-byte piece of the raw tile (four consecutive N values of an MN-major B, four consecutive K values of
// a K-major one); elements outside B are zero.
__global__ void b_images_kernel(const BImageParams q, uint8_t* __restrict__ dst) {
    ptx::grid_dep_launch();  // the contraction kernel may set itself up meanwhile; it waits for this grid before it reads an image
    const int H = q.half_cols, raw_bytes = H * 128, pieces = H * 8;
    const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long blobs = static_cast<long long>(q.num_kb) * q.halves;
    if (idx >= blobs * pieces) return;
    const int pi = static_cast<int>(idx % pieces);
    const long long blob = idx / pieces;
    const int kb = static_cast<int>(blob / q.halves), half = static_cast<int>(blob % q.halves);
    uint8_t* img = dst + blob * (2 * raw_bytes);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    int off_raw, off_hb, off_lb;
    if (q.mode == 1) {
        // K-major: row r (an n) holds 32 K values in 128 bytes, 16-byte chunk c stored at c ^ (r & 7); the bf16 tile
        // keeps the row pitch, bf16(b) in the first 64 bytes of the row, bf16(lo_b) in the second, same swizzle
        const int r = pi >> 3, c = pi & 7, x = r & 7;
        const long long n = static_cast<long long>(half) * H + r;
        const int k0 = kb * 32 + 4 * c;
        if (n < q.N)
            for (int j = 0; j < 4; ++j)
                if (k0 + j < q.K) v[j] = q.src[n * q.ld + k0 + j];
        off_raw = r * 128 + ((c ^ x) << 4);
        off_hb = raw_bytes + r * 128 + (((c >> 1) ^ x) << 4) + (c & 1) * 8;
        off_lb = raw_bytes + r * 128 + (((4 + (c >> 1)) ^ x) << 4) + (c & 1) * 8;
    } else {
        // MN-major: boxes of 32 K rows x 32 N values (128-byte rows) with 32-byte atoms swizzled (atom a of row k
        // stored at a ^ (k & 3)); the bf16 tiles are boxes of 32 K rows x 64 N values, 16-byte chunk c stored at
        // c ^ (k & 7), the boxes of bf16(b) first, then those of bf16(lo_b)
        const int groups = H / 4;
        const int k = pi / groups, g = pi % groups;
        const int n = half * H + 4 * g;
        const float* s = nullptr;
        if (q.mode == 0) {
            const int kg = kb * 32 + k;
            if (kg < q.K) s = q.src + static_cast<long long>(kg) * q.ld;
        } else if (q.mode == 2) {
            const int tap = kb / q.cblks, cb = kb % q.cblks, ky = tap % q.KY, kx = tap / q.KY, ci = cb * 32 + k;
            if (ci < q.K) s = q.src + static_cast<long long>(q.N) * kx + (static_cast<long long>(ci) + static_cast<long long>(ky) * q.K) * q.ld;
        } else {
            const int tap = kb / q.cblks, c = (kb % q.cblks) * 32 + k;
            if (c < q.K) {
                const int mk = c / q.CI, ci = c % q.CI, cii = ci % q.CII, cio = ci / q.CII;
                s = q.src + (static_cast<long long>(cii) + static_cast<long long>(tap) * q.CII +
                             static_cast<long long>(cio) * q.CII * q.taps + static_cast<long long>(mk) * q.CI * q.taps) * q.ld;
            }
        }
        if (s)
            for (int j = 0; j < 4; ++j)
                if (n + j < q.N) v[j] = s[n + j];
        const int jb = g >> 3, a = (g & 7) >> 1, sub = g & 1;
        off_raw = jb * 4096 + k * 128 + ((((a ^ (k & 3)) << 1) | sub) << 4);
        const int c8 = (jb & 1) * 4 + a;
        off_hb = raw_bytes + (jb >> 1) * 4096 + k * 128 + ((c8 ^ (k & 7)) << 4) + sub * 8;
        off_lb = off_hb + raw_bytes / 2;
    }
    *reinterpret_cast<float4*>(img + off_raw) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<uint2*>(img + off_hb) = make_uint2(presplit_pack(v[0], v[1]), presplit_pack(v[2], v[3]));
    *reinterpret_cast<uint2*>(img + off_lb) = make_uint2(presplit_pack(presplit_lo(v[0]), presplit_lo(v[1])),
                                                         presplit_pack(presplit_lo(v[2]), presplit_lo(v[3])));
}

// One thread per row and four consecutive columns; the sum over the slabs runs in slab order.
__global__ void splitk_finalize_kernel(const float* __restrict__ part, long long ld_part, long long slab_elems, int splits,
                                       const __grid_constant__ CoreParams f) {
    const int quads = (f.N + 3) >> 2;
    const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= static_cast<long long>(f.M) * quads) return;
    const int m = static_cast<int>(idx / quads), n = static_cast<int>(idx % quads) * 4;
    ptx::grid_dep_wait();  // launched while the kernel that writes the partial tiles may still be running
    const float* src = part + static_cast<long long>(m) * ld_part + n;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + s * slab_elems);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const float v[4] = {acc.x, acc.y, acc.z, acc.w};
    float* out = static_cast<float*>(f.out);
    if (f.epi == EPI_SCATTER) {
        const long long offm = digits_offset(f.dm, m);
        for (int j = 0; j < 4; ++j)
            if (n + j < f.N) out[offm + digits_offset(f.dn, n + j)] = v[j];
    } else if (f.epi == EPI_COLMAJOR) {
        for (int j = 0; j < 4; ++j)
            if (n + j < f.N) out[static_cast<long long>(n + j) * f.ldo + m] = v[j];
    } else {
        float* dst = out + static_cast<long long>(m) * f.ldo + n;
        for (int j = 0; j < 4; ++j) {
            if (n + j >= f.N) break;
            if (f.use_ab) {
                const float a = f.alpha * v[j];
                dst[j] = f.beta != 0.f ? a + f.beta * dst[j] : a;
            } else {
                dst[j] = v[j];
            }
        }
    }
}

__global__ void permute_copy_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                    const __grid_constant__ PermuteDesc d, long long total) {
    long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    long long so = 0, dof = 0;
#pragma unroll
    for (int i = 0; i < 6; ++i) {
        if (i < d.nd) {
            const int c = static_cast<int>(idx % d.ext[i]);
            idx /= d.ext[i];
            so += c * d.sstride[i];
            dof += c * d.dstride[i];
        }
    }
    dst[dof] = src[so];
}

__global__ void syrk_fold_kernel(const float* __restrict__ R, const float* __restrict__ C, float* __restrict__ O,
                                 const __grid_constant__ SyrkFold f) {
    const int t = f.III * f.II;  // rows (and columns) of one (i, j) block
    const long long total = static_cast<long long>(t) * t * (f.I + 1) * (f.I / 2);
    long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const int jjj = idx % f.III; idx /= f.III;
    const int iii = idx % f.III; idx /= f.III;
    const int jj = idx % f.II; idx /= f.II;
    const int ii = idx % f.II; idx /= f.II;
    const int j = idx % (f.I + 1);
    const int i = static_cast<int>(idx / (f.I + 1));
    const int n = t * f.I;
    const int ti = iii + f.III * ii + t * i, tj = jjj + f.III * jj + t * j;
    int r, c;
    if (i >= j) { r = n - 1 - ti; c = n - 1 - tj; }
    else { r = ti; c = tj - t; }
    float v = f.alpha * R[r * f.ldr + c];
    if (f.beta != 0.f) v += f.beta * C[r * f.ldc + c];
    O[jjj * f.ostride[0] + iii * f.ostride[1] + jj * f.ostride[2] + ii * f.ostride[3] + j * f.ostride[4] +
      i * f.ostride[5]] = v;
}

// One thread per VEC consecutive kkk of the tiled GER output, in output order, so that a dense output
// is written in whole lines; the matching run of a is read once (VEC = 4: 16-byte loads and stores
// with streaming hints, as neither a nor the output is touched again).
template <int VEC>
__global__ void ger_tiled_kernel(const float* __restrict__ a, const float* __restrict__ x, const float* __restrict__ y,
                                 float* __restrict__ o, const __grid_constant__ GerDesc d, long long total) {
    long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const int kv = d.ext[0] / VEC;
    const int kkk = static_cast<int>(idx % kv) * VEC; idx /= kv;
    const int iii = idx % d.ext[1]; idx /= d.ext[1];
    const int ii = idx % d.ext[2]; idx /= d.ext[2];
    const int kk = idx % d.ext[3]; idx /= d.ext[3];
    const int k = idx % d.ext[4];
    const int i = static_cast<int>(idx / d.ext[4]);
    const long long ti = iii + d.ext[1] * (ii + static_cast<long long>(d.ext[2]) * i);
    const long long tk = kkk + d.ext[0] * (kk + static_cast<long long>(d.ext[3]) * k);
    const long long off = kkk * d.ostride[0] + iii * d.ostride[1] + ii * d.ostride[2] + kk * d.ostride[3] +
                          k * d.ostride[4] + i * d.ostride[5];
    const float xv = __ldg(x + ti * d.sx);
    if constexpr (VEC == 4) {
        const float4 av = __ldcs(reinterpret_cast<const float4*>(a + ti * d.lda + tk));
        const float4 yv = __ldg(reinterpret_cast<const float4*>(y + tk));
        // a separately rounded product and sum, as the specification's two operations (no fused multiply-add)
        __stcs(reinterpret_cast<float4*>(o + off),
               make_float4(__fadd_rn(av.x, __fmul_rn(xv, yv.x)), __fadd_rn(av.y, __fmul_rn(xv, yv.y)),
                           __fadd_rn(av.z, __fmul_rn(xv, yv.z)), __fadd_rn(av.w, __fmul_rn(xv, yv.w))));
    } else {
        o[off] = __fadd_rn(a[ti * d.lda + tk * d.sa0], __fmul_rn(xv, __ldg(y + tk * d.sy)));
    }
}

// The dense, 16-byte-aligned case of the tiled GER: one CTA per (kk group, k, i). Q consecutive kk are
// taken together so that the threads of a row read Q * KKK consecutive floats of a (whole 128-byte
// lines for Q * KKK >= 32) and, with neighbouring rows adjacent in the output, write runs of whole
// lines too. A thread keeps its column position for all its rows, so the only index arithmetic in the
// loop is a row increment; U rows are loaded before any is stored.
template <int U>
__global__ void __launch_bounds__(256)
ger_rows_kernel(const float* __restrict__ a, const float* __restrict__ x, const float* __restrict__ y,
                float* __restrict__ o, const __grid_constant__ GerDesc d, int q, int kv) {
    unsigned b = blockIdx.x;
    const unsigned nkh = d.ext[3] / q;
    const int kkh = b % nkh; b /= nkh;
    const int k = b % static_cast<unsigned>(d.ext[4]);
    const int i = b / static_cast<unsigned>(d.ext[4]);
    const int lanes = kv * q;  // threads per row
    const int c = threadIdx.x % lanes;
    const int kk = kkh * q + c / kv, kkk = (c % kv) * 4;
    const long long tk = kkk + d.ext[0] * (kk + static_cast<long long>(d.ext[3]) * k);
    const int rows = d.ext[1] * d.ext[2];
    const long long ti0 = static_cast<long long>(rows) * i;
    const float4 yv = __ldg(reinterpret_cast<const float4*>(y + tk));
    const float* ap = a + ti0 * d.lda + tk;
    const float* xp = x + ti0 * d.sx;
    float* op = o + kkk + kk * d.ostride[3] + k * d.ostride[4] + i * d.ostride[5];
    const int rstep = 256 / lanes;
    for (int r0 = threadIdx.x / lanes; r0 < rows; r0 += rstep * U) {
        float4 av[U];
        float xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = r0 + u * rstep;
            if (r < rows) {
                av[u] = __ldcs(reinterpret_cast<const float4*>(ap + r * d.lda));
                xv[u] = __ldg(xp + r * d.sx);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = r0 + u * rstep;
            if (r < rows)
                __stcs(reinterpret_cast<float4*>(op + r * d.ostride[1]),
                       make_float4(__fadd_rn(av[u].x, __fmul_rn(xv[u], yv.x)), __fadd_rn(av[u].y, __fmul_rn(xv[u], yv.y)),
                                   __fadd_rn(av[u].z, __fmul_rn(xv[u], yv.z)), __fadd_rn(av[u].w, __fmul_rn(xv[u], yv.w))));
        }
    }
}

}  // namespace

int core_sm_count() {
    static std::atomic<int> cached[kMaxDev];
    int dev = 0;
    cudaGetDevice(&dev);
    const bool in_table = dev >= 0 && dev < kMaxDev;
    int n = in_table ? cached[dev].load(std::memory_order_relaxed) : 0;
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        if (in_table) cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int core_pick_bn(int arith, int op, int n_extent, long long m_extent) {
    const long long tiles_m = (m_extent + kBlockM - 1) / kBlockM;
    auto fills = [&](int bn) { return tiles_m * ((n_extent + bn - 1) / bn) >= core_sm_count(); };
    switch (arith) {
        case AR_F16:
        case AR_I8:
            if (op == OP_GEMM || op == OP_TTM) return (n_extent > 128 && fills(256)) ? 256 : 128;
            return 0;
        case AR_TF32X3:
            if (op == OP_MTTKRP) return n_extent <= 64 ? 64 : (n_extent <= 128 ? 128 : 0);
            if (op == OP_GEMM || op == OP_TTM || op == OP_CONV || op == OP_CAPSULE)
                return (n_extent > 64 && fills(128)) ? 128 : 64;
            return 0;
    }
    return 0;
}

// dst[z][c][r] = src[z][r][c] for `batch` matrices of rows x cols 32-bit elements (pitches and batch
// strides in elements), through a 32 x 32 shared-memory tile so that reads and writes both coalesce.
__global__ void transpose32_kernel(const uint32_t* __restrict__ src, long long ld_src, long long bs_src,
                                   uint32_t* __restrict__ dst, long long ld_dst, long long bs_dst, int rows, int cols) {
    __shared__ uint32_t tile[32][33];
    src += blockIdx.z * bs_src;
    dst += blockIdx.z * bs_dst;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = src[r * ld_src + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, r = r0 + threadIdx.x;  // dst[c][r] = src[r][c]
        if (r < rows && c < cols) dst[c * ld_dst + r] = tile[threadIdx.x][j];
    }
}

cudaError_t transpose32_launch(const void* src, long long ld_src, void* dst, long long ld_dst, int rows, int cols,
                               cudaStream_t stream, int batch, long long bs_src, long long bs_dst) {
    if (rows <= 0 || cols <= 0 || batch <= 0) return cudaSuccess;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
    transpose32_kernel<<<grid, block, 0, stream>>>(static_cast<const uint32_t*>(src), ld_src, bs_src,
                                                   static_cast<uint32_t*>(dst), ld_dst, bs_dst, rows, cols);
    return cudaGetLastError();
}

cudaError_t b_images_launch(const BImageParams& q, void* dst, cudaStream_t stream) {
    const long long work = static_cast<long long>(q.num_kb) * q.halves * q.half_cols * 8;
    if (work <= 0) return cudaSuccess;
    b_images_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(q, static_cast<uint8_t*>(dst));
    return cudaGetLastError();
}

cudaError_t splitk_finalize_launch(const float* partials, long long ld_part, int slab_rows, int splits,
                                   const CoreParams& final_p, cudaStream_t stream) {
    const long long work = static_cast<long long>(final_p.M) * ((final_p.N + 3) / 4);
    if (work <= 0) return cudaSuccess;
    const int threads = 256;
    // programmatic stream serialization: the launch is set up and its CTAs scheduled as the contraction
    // kernel's CTAs retire; the kernel itself waits for that grid before it reads a partial tile
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((work + threads - 1) / threads));
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitk_finalize_kernel, partials, ld_part, static_cast<long long>(slab_rows) * ld_part,
                              splits, final_p);
}

cudaError_t permute_copy_launch(const void* src, void* dst, const PermuteDesc& d, cudaStream_t stream) {
    long long total = 1;
    for (int i = 0; i < d.nd; ++i) total *= d.ext[i];
    if (total <= 0) return cudaSuccess;
    const int threads = 256;
    permute_copy_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(
        static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), d, total);
    return cudaGetLastError();
}

cudaError_t syrk_fold_launch(const float* R, const float* C, float* O, const SyrkFold& f, cudaStream_t stream) {
    const long long t = static_cast<long long>(f.III) * f.II;
    const long long total = t * t * (f.I + 1) * (f.I / 2);
    if (total <= 0) return cudaSuccess;
    const int threads = 256;
    syrk_fold_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(R, C, O, f);
    return cudaGetLastError();
}

cudaError_t ger_launch(const float* a, const float* x, const float* y, float* o, const GerDesc& d, cudaStream_t stream) {
    long long total = 1;
    for (int i = 0; i < 6; ++i) total *= d.ext[i];
    if (total <= 0) return cudaSuccess;
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    bool vec = d.ext[0] % 4 == 0 && d.ostride[0] == 1 && d.sa0 == 1 && d.sy == 1 && d.lda % 4 == 0 && aligned16(a) &&
               aligned16(y) && aligned16(o);
    for (int i = 1; i < 6; ++i) vec = vec && d.ostride[i] % 4 == 0;
    const int threads = 256;
    if (vec && d.ostride[2] == d.ext[1] * d.ostride[1]) {
        // rows (iii, ii) of one (kk, k, i) are evenly spaced in the output: the row-tiled kernel applies
        const int kv = d.ext[0] / 4;
        int q = d.ext[3] % 4 == 0 ? 4 : (d.ext[3] % 2 == 0 ? 2 : 1);
        while (q > 1 && kv * q > 64) q /= 2;
        const long long blocks = static_cast<long long>(d.ext[3] / q) * d.ext[4] * d.ext[5];
        if (kv * q <= 256 && 256 % (kv * q) == 0 && blocks < (1ll << 31)) {
            ger_rows_kernel<4><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(a, x, y, o, d, q, kv);
            return cudaGetLastError();
        }
    }
    if (vec) {
        total /= 4;
        ger_tiled_kernel<4><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(a, x, y, o, d, total);
    } else {
        ger_tiled_kernel<1><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(a, x, y, o, d, total);
    }
    return cudaGetLastError();
}

cudaError_t reduce_partials_launch(const float* partials, float* out, int rows, int cols, long long ld_out, int splits,
                                   cudaStream_t stream) {
    const int threads = 256;
    const long long elems = static_cast<long long>(rows) * cols;
    if (elems <= 0) return cudaSuccess;
    // programmatic stream serialization: the blocks are scheduled as the CTAs of the kernel before it retire; the
    // kernel itself waits for that grid before it reads a partial slab
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((elems * 4 + threads - 1) / threads));
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, reduce_partials_kernel, partials, out, rows, cols, ld_out, splits);
}

}  // namespace t2sp
