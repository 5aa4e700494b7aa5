// fp32 contraction on CTA pairs with the A operand in tensor memory and the cross terms at bf16 rate.
//
// x = hi + lo with hi = trunc_tf32(x) (what the tensor core reads from a raw fp32 word) and lo = x - hi (exact).
// a * b = hi_a * hi_b + lo_a * b + a * lo_b (+ lo_a * lo_b, dropped: 2^-22). The first product runs as TF32 MMAs on
// the raw words; the two cross products are 2^-11 of the result and run as bf16 MMAs on bf16(lo_a) x bf16(b) and
// bf16(a) x bf16(lo_b): each bf16 rounding is 2^-9 of a term that is 2^-11 of the product, so a product is off by
// at most about 2^-18 |a| |b| (3.8e-6) where plain fp32 arithmetic with K terms is off by K 2^-24. Per 32-deep
// k-block that is 4 + 4 MMAs of 256 x 256 (1024 tensor cycles) instead of the 12 TF32 MMAs (1536) of
// umma_x3pair.cuh.
//
// The pair kernel with all operands in shared memory is bound by shared-memory bandwidth as much as by the tensor
// pipe (per k-block and SM: 96 KB of MMA operand reads, 64 KB of split traffic, 32 KB of TMA writes). Here the split
// warps write the A tile, already split, into tensor memory (tcgen05.st), so the MMAs read only B from shared memory:
// the raw fp32 B tile for the TF32 pass and one 16 KB tile holding bf16(b) and bf16(lo_b) for the two bf16 passes.
//
// Per CTA: 16 warps as in umma_x3pair.cuh.
//   warp 0      TMA producer (own 128 A rows, own 128 of the 256 B columns) into a ring of raw fp32 stages
//   warp 1      MMA issuer (leader CTA only), TMEM owner
//   warps 2-3, 12-15  split warps. A warp may touch only the TMEM lanes of its quarter (warp % 4), so the A tile goes
//               by quarters: warps 12 and 13 take the rows of quarters 0 and 1, warps 2 / 14 and 3 / 15 share
//               quarters 2 and 3 by halves of the k-block; the B tile's 1024 16-byte pieces are dealt out so that
//               all six warps carry about the same number of pieces.
//               With BPRE the bf16 tiles of B come from a pre-pass over the whole operand (worth it when many row tiles
//               re-read a small B: weights, the factor of a TTM) and the split warps convert A only.
//   warps 4-11  epilogue as in umma_x3pair.cuh: every 8 k-blocks the accumulator is added into fp32 registers
//               (round to nearest) and handed back
// TMEM per CTA (512 columns): [accumulator 256 | 4 A slots of 64: hi 32, bf16(a) 16, bf16(lo) 16].
#pragma once
#include <cuda_bf16.h>

#include <type_traits>

#include "umma_core.cuh"
#include "umma_x3pair.cuh"

namespace t2sp {

template <int OP, int STAGES>
struct X3TmCfg {
    static constexpr bool kBMnMajor = (OP == OP_GEMM || OP == OP_CONV || OP == OP_CAPSULE);
    static constexpr int UN = 256;
    static constexpr int kHalfN = UN / 2;
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = kHalfN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSlots = 4;              // A slots in tensor memory = bf16 B tiles in shared memory
    static constexpr int kB16Bytes = kBBytes;     // bf16(b) and bf16(lo_b) of one k-block
    static constexpr int kBoxBytesMn = 32 * 128;  // MN-major fp32 box: 32 k-rows x 32 columns
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;
    static constexpr uint32_t kBSwizzle = kBMnMajor ? 1u : 2u;
    static constexpr uint32_t kBSbo = kBMnMajor ? 512u : 1024u;
    static constexpr int kThreads = 16 * 32;
    static constexpr int kTmemCols = 512;
    static constexpr int kASlotCol0 = UN;
    static constexpr int kChunkKb = 8;
    static constexpr int kColsPerWarp = UN / 2;
    static constexpr int kCStage = 8 * 4096;
    static constexpr int kNumBars = 2 * STAGES + 2 * kSlots + 2;
    static constexpr int kTailBytes = kNumBars * 8 + 16;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kSlots * kB16Bytes + kCStage + kTailBytes + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t x3_pack_bf16(float lo_elem, float hi_elem) {
#ifdef T2SP_X3_INT_PACK
    // round to nearest (ties up) with integer adds and one byte permute: full-rate instructions instead of a conversion
    return __byte_perm(__float_as_uint(lo_elem) + 0x8000u, __float_as_uint(hi_elem) + 0x8000u, 0x7632);
#else
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);  // .x (low half) = first argument
    return *reinterpret_cast<const uint32_t*>(&v);
#endif
}
__device__ __forceinline__ float x3_tf32_lo(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

template <int OP, int STAGES, bool BPRE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(X3TmCfg<OP, STAGES>::kThreads, 1)
umma_x3tm_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = X3TmCfg<OP, STAGES>;
    constexpr int UN = Cfg::UN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* b16_ring = smem + STAGES * Cfg::kStageBytes;
    uint8_t* cstage = b16_ring + Cfg::kSlots * Cfg::kB16Bytes;
    uint8_t* tail = cstage + Cfg::kCStage;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // own: this CTA's TMA data landed
    uint64_t* empty_bar = full_bar + STAGES;                 // own: MMAs that read the stage's B tile retired
    uint64_t* ready_bar = empty_bar + STAGES;                // leader's: both CTAs' A slot and bf16 B tile written (12)
    uint64_t* free_bar = ready_bar + Cfg::kSlots;            // own: MMAs that read the slot retired
    uint64_t* cfull_bar = free_bar + Cfg::kSlots;            // own: a chunk of the accumulator is complete
    uint64_t* cempty_bar = cfull_bar + 1;                    // leader's: the chunk was drained by both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cempty_bar + 1);
    uint32_t* abort_slot = tmem_slot + 1;
    long long* ntable = reinterpret_cast<long long*>(cstage);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    // Work items as in umma_x3pair.cuh: item t is range t % splits of tile t / splits.
    const int splits = p.splits > 1 ? p.splits : 1;
    const int num_tiles = p.tiles_m * p.tiles_n * splits;
    auto item_kb_begin = [&](int t) { return (t % splits) * p.num_kb; };
    auto item_kb_count = [&](int t) { return min(p.num_kb, p.total_kb - (t % splits) * p.num_kb); };
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < Cfg::kSlots; ++a) {
            ptx::mbar_init(&ready_bar[a], 12);  // 6 split warps in each CTA
            ptx::mbar_init(&free_bar[a], 1);
        }
        ptx::mbar_init(cfull_bar, 1);
        ptx::mbar_init(cempty_bar, 16);         // 8 epilogue warps in each CTA
        *abort_slot = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before_sync();
    ptx::grid_dep_launch();  // the split-K summing kernel may be scheduled while this grid runs
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) T2SP_TRACE(p, 10, 0);

    // Split role. `q`: TMEM lane quarter of the warp; `a_half0`, `a_halves`: which halves of the k-block's 32 columns
    // of the quarter's A rows this warp converts; `b0`, NB: its B pieces are b0 + lane + 32 i, i < NB.
    auto split_role = [&](const int q, const int a_half0, const int a_halves, const int b0, auto nb_const) {
        constexpr int NB = decltype(nb_const)::value;
        int it = 0;
        bool ok = true;
        const int row = q * 32 + lane;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            const int nkb = item_kb_count(t);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const int ls = it % Cfg::kSlots;
                const uint8_t* raw = smem + s * Cfg::kStageBytes;
                uint8_t* b16 = b16_ring + ls * Cfg::kB16Bytes;
                if (!bounded_wait_warp(&free_bar[ls], ((it / Cfg::kSlots) & 1) ^ 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
#ifdef T2SP_TRACE_HEAVY
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 8, it);
#endif
                if (!bounded_wait_warp(&full_bar[s], (it / STAGES) & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 1, it);
#ifdef T2SP_TRACE_HEAVY
                if (warp == 2 && lane == 0) T2SP_TRACE(p, 11, it);
#endif
                // A: this thread's tile row (16-byte chunk c sits at c ^ (row & 7)), half a k-block at a time:
                // raw words for the TF32 pass, bf16(a) and bf16(lo_a) (two k values per 32-bit column) for the others
                const uint8_t* rp = raw + row * 128;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::kASlotCol0 + ls * 64;
                for (int h = a_half0; h < a_half0 + a_halves; ++h) {
                    uint32_t vh[16], vb[8], vl[8];
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const float4 v = *reinterpret_cast<const float4*>(rp + (((4 * h + cc) ^ (row & 7)) << 4));
                        vh[4 * cc + 0] = __float_as_uint(v.x); vh[4 * cc + 1] = __float_as_uint(v.y);
                        vh[4 * cc + 2] = __float_as_uint(v.z); vh[4 * cc + 3] = __float_as_uint(v.w);
                        if (!p.single_pass) {
                            vb[2 * cc + 0] = x3_pack_bf16(v.x, v.y); vb[2 * cc + 1] = x3_pack_bf16(v.z, v.w);
                            vl[2 * cc + 0] = x3_pack_bf16(x3_tf32_lo(v.x), x3_tf32_lo(v.y));
                            vl[2 * cc + 1] = x3_pack_bf16(x3_tf32_lo(v.z), x3_tf32_lo(v.w));
                        }
                    }
                    ptx::tmem_st_32x16(taddr + 16 * h, vh);
                    if (!p.single_pass) {
                        ptx::tmem_st_32x8(taddr + 32 + 8 * h, vb);
                        ptx::tmem_st_32x8(taddr + 48 + 8 * h, vl);
                    }
                }
#ifdef T2SP_TRACE_HEAVY
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 7, it);
#endif
#ifdef T2SP_TRACE_HEAVY
                if (warp == 2 && lane == 0) T2SP_TRACE(p, 12, it);
#endif
                // B: 16-byte pieces of the raw tile (four consecutive K or N values) become two 8-byte pieces
                if (!BPRE && !p.single_pass) {
                    const uint8_t* braw = raw + Cfg::kABytes;
                    // in batches of up to four pieces: loads first, then conversions and stores, so that a batch's loads overlap
                    // (all of a warp's pieces at once spilled registers in the warps with the small budget)
#pragma unroll
                    for (int i0 = 0; i0 < NB; i0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i0 + i < NB) v[i] = *reinterpret_cast<const float4*>(braw + ((b0 + lane + 32 * (i0 + i)) << 4));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (i0 + i >= NB) break;
                        const int ci = b0 + lane + 32 * (i0 + i);
                        const uint2 hb = make_uint2(x3_pack_bf16(v[i].x, v[i].y), x3_pack_bf16(v[i].z, v[i].w));
                        const uint2 lb = make_uint2(x3_pack_bf16(x3_tf32_lo(v[i].x), x3_tf32_lo(v[i].y)),
                                                    x3_pack_bf16(x3_tf32_lo(v[i].z), x3_tf32_lo(v[i].w)));
                        if constexpr (!Cfg::kBMnMajor) {
                            // K-major tile: row r (an n) holds 32 K values in 128 bytes, chunk c stored at c ^ (r & 7). The
                            // bf16 tile keeps the row pitch: bf16(b) of the row in its first 64 bytes, bf16(lo_b) in its
                            // second 64 bytes, same swizzle.
                            const int r = ci >> 3, x = r & 7, c = (ci & 7) ^ x;
                            uint8_t* drow = b16 + r * 128 + (c & 1) * 8;
                            *reinterpret_cast<uint2*>(drow + (((c >> 1) ^ x) << 4)) = hb;
                            *reinterpret_cast<uint2*>(drow + (((4 + (c >> 1)) ^ x) << 4)) = lb;
                        } else {
                            // MN-major fp32 tile: boxes of 32 K rows x 32 N values (128-byte rows) with 32-byte atoms
                            // swizzled: atom a of row k stored at a ^ (k & 3). The bf16 tiles are MN-major in the layout
                            // 16-bit operands use: boxes of 32 K rows x 64 N values, 16-byte chunk c stored at c ^ (k & 7);
                            // the boxes of bf16(b) first, then those of bf16(lo_b).
                            const int jb = ci >> 8, k = (ci >> 3) & 31, cs = ci & 7;
                            const int a = (cs >> 1) ^ (k & 3), c8 = (jb & 1) * 4 + a;
                            uint8_t* d = b16 + (jb >> 1) * 4096 + k * 128 + ((c8 ^ (k & 7)) << 4) + (cs & 1) * 8;
                            *reinterpret_cast<uint2*>(d) = hb;
                            *reinterpret_cast<uint2*>(d + Cfg::kB16Bytes / 2) = lb;
                        }
                    }
                    asm volatile("" ::: "memory");
                    }
#ifdef T2SP_TRACE_HEAVY
                    if (warp == 2 && lane == 0) T2SP_TRACE(p, 15, it);
#endif
                    ptx::fence_proxy_async_smem();
                }
#ifdef T2SP_TRACE_HEAVY
                if (warp == 2 && lane == 0) T2SP_TRACE(p, 14, it);
#endif
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) ptx::mbar_arrive(&ready_bar[ls]);
                    else ptx::mbar_arrive_peer(&ready_bar[ls], 0);
                }
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 2, it);
#ifdef T2SP_TRACE_HEAVY
                if (warp == 2 && lane == 0) T2SP_TRACE(p, 13, it);
#endif
#ifdef T2SP_TRACE_HEAVY
                if (lane == 0) T2SP_TRACE(p, 16 + (warp < 4 ? warp - 2 : warp - 10), it);
#endif
            }
        }
    };

    if (warp < 4) {
        set_max_regs_dec<72>();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            if constexpr (OP == OP_CAPSULE) {
                for (int i = 0; i < 4; ++i) ptx::prefetch_tensormap(&p.mapA[i]);
            } else {
                ptx::prefetch_tensormap(&p.mapA[0]);
            }
            ptx::prefetch_tensormap(&p.mapB);
            if (BPRE) {
                ptx::prefetch_tensormap(&p.mapB2);
                if (Cfg::kBMnMajor) ptx::prefetch_tensormap(&p.mapB3);
            }
            int it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mb, nb;
                tile_coords(t / splits, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                const int m0 = mb * 256 + static_cast<int>(rank) * kBlockM;
                const int n0 = nb * UN + static_cast<int>(rank) * Cfg::kHalfN;
                const int kb_begin = item_kb_begin(t), nkb = item_kb_count(t);
                // Tiles walk their k-blocks from different starting points (a sum over k either way), so that CTAs
                // running in step do not all ask for the same 128-byte column of every operand row at the same time.
                const int rot = t % nkb;
                for (int step = 0; step < nkb; ++step, ++it) {
                    const int kb = kb_begin + (step + rot) % nkb;
                    const int s = it % STAGES;
                    if (!bounded_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    uint8_t* sa = smem + s * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    const int ls = it % Cfg::kSlots;
                    uint8_t* b16 = b16_ring + ls * Cfg::kB16Bytes;
                    // BPRE: bf16(b) and bf16(lo_b) were computed once per call by a pre-pass and come by TMA, straight
                    // into the slot the MMAs read them from (free once the MMAs of k-block it - kSlots retired)
                    if (BPRE && !p.single_pass &&
                        !bounded_wait(&free_bar[ls], ((it / Cfg::kSlots) & 1) ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    T2SP_TRACE(p, 0, it);
                    ptx::mbar_expect_tx(&full_bar[s], Cfg::kStageBytes + ((BPRE && !p.single_pass) ? Cfg::kB16Bytes : 0));
                    if (BPRE && !p.single_pass) {
                        if constexpr (OP == OP_TTM) {
                            // rows of [bf16(b) 32 k | bf16(lo_b) 32 k] per k-block
                            ptx::tma_load_2d(b16, &p.mapB2, &full_bar[s], kb * 64, n0);
                        } else if constexpr (OP == OP_GEMM) {
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                ptx::tma_load_2d(b16 + j * 4096, &p.mapB2, &full_bar[s], n0 + j * 64, kb * 32);
                                ptx::tma_load_2d(b16 + Cfg::kB16Bytes / 2 + j * 4096, &p.mapB3, &full_bar[s], n0 + j * 64, kb * 32);
                            }
                        } else if constexpr (OP == OP_CONV) {
                            const int tap = kb / p.cblks, cb = kb % p.cblks;
                            const int ky = tap % p.KY, kx = tap / p.KY;
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                ptx::tma_load_4d(b16 + j * 4096, &p.mapB2, &full_bar[s], n0 + j * 64, kx, cb * 32, ky);
                                ptx::tma_load_4d(b16 + Cfg::kB16Bytes / 2 + j * 4096, &p.mapB3, &full_bar[s], n0 + j * 64, kx, cb * 32, ky);
                            }
                        }
                    }
                    if constexpr (OP == OP_GEMM || OP == OP_TTM) {
                        ptx::tma_load_2d(sa, &p.mapA[0], &full_bar[s], kb * 32, m0);
                        if constexpr (OP == OP_TTM) {
                            ptx::tma_load_2d(sb, &p.mapB, &full_bar[s], kb * 32, n0);
                        } else {
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_2d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s], n0 + j * 32, kb * 32);
                        }
                    } else {
                        const int tap = kb / p.cblks, cb = kb % p.cblks;
                        const int ky = tap % p.KY, kx = tap / p.KY;
                        const int c0 = cb * 32;
                        for (int j = 0; j < p.rows.boxes_per_tile; ++j) {
                            int r = m0 + j * p.rows.rows_per_box;
                            int c[4] = {0, 0, 0, 0};
#pragma unroll
                            for (int d = 0; d < 4; ++d) {
                                if (d < p.rows.nd - 1) { c[d] = r % p.rows.ext[d]; r /= p.rows.ext[d]; }
                                else if (d == p.rows.nd - 1) { c[d] = r; }
                            }
                            uint8_t* dst = sa + j * p.rows.rows_per_box * 128;
                            if constexpr (OP == OP_CONV) {
                                ptx::tma_load_4d(dst, &p.mapA[0], &full_bar[s], c0, c[0], c[1] + ky, c[2] + kx);
                            } else {
                                const int sy = ky % p.stride, sx = kx % p.stride;
                                ptx::tma_load_5d(dst, &p.mapA[sy + 2 * sx], &full_bar[s], c0, c[0], c[1] + ky / p.stride,
                                                 c[2] + kx / p.stride, c[3]);
                            }
                        }
                        if constexpr (OP == OP_CONV) {
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_4d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s], n0 + j * 32, kx, c0, ky);
                        } else {
                            const int mk0 = c0 / p.CI, ci0 = c0 % p.CI;
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_5d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s], n0 + j * 32, ci0 % p.CII,
                                                 tap, ci0 / p.CII, mk0);
                        }
                    }
                    T2SP_TRACE(p, 22, it);
                }
            }
        } else if (warp >= 2) {
            // quarters 2 and 3, first half of the k-block. B pieces: 8 per thread in warps 12 and 13, 4 per thread in the
            // other four, so that each of the SM's four schedulers (warp % 4) carries the same number of conversions
            split_role(warp, 0, 1, 512 + (warp - 2) * 128, std::integral_constant<int, 4>{});
        } else if (warp == 1 && lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (leader CTA)
            int it = 0, gch = 0;
            bool ok = true;
            constexpr uint32_t kStepB = Cfg::kBMnMajor ? ((8 * 128) >> 4) : 2u;      // 8 K values of the fp32 tile
            constexpr uint32_t kLboB = Cfg::kBMnMajor ? Cfg::kBoxBytesMn : 16;
            constexpr uint32_t kStepB16 = Cfg::kBMnMajor ? ((16 * 128) >> 4) : 2u;   // 16 K values of a bf16 tile
            // the same tile shape and operand majors as p.idesc, with bf16 operands
            const uint32_t idesc16 = (p.idesc & ~((7u << 7) | (7u << 10))) | (1u << 7) | (1u << 10);
            const uint32_t d_acc = tmem_base;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                const int nkb = item_kb_count(t);
                for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                    const int kend = min(kb0 + Cfg::kChunkKb, nkb);
                    for (int kb = kb0; kb < kend; ++kb, ++it) {
                        const int s = it % STAGES;
                        const int ls = it % Cfg::kSlots;
                        if (!bounded_wait(&ready_bar[ls], (it / Cfg::kSlots) & 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        if (kb == kb0) {
                            // the accumulator is free once the epilogue warps of both CTAs drained the previous chunk
                            if (!bounded_wait(cempty_bar, (gch & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        }
                        ptx::tc_fence_after_sync();
                        T2SP_TRACE(p, 3, it);
                        const uint32_t sb = ptx::smem_u32(smem + s * Cfg::kStageBytes + Cfg::kABytes);
                        const uint32_t s16 = ptx::smem_u32(b16_ring + ls * Cfg::kB16Bytes);
                        const uint64_t db = ptx::make_smem_desc(sb, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                        const uint64_t db_hb = Cfg::kBMnMajor ? ptx::make_smem_desc(s16, 4096, 1024) : ptx::make_smem_desc(s16, 16, 1024);
                        const uint64_t db_lb = Cfg::kBMnMajor ? ptx::make_smem_desc(s16 + Cfg::kB16Bytes / 2, 4096, 1024)
                                                              : ptx::make_smem_desc(s16 + 64, 16, 1024);
                        const uint32_t a_hi = tmem_base + Cfg::kASlotCol0 + ls * 64, a_hb = a_hi + 32, a_lb = a_hi + 48;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ptx::umma_a_tmem<ptx::KIND_TF32, 2>(d_acc, a_hi + 8 * j, db + j * kStepB, p.idesc, ((kb - kb0) | j) ? 1u : 0u);
                        if (!p.single_pass) {
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                ptx::umma_a_tmem<ptx::KIND_F16, 2>(d_acc, a_lb + 8 * j, db_hb + j * kStepB16, idesc16, 1u);
                                ptx::umma_a_tmem<ptx::KIND_F16, 2>(d_acc, a_hb + 8 * j, db_lb + j * kStepB16, idesc16, 1u);
                            }
                        }
                        ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 1));
                        ptx::umma_commit_pair(ptx::map_to_cta(&free_bar[ls], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&free_bar[ls], 1));
                        T2SP_TRACE(p, 4, it);
                    }
                    if (ok) {
                        ptx::umma_commit_pair(ptx::map_to_cta(cfull_bar, 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(cfull_bar, 1));
                    }
                }
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------ epilogue (both CTAs)
        set_max_regs_inc<176>();
        const int e = warp - 4;               // 0..7
        const int q = warp & 3;               // TMEM lane quarter
        const int half = e >> 2;              // which half of the tile's columns
        constexpr int CW = Cfg::kColsPerWarp;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * CW;
        int lt = 0, gch = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
            int mb, nb;
            tile_coords(t / splits, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
            const int nkb = item_kb_count(t);
            const int row_shift = (t % splits) * p.slab_rows;
            const int row = q * 32 + lane;
            const int m_cta0 = mb * 256 + static_cast<int>(rank) * kBlockM;
            const int m = m_cta0 + row;
            const int n0 = nb * UN + half * CW;
            long long* ntab = ntable + e * 256;
            long long offm = 0;
            if (p.epi == EPI_SCATTER) {
                __syncwarp();
                for (int j = lane; j < CW; j += 32) ntab[j] = digits_offset(p.dn, n0 + j);
                offm = digits_offset(p.dm, m);
                __syncwarp();
            }
            // (one uniform add-from-zero loop: with the first chunk loaded straight into `sum` the compiler spilled)
            uint32_t sum[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) sum[j] = 0u;
            for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                if (!bounded_wait_warp(cfull_bar, gch & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                if (threadIdx.x == 128) T2SP_TRACE(p, 5, gch);
#pragma unroll
                for (int c = 0; c < CW / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(lane_base + c * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_peer(cempty_bar, 0);
                if (threadIdx.x == 128) T2SP_TRACE(p, 6, gch);
            }
            if (!ok) break;
            uint32_t* out32 = reinterpret_cast<uint32_t*>(p.out);
#pragma unroll
            for (int c = 0; c < CW / 32; ++c) {
                if (p.epi == EPI_TMA)
                    store_chunk_tma(p, cstage + e * 4096, row_shift + m_cta0 + q * 32, n0 + c * 32,
                                    *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]), lane);
                else if (m < p.M)
                    store_row_chunk(p, out32, m, n0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]), offm,
                                    ntab + c * 32);
            }
            if (threadIdx.x == 128) T2SP_TRACE(p, 9, lt);
        }
        if (lane == 0) ptx::bulk_wait_all();
    } else {
        // ------------------------------------------------------------ split warps (both CTAs)
        set_max_regs_dec<88>();
        if (warp < 14) split_role(warp & 3, 0, 2, (warp - 12) * 256, std::integral_constant<int, 8>{});                // quarters 0 and 1, whole rows
        else split_role(warp & 3, 1, 1, 512 + (warp - 12) * 128, std::integral_constant<int, 4>{});                    // quarters 2 and 3, second half
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_slot) __nanosleep(200000);
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<2>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace t2sp
