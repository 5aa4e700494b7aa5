// 3xTF32 contraction on CTA pairs: the fp32 counterpart of umma_pair.cuh.
//
// With 128 x 128 tiles the 3xTF32 path is bound by shared-memory bandwidth, not by the tensor
// cores: per k-block the three MMAs re-read 96 KB of operands while the split warps move another
// 64 KB. Pairing two CTAs on a 256 x UN tile (tcgen05.mma.cta_group::2, UN = 256 or 128) halves the
// operand bytes each SM reads per flop, which brings shared-memory time down to about the MMA time.
//
// Per CTA: 16 warps in four groups with their own register budgets (setmaxnreg):
//   warps 0-3   warp 0 = TMA producer (own A rows, own half of the B columns), warp 1 = MMA issuer
//               (leader CTA only) and TMEM owner, warps 2-3 split warps
//   warps 4-11  epilogue: two warps per TMEM lane quarter, each owning half of the columns; they add
//               every K-chunk of the hi*hi accumulator into fp32 registers (round-to-nearest), then the
//               cross-term accumulator, then store
//   warps 12-15 split warps (with 2-3): lo = x - trunc_tf32(x) of this CTA's raw tiles into the lo ring
// TMEM per CTA: [main UN columns | cross terms UN columns]. The main accumulator is single-buffered:
// the MMA issuer pauses for the drain once per chunk (a few per cent of a chunk's MMA time).
#pragma once
#include "umma_core.cuh"

namespace t2sp {

template <int OP, int UN, int STAGES, int LOSLOTS = 2>
struct X3PairCfg {
    static constexpr bool kBMnMajor = (OP == OP_GEMM || OP == OP_CONV || OP == OP_CAPSULE);
    static constexpr int kHalfN = UN / 2;         // B columns staged by one CTA
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = kHalfN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kLoSlots = LOSLOTS;
    static constexpr int kBoxBytesMn = 32 * 128;  // MN-major fp32 box: 32 k-rows x 32 columns
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;
    static constexpr uint32_t kBSwizzle = kBMnMajor ? 1u : 2u;
    static constexpr uint32_t kBSbo = kBMnMajor ? 512u : 1024u;
    static constexpr int kThreads = 16 * 32;
    static constexpr int kSplitThreads = 6 * 32;
    static constexpr int kTmemCols = 2 * UN;
    static constexpr int kChunkKb = 8;
    static constexpr int kColsPerWarp = UN / 2;   // epilogue: columns summed by one warp
    // EPI_TMA staging (one 4 KiB tile per epilogue warp); the same bytes hold the per-warp column
    // offset tables of EPI_SCATTER (8 x 256 x 8 B = 16 KiB), the two modes never run together
    static constexpr int kCStage = 8 * 4096;
    static constexpr int kNumBars = 2 * STAGES + 2 * LOSLOTS + 4;
    static constexpr int kTailBytes = kNumBars * 8 + 16;
    static constexpr int kSmemBytes = (STAGES + kLoSlots) * kStageBytes + kCStage + kTailBytes + 1024;
    static_assert(kTmemCols == 256 || kTmemCols == 512, "TMEM columns must be a power of two");
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

template <int N>
__device__ __forceinline__ void set_max_regs_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void set_max_regs_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <int OP, int UN, int STAGES, int LOSLOTS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(X3PairCfg<OP, UN, STAGES, LOSLOTS>::kThreads, 1)
umma_x3pair_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = X3PairCfg<OP, UN, STAGES, LOSLOTS>;
    constexpr int kKind = ptx::KIND_TF32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* lo_ring = smem + STAGES * Cfg::kStageBytes;
    uint8_t* cstage = lo_ring + Cfg::kLoSlots * Cfg::kStageBytes;
    uint8_t* tail = cstage + Cfg::kCStage;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // own: this CTA's TMA data landed
    uint64_t* empty_bar = full_bar + STAGES;                 // own: MMAs that read the stage retired
    uint64_t* ready_bar = empty_bar + STAGES;                // leader's: both CTAs' lo slots written (2)
    uint64_t* lofree_bar = ready_bar + Cfg::kLoSlots;        // own: MMAs that read the lo slot retired
    uint64_t* cfull_bar = lofree_bar + Cfg::kLoSlots;                    // own: a chunk of the main accumulator is complete
    uint64_t* cempty_bar = cfull_bar + 1;                    // leader's: the chunk was drained by both CTAs
    uint64_t* sempty_bar = cempty_bar + 1;                   // leader's: cross terms drained by both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sempty_bar + 1);
    uint32_t* abort_slot = tmem_slot + 1;
    long long* ntable = reinterpret_cast<long long*>(cstage);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    // Work items: tiles of 256 x UN, each cut along the contraction into `splits` ranges of num_kb
    // k-blocks (the last one may be shorter). Item t is range t % splits of tile t / splits; with
    // splits > 1 range s writes its partial tile to rows [s * slab_rows, ...) of the output map.
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
        for (int a = 0; a < Cfg::kLoSlots; ++a) {
            ptx::mbar_init(&ready_bar[a], 12);  // 6 split warps in each CTA
            ptx::mbar_init(&lofree_bar[a], 1);
        }
        ptx::mbar_init(cfull_bar, 1);
        ptx::mbar_init(cempty_bar, 16);         // 8 epilogue warps in each CTA
        ptx::mbar_init(sempty_bar, 16);
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
    if (threadIdx.x == 0) T2SP_TRACE(p, 10, 0);  // both CTAs leave the cluster barrier together: clock offset

    // Split role (warps 2-3 and 12-15 of both CTAs): lo = x - trunc_tf32(x) of this CTA's raw tiles.
    auto split_role = [&](const int st) {
        int it = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            const int nkb = item_kb_count(t);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const int ls = it % Cfg::kLoSlots;
                const uint8_t* hi = smem + s * Cfg::kStageBytes;
                uint8_t* lo = lo_ring + ls * Cfg::kStageBytes;
                if (!bounded_wait_warp(&lofree_bar[ls], ((it / Cfg::kLoSlots) & 1) ^ 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                if (st == 0) T2SP_TRACE(p, 8, it);
                if (!bounded_wait_warp(&full_bar[s], ph, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                if (st == 0) T2SP_TRACE(p, 1, it);
                if (!p.single_pass) {
#pragma unroll 4
                    for (int off = st * 16; off < Cfg::kStageBytes; off += Cfg::kSplitThreads * 16) {
                        const float4 v = *reinterpret_cast<const float4*>(hi + off);
                        float4 l;
                        l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
                        l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
                        l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
                        l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
                        *reinterpret_cast<float4*>(lo + off) = l;
                    }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (st == 0) T2SP_TRACE(p, 2, it);
                if (lane == 0) {
                    if (rank == 0) ptx::mbar_arrive(&ready_bar[ls]);
                    else ptx::mbar_arrive_peer(&ready_bar[ls], 0);
                }
                if (st == 0) T2SP_TRACE(p, 11, it);
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
            int it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mb, nb;
                tile_coords(t / splits, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                const int m0 = mb * 256 + static_cast<int>(rank) * kBlockM;
                const int n0 = nb * UN + static_cast<int>(rank) * Cfg::kHalfN;
                const int kb_begin = item_kb_begin(t), nkb = item_kb_count(t);
                // Tiles walk their k-blocks from different starting points (a sum over k either way): CTAs
                // that run in step would otherwise all ask for the same 128-byte column of every operand
                // row at the same time, which lands on a fraction of the DRAM channels.
                const int rot = t % nkb;
                for (int step = 0; step < nkb; ++step, ++it) {
                    const int kb = kb_begin + (step + rot) % nkb;
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bounded_wait(&empty_bar[s], ph ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    uint8_t* sa = smem + s * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    T2SP_TRACE(p, 0, it);
                    ptx::mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
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
                }
            }
        } else if (warp >= 2) {
            split_role((warp - 2) * 32 + lane);
        } else if (warp == 1 && lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (leader CTA)
            int it = 0, lt = 0, gch = 0;
            bool ok = true;
            constexpr uint32_t kStepK = 32 >> 4;
            constexpr uint32_t kStepB = Cfg::kBMnMajor ? ((8 * 128) >> 4) : kStepK;
            constexpr uint32_t kLboB = Cfg::kBMnMajor ? Cfg::kBoxBytesMn : 16;
            const uint32_t d_main = tmem_base, d_small = tmem_base + UN;
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
                const int nkb = item_kb_count(t);
                for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                    const int kend = min(kb0 + Cfg::kChunkKb, nkb);
                    for (int kb = kb0; kb < kend; ++kb, ++it) {
                        const int s = it % STAGES;
                        const int ls = it % Cfg::kLoSlots;
                        if (!bounded_wait(&ready_bar[ls], (it / Cfg::kLoSlots) & 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                        T2SP_TRACE(p, 3, it);
                        const uint32_t sa = ptx::smem_u32(smem + s * Cfg::kStageBytes);
                        const uint32_t la = ptx::smem_u32(lo_ring + ls * Cfg::kStageBytes);
                        const uint64_t da = ptx::make_smem_desc(sa, 16, 1024);
                        const uint64_t db = ptx::make_smem_desc(sa + Cfg::kABytes, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                        const uint64_t dal = ptx::make_smem_desc(la, 16, 1024);
                        const uint64_t dbl = ptx::make_smem_desc(la + Cfg::kABytes, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                        auto issue_main = [&]() {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                ptx::umma<kKind, 2>(d_main, da + j * kStepK, db + j * kStepB, p.idesc, ((kb - kb0) | j) ? 1u : 0u);
                        };
                        auto issue_cross = [&]() {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                ptx::umma<kKind, 2>(d_small, dal + j * kStepK, db + j * kStepB, p.idesc, (kb | j) ? 1u : 0u);
                                ptx::umma<kKind, 2>(d_small, da + j * kStepK, dbl + j * kStepB, p.idesc, 1u);
                            }
                        };
                        // The main accumulator is free once the epilogue warps drained the previous chunk
                        // (cempty), the cross-term accumulator once they drained the previous tile (sempty,
                        // which follows that tile's last cempty). Inside a tile the cross terms of a chunk's
                        // first k-block are issued before the wait on cempty, so the drain overlaps them.
                        if (kb == 0) {
                            if (!bounded_wait(cempty_bar, (gch & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                            ptx::tc_fence_after_sync();
                            issue_main();
                            if (!bounded_wait(sempty_bar, (lt & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                            ptx::tc_fence_after_sync();
                            if (!p.single_pass) issue_cross();
                        } else {
                            if (!p.single_pass) issue_cross();
                            if (kb == kb0) {
                                if (!bounded_wait(cempty_bar, (gch & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                                ptx::tc_fence_after_sync();
                            }
                            issue_main();
                        }
                        ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 1));
                        ptx::umma_commit_pair(ptx::map_to_cta(&lofree_bar[ls], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&lofree_bar[ls], 1));
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
            uint32_t sum[CW];
            for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                if (!bounded_wait_warp(cfull_bar, gch & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                if (threadIdx.x == 128) T2SP_TRACE(p, 5, gch);
                if (kb0 == 0) {
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c)
                        ptx::tmem_ld_32x32(lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]));
                    ptx::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld_32x32(lane_base + c * 32, r);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_peer(cempty_bar, 0);
                if (threadIdx.x == 128) T2SP_TRACE(p, 6, gch);
            }
            if (!ok) break;
            if (!p.single_pass) {
#pragma unroll
                for (int c = 0; c < CW / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(lane_base + UN + c * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_peer(sempty_bar, 0);
            if (threadIdx.x == 128) T2SP_TRACE(p, 7, lt);
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
        split_role((warp - 10) * 32 + lane);
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
