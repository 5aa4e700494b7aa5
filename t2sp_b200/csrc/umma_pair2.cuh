// CTA-pair GEMM with 512 x 256 tiles: each CTA of the pair owns 256 rows (two 128-row sub-tiles)
// and 128 columns of B, so per k-block an SM receives 48 KiB for twice the work of umma_pair.cuh's
// 32 KiB: 25 % fewer bytes per flop through L2 -> SM, the resource that balances against the MMAs
// there. The price: both TMEM accumulators (2 x 256 columns) belong to one tile, so the drain of a
// tile overlaps only the first sub-tile's share of the next tile's first k-blocks.
// Roles as in umma_pair.cuh. 16-bit and 8-bit arithmetics, OP_GEMM (B MN-major) / OP_TTM (B K-major).
#pragma once
#include "umma_pair.cuh"

namespace t2sp {

template <int ARITH, int OP, int STAGES>
struct Pair2Cfg {
    using AT = ArithTraits<ARITH>;
    static constexpr bool kBMnMajor = (OP == OP_GEMM);
    static constexpr int kUmmaN = 256, kHalfN = 128;
    static constexpr int kSubBytes = kBlockM * 128;      // one 128-row A sub-tile
    static constexpr int kABytes = 2 * kSubBytes;
    static constexpr int kBBytes = kHalfN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBoxBytesMn = AT::kBlockK * 128;
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;
    static constexpr int kBoxElemsMn = 128 / AT::kElem;
    static constexpr int kThreads = 6 * 32;
    static constexpr int kTmemCols = 512;
    static constexpr int kLead = STAGES - 1;  // k-blocks sub-tile 0 runs ahead of sub-tile 1 at a tile's ends
    static constexpr int kNumBars = 2 * STAGES + 4;
    // two 32 x 32 fp32 staging tiles per epilogue warp for the TMA-store epilogue; the scatter epilogue,
    // which does not stage, keeps its per-warp column tables (4 x 256 offsets) in the same bytes
    static constexpr int kCStageBytes2 = 4 * 2 * 4096;
    static_assert(kCStageBytes2 >= 4 * 256 * 8, "column tables must fit the staging bytes");
    static constexpr int kTailBytes = kNumBars * 8 + 16;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kCStageBytes2 + kTailBytes + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

template <int ARITH, int OP, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Pair2Cfg<ARITH, OP, STAGES>::kThreads, 1)
umma_pair2_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = Pair2Cfg<ARITH, OP, STAGES>;
    using AT = typename Cfg::AT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* cstage = smem + STAGES * Cfg::kStageBytes;
    uint8_t* tail = cstage + Cfg::kCStageBytes2;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // leader's: both CTAs' TMA data landed
    uint64_t* empty_bar = full_bar + STAGES;                 // per CTA: MMAs that read the stage retired
    uint64_t* tfull_bar = empty_bar + STAGES;                // per CTA: the tile's accumulator of sub-tile 0 / 1 is complete
    uint64_t* tempty_bar = tfull_bar + 2;                    // leader's: accumulator of sub-tile 0 / 1 drained by both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    uint32_t* abort_slot = tmem_slot + 1;
    long long* ntable = reinterpret_cast<long long*>(cstage);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles of 512 x 256
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tfull_bar[a], 1);
            ptx::mbar_init(&tempty_bar[a], 8);
        }
        *abort_slot = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            ptx::prefetch_tensormap(&p.mapA[0]);
            ptx::prefetch_tensormap(&p.mapB);
            T2SP_TRACE_CLOCK(p, 0);
            int it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mb, nb;
                tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                // sub-tile u of this CTA covers rows mb*512 + u*256 + rank*128 .. +127: MMA u then spans
                // 256 consecutive rows (128 from each CTA)
                const int m0 = mb * 512 + static_cast<int>(rank) * kBlockM;
                const int n0 = nb * Cfg::kUmmaN + static_cast<int>(rank) * Cfg::kHalfN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bounded_wait(&empty_bar[s], ph ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    T2SP_TRACE(p, 0, it);
                    uint8_t* sa = smem + s * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    const uint32_t leader_full = ptx::map_to_cta(&full_bar[s], 0);
                    if (rank == 0) ptx::mbar_expect_tx(&full_bar[s], 2 * Cfg::kStageBytes);
                    ptx::tma_load_2d_pair(sa, &p.mapA[0], leader_full, kb * AT::kBlockK, m0);
                    ptx::tma_load_2d_pair(sa + Cfg::kSubBytes, &p.mapA[0], leader_full, kb * AT::kBlockK, m0 + 256);
                    if constexpr (Cfg::kBMnMajor) {
#pragma unroll
                        for (int j = 0; j < Cfg::kBoxesMn; ++j)
                            ptx::tma_load_2d_pair(sb + j * Cfg::kBoxBytesMn, &p.mapB, leader_full,
                                                  n0 + j * Cfg::kBoxElemsMn, kb * AT::kBlockK);
                    } else {
                        ptx::tma_load_2d_pair(sb, &p.mapB, leader_full, kb * AT::kBlockK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            int it = 0, lt = 0;
            bool ok = true;
            constexpr uint32_t kStepK = 32 >> 4;
            constexpr uint32_t kStepMn = (AT::kUmmaK * 128) >> 4;
            constexpr uint32_t kStepB = Cfg::kBMnMajor ? kStepMn : kStepK;
            constexpr uint32_t kLboB = Cfg::kBMnMajor ? Cfg::kBoxBytesMn : 16;
            // Sub-tile 0 runs `lead` k-blocks ahead of sub-tile 1 at both ends of a tile: at the start its MMAs
            // begin as soon as accumulator 0 has been drained, while accumulator 1 is still leaving; at the end
            // it finishes early, so its drain runs under sub-tile 1's last MMAs. In between the two advance in
            // step, one stage per k-block. All `lead` stages are held while a sub-tile runs alone.
            const int lead = Cfg::kLead < p.num_kb / 2 ? Cfg::kLead : p.num_kb / 2;
            auto wait_full = [&](int i) -> bool {
                T2SP_TRACE(p, 8, i);
                if (!bounded_wait(&full_bar[i % STAGES], (i / STAGES) & 1, ab, ST_TIMEOUT_MMA)) return false;
                ptx::tc_fence_after_sync();
                T2SP_TRACE(p, 3, i);
                return true;
            };
            auto issue = [&](int u, int kb, int i) {
                const uint32_t sa = ptx::smem_u32(smem + (i % STAGES) * Cfg::kStageBytes);
                const uint64_t db = ptx::make_smem_desc(sa + Cfg::kABytes, kLboB, 1024);
                const uint64_t da = ptx::make_smem_desc(sa + u * Cfg::kSubBytes, 16, 1024);
#pragma unroll
                for (int j = 0; j < AT::kBlockK / AT::kUmmaK; ++j)
                    ptx::umma<AT::kKind, 2>(tmem_base + u * Cfg::kUmmaN, da + j * kStepK, db + j * kStepB, p.idesc,
                                            (kb | j) ? 1u : 0u);
            };
            auto release = [&](int i) {  // both sub-tiles' MMAs on the stage have been issued
                ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[i % STAGES], 0));
                ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[i % STAGES], 1));
                T2SP_TRACE(p, 4, i);
            };
            auto wait_drained = [&](int u) -> bool {  // the previous tile's accumulator u, by both CTAs
                if (!bounded_wait(&tempty_bar[u], (lt & 1) ^ 1, ab, ST_TIMEOUT_MMA)) return false;
                ptx::tc_fence_after_sync();
                T2SP_TRACE(p, 10, lt * 2 + u);
                return true;
            };
            auto accumulator_done = [&](int u) {
                ptx::umma_commit_pair(ptx::map_to_cta(&tfull_bar[u], 0));
                ptx::umma_commit_pair(ptx::map_to_cta(&tfull_bar[u], 1));
            };
            const int n = p.num_kb;
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt, it += n) {
                ok = wait_drained(0);
                for (int kb = 0; kb < lead && ok; ++kb) {
                    ok = wait_full(it + kb);
                    if (ok) issue(0, kb, it + kb);
                }
                ok = ok && wait_drained(1);
                for (int kb = 0; kb < lead && ok; ++kb) {
                    issue(1, kb, it + kb);
                    release(it + kb);
                }
                for (int kb = lead; kb < n - lead && ok; ++kb) {
                    ok = wait_full(it + kb);
                    if (!ok) break;
                    issue(0, kb, it + kb);
                    issue(1, kb, it + kb);
                    release(it + kb);
                }
                for (int kb = n - lead; kb < n && ok; ++kb) {
                    ok = wait_full(it + kb);
                    if (ok) issue(0, kb, it + kb);
                }
                if (!ok) break;
                accumulator_done(0);
                for (int kb = n - lead; kb < n; ++kb) {
                    issue(1, kb, it + kb);
                    release(it + kb);
                }
                accumulator_done(1);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 2 x 128 rows)
        const int q = warp & 3;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        int lt = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
            int mb, nb;
            tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
            const int n0 = nb * Cfg::kUmmaN;
            long long* ntab = ntable + (warp - 2) * 256;
            if (p.epi == EPI_SCATTER) {
                __syncwarp();
                for (int j = lane; j < Cfg::kUmmaN; j += 32) ntab[j] = digits_offset(p.dn, n0 + j);
                __syncwarp();
            }
            if (!bounded_wait_warp(&tfull_bar[0], lt & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
            ptx::tc_fence_after_sync();
            if (warp == 2 && lane == 0) T2SP_TRACE(p, 5, lt);
            uint32_t* out32 = reinterpret_cast<uint32_t*>(p.out);
            if (p.epi == EPI_TMA) {
                // The 16 chunks of 32 columns (sub-tile 0's eight, then sub-tile 1's) go through two
                // staging tiles in turn: the load of chunk c+1 from tensor memory is in flight while chunk
                // c is written to shared memory and handed to the TMA, and a staging tile is rewritten once
                // the store issued two chunks earlier has read it. An accumulator is released as soon as
                // its last chunk is in registers. The drain runs at the rate one SM can write towards L2
                // (measured: a CTA's 256 KB take 8100-8500 cycles, 31-32 bytes per cycle, the same with
                // coalesced st.global.v4 instead of TMA stores and with the CTAs' drains staggered in time).
                uint8_t* stage0 = cstage + (warp - 2) * 8192;
                const int m_q = mb * 512 + static_cast<int>(rank) * kBlockM + q * 32;
                auto put = [&](const uint32_t (&r)[32], int c) {
                    uint8_t* buf = stage0 + (c & 1) * 4096;
                    if (lane == 0) ptx::bulk_wait_read_1();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                            make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    const int m_warp0 = m_q + (c >> 3) * 256, nc = n0 + (c & 7) * 32;
                    if (lane == 0) {
                        if (m_warp0 < p.M && nc < p.N) ptx::tma_store_2d(&p.mapC, buf, nc, m_warp0);
                        ptx::bulk_commit_group();  // also when nothing was stored: the wait above counts groups
                    }
                };
                auto loaded = [&](int c) {  // chunk c has left tensor memory
                    ptx::tmem_ld_wait();
                    if ((c & 7) == 7) {
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_peer(&tempty_bar[c >> 3], 0);
                    }
                    if (warp == 2 && lane == 0) T2SP_TRACE(p, 6, lt * 16 + c);
                };
                uint32_t ra[32], rb[32];
                ptx::tmem_ld_32x32(lane_base, ra);
                loaded(0);
#pragma unroll 1
                for (int c = 0; c < 16; c += 2) {
                    ptx::tmem_ld_32x32(lane_base + (c + 1) * 32, rb);
                    put(ra, c);
                    loaded(c + 1);
                    if (c + 2 == 8) {  // sub-tile 1's accumulator completes later than sub-tile 0's
                        if (!bounded_wait_warp(&tfull_bar[1], lt & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                    }
                    if (c + 2 < 16) ptx::tmem_ld_32x32(lane_base + (c + 2) * 32, ra);
                    put(rb, c + 1);
                    if (c + 2 < 16) loaded(c + 2);
                    if (warp == 2 && lane == 0) T2SP_TRACE(p, 7, lt * 16 + c + 1);
                }
            } else {
#pragma unroll 1
                for (int u = 0; u < 2; ++u) {
                    if (u == 1) {
                        if (!bounded_wait_warp(&tfull_bar[1], lt & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                    }
                    const int m = mb * 512 + u * 256 + static_cast<int>(rank) * kBlockM + q * 32 + lane;
                    const long long offm = (p.epi == EPI_SCATTER) ? digits_offset(p.dm, m) : 0;
#pragma unroll 1
                    for (int c = 0; c < Cfg::kUmmaN / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld_32x32(lane_base + u * Cfg::kUmmaN + c * 32, r);
                        ptx::tmem_ld_wait();
                        if (m < p.M) store_row_chunk(p, out32, m, n0 + c * 32, r, offm, ntab + c * 32);
                    }
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_peer(&tempty_bar[u], 0);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (threadIdx.x == 0) T2SP_TRACE_CLOCK(p, 1);
    if (warp >= 2 && lane == 0) ptx::bulk_wait_all();
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
