// The large-GEMM variant of the contraction kernel: two CTAs on neighbouring SMs (a cluster of
// 2) cooperate on one 256 x 256 output tile with tcgen05.mma.cta_group::2. Each CTA stages its
// own 128 rows of A and its own 128 columns of B, so every byte of B is fetched by one SM of
// the pair only: per MMA an SM reads 8 KiB of shared memory instead of 12 KiB and receives
// 32 KiB instead of 48 KiB per k-block from L2, which is what keeps the tensor pipe fed.
// No TMA multicast is involved: both CTAs issue plain (cta_group::2) tensor copies into their
// own shared memory and credit the leader CTA's barrier.
//
// Roles per CTA as in umma_core.cuh (warp 0 producer, warp 1 MMA/TMEM, warps 2-5 epilogue); only
// the leader CTA (cluster rank 0) issues MMAs and commits, to the barriers of both CTAs.
#pragma once
#include "umma_core.cuh"

namespace t2sp {

template <int ARITH, int OP, int STAGES>
struct PairCfg {
    using AT = ArithTraits<ARITH>;
    static_assert(ARITH != AR_TF32X3, "the pair kernel serves the 16-bit and 8-bit arithmetics");
    static constexpr bool kBMnMajor = (OP == OP_GEMM);
    static constexpr int kUmmaN = 256;            // columns of the pair's tile
    static constexpr int kHalfN = 128;            // columns of B this CTA stages
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = kHalfN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBoxBytesMn = AT::kBlockK * 128;
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;
    static constexpr int kBoxElemsMn = 128 / AT::kElem;
    static constexpr int kThreads = 6 * 32;
    static constexpr int kTmemCols = 512;         // two 256-column accumulators
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTailBytes = kNumBars * 8 + 16 + 4 * 256 * 8;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kCStageBytes + kTailBytes + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

template <int ARITH, int OP, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<ARITH, OP, STAGES>::kThreads, 1)
umma_pair_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = PairCfg<ARITH, OP, STAGES>;
    using AT = typename Cfg::AT;
    extern __shared__ uint8_t smem_raw[];
    // Both CTAs must place their tiles and barriers at the same shared-memory offsets.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* cstage = smem + STAGES * Cfg::kStageBytes;  // EPI_TMA staging tiles, one per epilogue warp
    uint8_t* tail = cstage + kCStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // leader's: both CTAs' TMA data landed
    uint64_t* empty_bar = full_bar + STAGES;                 // per CTA: MMAs that read the stage retired
    uint64_t* tfull_bar = empty_bar + STAGES;                // per CTA: accumulator complete (2)
    uint64_t* tempty_bar = tfull_bar + 2;                    // leader's: accumulator drained by both CTAs (2)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    uint32_t* abort_slot = tmem_slot + 1;
    long long* ntable = reinterpret_cast<long long*>(tmem_slot + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles of 256 x 256
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tfull_bar[a], 1);
            ptx::mbar_init(&tempty_bar[a], 8);  // 4 epilogue warps in each CTA
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
    ptx::cluster_sync();  // the peer's barriers must be initialised before anything is signalled to them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            ptx::prefetch_tensormap(&p.mapA[0]);
            ptx::prefetch_tensormap(&p.mapB);
            int it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mb, nb;
                tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                const int m0 = mb * 256 + static_cast<int>(rank) * kBlockM;
                const int n0 = nb * Cfg::kUmmaN + static_cast<int>(rank) * Cfg::kHalfN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bounded_wait(&empty_bar[s], ph ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    uint8_t* sa = smem + s * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    const uint32_t leader_full = ptx::map_to_cta(&full_bar[s], 0);
                    if (rank == 0) ptx::mbar_expect_tx(&full_bar[s], 2 * Cfg::kStageBytes);
                    ptx::tma_load_2d_pair(sa, &p.mapA[0], leader_full, kb * AT::kBlockK, m0);
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
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
                const int acc = lt & 1;
                if (!bounded_wait(&tempty_bar[acc], ((lt >> 1) & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kUmmaN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bounded_wait(&full_bar[s], ph, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t sa = ptx::smem_u32(smem + s * Cfg::kStageBytes);
                    const uint64_t da = ptx::make_smem_desc(sa, 16, 1024);
                    const uint64_t db = ptx::make_smem_desc(sa + Cfg::kABytes, kLboB, 1024);
#pragma unroll
                    for (int j = 0; j < AT::kBlockK / AT::kUmmaK; ++j)
                        ptx::umma<AT::kKind, 2>(d_tmem, da + j * kStepK, db + j * kStepB, p.idesc, (kb | j) ? 1u : 0u);
                    // free the stage in both CTAs once these MMAs have read it
                    ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 0));
                    ptx::umma_commit_pair(ptx::map_to_cta(&empty_bar[s], 1));
                }
                if (ok) {
                    ptx::umma_commit_pair(ptx::map_to_cta(&tfull_bar[acc], 0));
                    ptx::umma_commit_pair(ptx::map_to_cta(&tfull_bar[acc], 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int q = warp & 3;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        int lt = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++lt) {
            int mb, nb;
            tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
            const int acc = lt & 1;
            const int m = mb * 256 + static_cast<int>(rank) * kBlockM + q * 32 + lane;
            const int n0 = nb * Cfg::kUmmaN;
            long long* ntab = ntable + (warp - 2) * 256;
            long long offm = 0;
            if (p.epi == EPI_SCATTER) {
                __syncwarp();
                for (int j = lane; j < Cfg::kUmmaN; j += 32) ntab[j] = digits_offset(p.dn, n0 + j);
                offm = digits_offset(p.dm, m);
                __syncwarp();
            }
            if (!bounded_wait_warp(&tfull_bar[acc], (lt >> 1) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
            ptx::tc_fence_after_sync();
            uint32_t* out32 = reinterpret_cast<uint32_t*>(p.out);
#pragma unroll 1
            for (int c = 0; c < Cfg::kUmmaN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(lane_base + acc * Cfg::kUmmaN + c * 32, r);
                ptx::tmem_ld_wait();
                if (p.epi == EPI_TMA)
                    store_chunk_tma(p, cstage + (warp - 2) * 4096, mb * 256 + static_cast<int>(rank) * kBlockM + q * 32,
                                    n0 + c * 32, r, lane);
                else if (m < p.M)
                    store_row_chunk(p, out32, m, n0 + c * 32, r, offm, ntab + c * 32);
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_peer(&tempty_bar[acc], 0);
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= 2 && lane == 0) ptx::bulk_wait_all();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_slot) __nanosleep(200000);
    ptx::cluster_sync();  // neither CTA may release shared memory or TMEM the pair's MMAs still use
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<2>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace t2sp
