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
// pipe. Here the split warps write the A tile, already split, into tensor memory (tcgen05.st), so the MMAs read only
// B from shared memory: the raw fp32 B tile for the TF32 pass and one 16 KB tile holding bf16(b) and bf16(lo_b) for
// the two bf16 passes.
//
// Three rings per CTA:
//   A stages   kAStages x 16 KB raw fp32 rows, filled by TMA, handed back by the split warps as soon as they hold the
//              values in registers (so the copies of A, the operand that streams from DRAM, run ahead of the split
//              warps, which themselves run up to four k-blocks ahead of the MMAs)
//   B slots    kBSlots x 32 KB [raw fp32 tile | bf16(b), bf16(lo_b) tile], handed back by the MMAs' commit. Both halves
//              come, ready made, from a pre-pass over the whole of B (one 32 KB bulk copy per k-block of the tile
//              images the pre-pass wrote). That pays when many row tiles re-read a small B (weights, the factor of
//              a TTM), which is when the host side picks this kernel; otherwise umma_x3pair.cuh runs.
//   A slots    4 x 64 columns of tensor memory [hi 32 | bf16(a) 16 | bf16(lo_a) 16], handed back by the MMAs' commit
//              (the same commit that hands back B slot i: k-block it uses slot it % 4 of both)
//
// Per CTA: 16 warps as in umma_x3pair.cuh.
//   warp 0      producer (own 128 A rows, own 128 of the 256 B columns); serves the A and the B queue as they open
//   warp 1      MMA issuer (leader CTA only), TMEM owner
//   warps 2-3, 12-15  split warps. A warp may touch only the TMEM lanes of its quarter (warp % 4), so the A tile goes
//               by quarters: warps 12 and 13 take the rows of quarters 0 and 1, warps 2 / 14 and 3 / 15 share
//               quarters 2 and 3 by halves of the k-block.
//   warps 4-11  epilogue as in umma_x3pair.cuh: every 8 k-blocks the accumulator is added into fp32 registers
//               (round to nearest) and handed back
// TMEM per CTA (512 columns): [accumulator 256 | 4 A slots of 64]; with 128-column tiles [2 accumulators of 128 | 4 A
// slots of 64], so that a chunk accumulates while the one before it is drained, and six A stages.
#pragma once
#include <cuda_bf16.h>

#include <type_traits>

#include "umma_core.cuh"
#include "umma_x3pair.cuh"

namespace t2sp {

template <int OP, int UN_>
struct X3TmCfg {
    static_assert(UN_ == 256 || UN_ == 128, "tile width");
    static constexpr bool kBMnMajor = (OP == OP_GEMM || OP == OP_CONV || OP == OP_CAPSULE);
    static constexpr int UN = UN_;
    static constexpr int kHalfN = UN / 2;
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = kHalfN * 128;  // raw fp32 B tile; the bf16 tile [bf16(b) | bf16(lo_b)] is as large
    static constexpr int kBSlotBytes = 2 * kBBytes;
    static constexpr int kAStages = UN == 256 ? 4 : 6;
    static constexpr int kBSlots = 4;                  // as many as A slots: slot i of both is handed back by one commit
    static constexpr int kTSlots = 4;                  // A slots in tensor memory
    static constexpr int kAccBufs = UN == 256 ? 1 : 2; // 128-column tiles: a chunk accumulates while the one before drains
    static constexpr int kBoxBytesMn = 32 * 128;       // MN-major fp32 box: 32 k-rows x 32 columns
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;
    static constexpr uint32_t kBSwizzle = kBMnMajor ? 1u : 2u;
    static constexpr uint32_t kBSbo = kBMnMajor ? 512u : 1024u;
    static constexpr int kThreads = 16 * 32;
    static constexpr int kTmemCols = 512;
    static constexpr int kASlotCol0 = kAccBufs * UN;
    static constexpr int kChunkKb = 8;
    static constexpr int kColsPerWarp = UN / 2;
    static constexpr int kCStage = 8 * 4096;
    static constexpr int kNumBars = 2 * kAStages + 2 * kBSlots + 2 * kTSlots + 2 * kAccBufs;
    static constexpr int kMaxBoxTab = 16;  // conv / capsule: boxes of an A tile whose row coordinates are kept per tile
    static constexpr int kTailBytes = kNumBars * 8 + 16 + kMaxBoxTab * 16;
    static constexpr int kSmemBytes = kAStages * kABytes + kBSlots * kBSlotBytes + kCStage + kTailBytes + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t x3_pack_bf16(float lo_elem, float hi_elem) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);  // .x (low half) = first argument
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float x3_tf32_lo(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// ONE_CHUNK: every work item has at most kChunkKb k-blocks, so a tile is one chunk and the epilogue loads it straight
// into its registers, all loads in flight at once, instead of adding chunk after chunk: the single accumulator of the
// 256-column form is handed back after a third of the time (a TTM with a contraction of 256, 8 k-blocks per tile).
template <int OP, int UN_, bool ONE_CHUNK = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(X3TmCfg<OP, UN_>::kThreads, 1)
umma_x3tm_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = X3TmCfg<OP, UN_>;
    constexpr int AB = Cfg::kAccBufs;
    constexpr int UN = Cfg::UN, NA = Cfg::kAStages, NB = Cfg::kBSlots, TS = Cfg::kTSlots;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* b_ring = smem + NA * Cfg::kABytes;
    uint8_t* cstage = b_ring + NB * Cfg::kBSlotBytes;
    uint8_t* tail = cstage + Cfg::kCStage;
    uint64_t* afull_bar = reinterpret_cast<uint64_t*>(tail);  // own: this CTA's A rows landed
    uint64_t* aempty_bar = afull_bar + NA;                    // own: all six split warps hold their part in registers
    uint64_t* bfull_bar = aempty_bar + NA;                    // own: this CTA's B columns landed
    uint64_t* ready_bar = bfull_bar + 2 * NB;                 // leader's: both CTAs' A slot written and B slot complete (12)
    uint64_t* tfree_bar = ready_bar + TS;                     // own: MMAs that read the A slot and the B slot retired
    uint64_t* bfree_bar = tfree_bar;                          // (k-block it uses A slot it % 4 and B slot it % 4: one commit)
    static_assert(NB == TS, "the A slots in tensor memory and the B slots share their hand-back barriers");
    uint64_t* cfull_bar = tfree_bar + TS;                     // own: a chunk of an accumulator is complete
    uint64_t* cempty_bar = cfull_bar + AB;                    // leader's: the chunk was drained by both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cempty_bar + AB);
    uint32_t* abort_slot = tmem_slot + 1;
    int* box_tab = reinterpret_cast<int*>(tmem_slot + 4);  // the producer's own
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
        for (int s = 0; s < NA; ++s) {
            ptx::mbar_init(&afull_bar[s], 1);
            ptx::mbar_init(&aempty_bar[s], 6);
        }
        for (int s = 0; s < NB; ++s) {
            ptx::mbar_init(&bfull_bar[s], 1);
        }
        for (int a = 0; a < TS; ++a) {
            ptx::mbar_init(&ready_bar[a], 12);  // 6 split warps in each CTA
            ptx::mbar_init(&tfree_bar[a], 1);
        }
        for (int a = 0; a < AB; ++a) {
            ptx::mbar_init(&cfull_bar[a], 1);
            ptx::mbar_init(&cempty_bar[a], 16);  // 8 epilogue warps in each CTA
        }
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

    // Split role. `q`: TMEM lane quarter of the warp; `a_half0`, A_HALVES: which halves of the k-block's 32 columns of
    // the quarter's A rows this warp converts.
    auto split_role = [&](const int q, const int a_half0, auto halves_const) {
        constexpr int A_HALVES = decltype(halves_const)::value;
        int it = 0;
        bool ok = true;
        const int row = q * 32 + lane;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            const int nkb = item_kb_count(t);
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int sa = it % NA, ts = it % TS;
                const uint8_t* araw = smem + sa * Cfg::kABytes;
                if (!bounded_wait_warp(&afull_bar[sa], (it / NA) & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 1, it);
                if (!bounded_wait_warp(&tfree_bar[ts], ((it / TS) & 1) ^ 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                // A: this thread's tile row (16-byte chunk c sits at c ^ (row & 7)), half a k-block at a time:
                // raw words for the TF32 pass, bf16(a) and bf16(lo_a) (two k values per 32-bit column) for the others
                const uint8_t* rp = araw + row * 128;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::kASlotCol0 + ts * 64;
#pragma unroll
                for (int hh = 0; hh < A_HALVES; ++hh) {
                    const int h = a_half0 + hh;
                    uint32_t vh[16], vb[8], vl[8];
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const float4 v = *reinterpret_cast<const float4*>(rp + (((4 * h + cc) ^ (row & 7)) << 4));
                        vh[4 * cc + 0] = __float_as_uint(v.x); vh[4 * cc + 1] = __float_as_uint(v.y);
                        vh[4 * cc + 2] = __float_as_uint(v.z); vh[4 * cc + 3] = __float_as_uint(v.w);
                        vb[2 * cc + 0] = x3_pack_bf16(v.x, v.y); vb[2 * cc + 1] = x3_pack_bf16(v.z, v.w);
                        vl[2 * cc + 0] = x3_pack_bf16(x3_tf32_lo(v.x), x3_tf32_lo(v.y));
                        vl[2 * cc + 1] = x3_pack_bf16(x3_tf32_lo(v.z), x3_tf32_lo(v.w));
                    }
                    ptx::tmem_st_32x16(taddr + 16 * h, vh);
                    ptx::tmem_st_32x8(taddr + 32 + 8 * h, vb);
                    ptx::tmem_st_32x8(taddr + 48 + 8 * h, vl);
                }
                // every loaded value has been consumed by the stores' operands: the stage can take the next copy, long
                // before the MMAs of this k-block run
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&aempty_bar[sa]);
                // B comes ready made; one warp of each CTA (warp 2, which has the least to do) vouches for its arrival,
                // so that `ready` covers both CTAs' B slots
                if (warp == 2) {
                    if (!bounded_wait_warp(&bfull_bar[it % NB], (it / NB) & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) ptx::mbar_arrive(&ready_bar[ts]);
                    else ptx::mbar_arrive_peer(&ready_bar[ts], 0);
                }
                if (warp == 12 && lane == 0) T2SP_TRACE(p, 2, it);
            }
        }
    };

    if (warp < 4) {
        set_max_regs_dec<72>();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ producer (both CTAs)
            if constexpr (OP == OP_CAPSULE) {
                for (int i = 0; i < 4; ++i) ptx::prefetch_tensormap(&p.mapA[i]);
            } else {
                ptx::prefetch_tensormap(&p.mapA[0]);
            }
            // Two walks over the same sequence of (tile, k-block): one for the copies of A, one for those of B. A walk
            // keeps its k-block and (conv, capsule) the tap and channel block it stands for up to date by increments:
            // this thread issues every copy of the CTA, and integer divisions per k-block made it the slowest role.
            struct Walk { int t, step, nkb, kb_begin, kb, m0, half, cb, ky, kx; };
            auto decode_kb = [&](Walk& w) {
                if constexpr (OP == OP_CONV || OP == OP_CAPSULE) {
                    const int tap = w.kb / p.cblks;
                    w.cb = w.kb % p.cblks;
                    w.ky = tap % p.KY;
                    w.kx = tap / p.KY;
                }
            };
            auto tile_setup = [&](Walk& w, bool with_rows) {
                if (w.t >= num_tiles) return;
                int mb, nb;
                tile_coords(w.t / splits, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                w.m0 = mb * 256 + static_cast<int>(rank) * kBlockM;
                w.half = nb * 2 + static_cast<int>(rank);
                w.kb_begin = item_kb_begin(w.t);
                w.nkb = item_kb_count(w.t);
                // Tiles walk their k-blocks from different starting points (a sum over k either way), so that CTAs
                // running in step do not all ask for the same 128-byte column of every operand row at the same time.
                w.kb = w.kb_begin + w.t % w.nkb;
                w.step = 0;
                decode_kb(w);
                if constexpr (OP == OP_CONV || OP == OP_CAPSULE) {
                    // row coordinates of the tile's boxes, once per tile (the first kMaxBoxTab of them)
                    if (with_rows)
                        for (int j = 0; j < min(p.rows.boxes_per_tile, Cfg::kMaxBoxTab); ++j) {
                            int r = w.m0 + j * p.rows.rows_per_box;
#pragma unroll
                            for (int d = 0; d < 4; ++d) {
                                int c = 0;
                                if (d < p.rows.nd - 1) { c = r % p.rows.ext[d]; r /= p.rows.ext[d]; }
                                else if (d == p.rows.nd - 1) { c = r; }
                                box_tab[j * 4 + d] = c;
                            }
                        }
                }
            };
            auto advance = [&](Walk& w, bool with_rows) {
                if (++w.step >= w.nkb) {
                    w.t += num_pairs;
                    tile_setup(w, with_rows);
                } else if (++w.kb == w.kb_begin + w.nkb) {
                    w.kb = w.kb_begin;
                    decode_kb(w);
                } else if constexpr (OP == OP_CONV || OP == OP_CAPSULE) {
                    if (++w.cb == p.cblks) {
                        w.cb = 0;
                        if (++w.ky == p.KY) { w.ky = 0; ++w.kx; }
                    }
                }
            };
            bool b_images_ready = false;  // the pre-pass that wrote them may still be running when this grid starts
            Walk wa, wb;
            wa.t = wb.t = pair;
            tile_setup(wa, true);
            tile_setup(wb, false);
            // The two queues are served as they open, neither waits for the other: a copy of A needs a stage the
            // split warps have read, a copy of B a slot whose MMAs have retired, and which of the two comes first
            // changes with how far the split warps are ahead of the MMAs.
            int ia = 0, ib = 0;
            bool ok = true;
            long long idle_since = -1;
            while ((wa.t < num_tiles || wb.t < num_tiles) && ok) {
                bool progressed = false;
                if (wa.t < num_tiles && ptx::mbar_test_wait(&aempty_bar[ia % NA], ((ia / NA) & 1) ^ 1)) {
                    const int s = ia % NA;
                    uint8_t* sa = smem + s * Cfg::kABytes;
                    T2SP_TRACE(p, 0, ia);
                    ptx::mbar_expect_tx(&afull_bar[s], Cfg::kABytes);
                    if constexpr (OP == OP_GEMM || OP == OP_TTM) {
                        ptx::tma_load_2d(sa, &p.mapA[0], &afull_bar[s], wa.kb * 32, wa.m0);
                    } else {
                        const int c0 = wa.cb * 32;
                        for (int j = 0; j < p.rows.boxes_per_tile; ++j) {
                            int c[4];
                            if (j < Cfg::kMaxBoxTab) {
#pragma unroll
                                for (int d = 0; d < 4; ++d) c[d] = box_tab[j * 4 + d];
                            } else {
                                int r = wa.m0 + j * p.rows.rows_per_box;
#pragma unroll
                                for (int d = 0; d < 4; ++d) {
                                    c[d] = 0;
                                    if (d < p.rows.nd - 1) { c[d] = r % p.rows.ext[d]; r /= p.rows.ext[d]; }
                                    else if (d == p.rows.nd - 1) { c[d] = r; }
                                }
                            }
                            uint8_t* dst = sa + j * p.rows.rows_per_box * 128;
                            if constexpr (OP == OP_CONV) {
                                ptx::tma_load_4d(dst, &p.mapA[0], &afull_bar[s], c0, c[0], c[1] + wa.ky, c[2] + wa.kx);
                            } else {
                                // (stride 1 spelled out: this thread issues every copy of the CTA and has no time for divisions)
                                const bool unit = p.stride == 1;
                                const int sy = unit ? 0 : wa.ky % p.stride, sx = unit ? 0 : wa.kx % p.stride;
                                const int dy = unit ? wa.ky : wa.ky / p.stride, dx = unit ? wa.kx : wa.kx / p.stride;
                                ptx::tma_load_5d(dst, &p.mapA[sy + 2 * sx], &afull_bar[s], c0, c[0], c[1] + dy, c[2] + dx, c[3]);
                            }
                        }
                    }
                    ++ia;
                    advance(wa, true);
                    progressed = true;
                }
                if (wb.t < num_tiles && ptx::mbar_test_wait(&bfree_bar[ib % NB], ((ib / NB) & 1) ^ 1)) {
                    const int sl = ib % NB;
                    if (!b_images_ready) { ptx::grid_dep_wait(); b_images_ready = true; }
                    T2SP_TRACE(p, 22, ib);
                    // the pre-pass wrote, per k-block and half tile, the 32 KB image of the slot
                    ptx::mbar_expect_tx(&bfull_bar[sl], Cfg::kBSlotBytes);
                    ptx::bulk_load(b_ring + sl * Cfg::kBSlotBytes,
                                   static_cast<const uint8_t*>(p.b_images) +
                                       (static_cast<size_t>(wb.kb) * p.b_halves + wb.half) * Cfg::kBSlotBytes,
                                   Cfg::kBSlotBytes, &bfull_bar[sl]);
                    ++ib;
                    advance(wb, false);
                    progressed = true;
                }
                if (progressed) {
                    idle_since = -1;
                } else {
                    // bounded like every other wait: give up when neither queue has opened for the limit
                    const long long now = clock64();
                    if (idle_since < 0) idle_since = now;
                    if (*ab.flag) { ok = false; break; }
                    if (now - idle_since > ab.limit) {
                        *ab.flag = 1u;
                        atomicOr(ab.status, ST_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    __nanosleep(64);
                }
            }
        } else if (warp >= 2) {
            split_role(warp, 0, std::integral_constant<int, 1>{});  // quarters 2 and 3, first half of the k-block
        } else if (warp == 1 && lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (leader CTA)
            int it = 0, gch = 0;
            bool ok = true;
            constexpr uint32_t kStepB = Cfg::kBMnMajor ? ((8 * 128) >> 4) : 2u;      // 8 K values of the fp32 tile
            constexpr uint32_t kLboB = Cfg::kBMnMajor ? Cfg::kBoxBytesMn : 16;
            constexpr uint32_t kStepB16 = Cfg::kBMnMajor ? ((16 * 128) >> 4) : 2u;   // 16 K values of a bf16 tile
            // the same tile shape and operand majors as p.idesc, with bf16 operands
            const uint32_t idesc16 = (p.idesc & ~((7u << 7) | (7u << 10))) | (1u << 7) | (1u << 10);
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                const int nkb = item_kb_count(t);
                for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                    const int kend = min(kb0 + Cfg::kChunkKb, nkb);
                    const int acc = gch % AB;
                    const uint32_t d_acc = tmem_base + acc * UN;
                    for (int kb = kb0; kb < kend; ++kb, ++it) {
                        const int sl = it % NB, ts = it % TS;
                        if (!bounded_wait(&ready_bar[ts], (it / TS) & 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        if (kb == kb0) {
                            // the accumulator is free once the epilogue warps of both CTAs drained the chunk that used it last
                            if (!bounded_wait(&cempty_bar[acc], ((gch / AB) & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        }
                        ptx::tc_fence_after_sync();
                        T2SP_TRACE(p, 3, it);
                        const uint32_t sb = ptx::smem_u32(b_ring + sl * Cfg::kBSlotBytes);
                        const uint32_t s16 = sb + Cfg::kBBytes;
                        const uint64_t db = ptx::make_smem_desc(sb, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                        const uint64_t db_hb = Cfg::kBMnMajor ? ptx::make_smem_desc(s16, 4096, 1024) : ptx::make_smem_desc(s16, 16, 1024);
                        const uint64_t db_lb = Cfg::kBMnMajor ? ptx::make_smem_desc(s16 + Cfg::kBBytes / 2, 4096, 1024)
                                                              : ptx::make_smem_desc(s16 + 64, 16, 1024);
                        const uint32_t a_hi = tmem_base + Cfg::kASlotCol0 + ts * 64, a_hb = a_hi + 32, a_lb = a_hi + 48;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ptx::umma_a_tmem<ptx::KIND_TF32, 2>(d_acc, a_hi + 8 * j, db + j * kStepB, p.idesc, ((kb - kb0) | j) ? 1u : 0u);
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            ptx::umma_a_tmem<ptx::KIND_F16, 2>(d_acc, a_lb + 8 * j, db_hb + j * kStepB16, idesc16, 1u);
                            ptx::umma_a_tmem<ptx::KIND_F16, 2>(d_acc, a_hb + 8 * j, db_lb + j * kStepB16, idesc16, 1u);
                        }
                        ptx::umma_commit_pair(ptx::map_to_cta(&tfree_bar[ts], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&tfree_bar[ts], 1));
                        T2SP_TRACE(p, 4, it);
                    }
                    if (ok) {
                        ptx::umma_commit_pair(ptx::map_to_cta(&cfull_bar[acc], 0));
                        ptx::umma_commit_pair(ptx::map_to_cta(&cfull_bar[acc], 1));
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
            if constexpr (ONE_CHUNK) {
                const int acc = gch % AB;
                if (!bounded_wait_warp(&cfull_bar[acc], (gch / AB) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                if (threadIdx.x == 128) T2SP_TRACE(p, 5, gch);
#pragma unroll
                for (int c = 0; c < CW / 32; ++c)
                    ptx::tmem_ld_32x32(lane_base + acc * UN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]));
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_peer(&cempty_bar[acc], 0);
                if (threadIdx.x == 128) T2SP_TRACE(p, 6, gch);
                ++gch;
            } else {
                // (one uniform add-from-zero loop: with the first chunk loaded straight into `sum` and the later ones
                // added the compiler spilled)
                // 256-column form (one accumulator, the MMAs wait for every drain): the first chunk goes straight into
                // the sums, all loads in flight at once (conv cfg2, three chunks per item: 68.2 -> 66.5 us). The
                // 128-column form drains behind the MMAs of the next chunk and was slower with it (capsule 65 -> 70 us).
                constexpr bool kPeel = UN == 256;
                if constexpr (!kPeel) {
#pragma unroll
                    for (int j = 0; j < CW; ++j) sum[j] = 0u;
                } else {
                    const int acc = gch % AB;
                    if (!bounded_wait_warp(&cfull_bar[acc], (gch / AB) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c)
                        ptx::tmem_ld_32x32(lane_base + acc * UN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]));
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_peer(&cempty_bar[acc], 0);
                    ++gch;
                }
                for (int kb0 = kPeel ? Cfg::kChunkKb : 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                    const int acc = gch % AB;
                    if (!bounded_wait_warp(&cfull_bar[acc], (gch / AB) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (threadIdx.x == 128) T2SP_TRACE(p, 5, gch);
#pragma unroll
                    for (int c = 0; c < CW / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld_32x32(lane_base + acc * UN + c * 32, r);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                    }
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_peer(&cempty_bar[acc], 0);
                    if (threadIdx.x == 128) T2SP_TRACE(p, 6, gch);
                }
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
        if (warp < 14)  // quarters 0 and 1, whole rows
            split_role(warp & 3, 0, std::integral_constant<int, 2>{});
        else            // quarters 2 and 3, second half of the k-block
            split_role(warp & 3, 1, std::integral_constant<int, 1>{});
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
