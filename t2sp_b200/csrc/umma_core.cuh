// The one contraction kernel every operator lowers to.
//
// D[M,N] = sum_K A[M,K] * B[K,N] on the sm_100a tensor cores: TMA streams 128-byte-swizzled
// operand tiles into a multi-stage shared-memory ring, one thread issues tcgen05.mma into a
// double-buffered TMEM accumulator, four epilogue warps drain TMEM to global memory.
// Operators differ only in (a) how a (tile, k-block) pair turns into TMA box coordinates
// (plain matrix, implicit-GEMM convolution, capsule convolution, 3-D tensor slab) and (b)
// how an output (row, column) turns into an address (row-major, column-major, mixed-radix
// scatter for the tiled systolic-array layouts).
//
// Arithmetic variants: 16-bit floats (bf16/f16, fp32 accumulate), int8 (int32 accumulate,
// exact) and "3xTF32" for fp32 data: kind::tf32 reads only the top 19 bits of each fp32 word
// (measured: it truncates), so the raw tile is the hi operand, lo = x - trunc(x) is computed
// into a second tile in shared memory, and three TF32 MMAs (lo*hi, hi*lo, hi*hi) are
// accumulated so the product keeps ~fp32 accuracy. The tensor core adds into its fp32
// accumulator with truncation, a bias that grows with the number of accumulate steps, so the
// 3xTF32 path (a) sums the small cross terms in an accumulator of their own and (b) lets
// the hi*hi accumulator run for only kChunkKb k-blocks before the epilogue warps add it,
// round-to-nearest, into fp32 registers.
//
// Every wait on an mbarrier is bounded: after CoreParams::wait_cycles (kWaitTimeoutCycles by default) the waiting thread raises a
// status bit in global memory, tells the rest of the CTA to stop, and the CTA drains and
// frees its TMEM before returning.
#pragma once
#include "ptx.cuh"
#include "umma_params.h"

namespace t2sp {

template <int ARITH> struct ArithTraits;
template <> struct ArithTraits<AR_F16> {
    static constexpr int kElem = 2, kBlockK = 64, kUmmaK = 16, kKind = ptx::KIND_F16;
};
template <> struct ArithTraits<AR_TF32X3> {
    static constexpr int kElem = 4, kBlockK = 32, kUmmaK = 8, kKind = ptx::KIND_TF32;
};
template <> struct ArithTraits<AR_I8> {
    static constexpr int kElem = 1, kBlockK = 128, kUmmaK = 32, kKind = ptx::KIND_I8;
};

template <int ARITH, int OP, int BN, int STAGES>
struct CoreCfg {
    using AT = ArithTraits<ARITH>;
    static constexpr bool kX3 = (ARITH == AR_TF32X3);
    static constexpr bool kBMnMajor = (OP == OP_GEMM || OP == OP_CONV || OP == OP_CAPSULE);
    static constexpr bool kBGenerated = (OP == OP_MTTKRP);
    // MN-major fp32 tiles use the 32-byte-atom flavour of the 128-byte swizzle (4-row atoms).
    static constexpr uint32_t kBSwizzle = (kBMnMajor && ARITH == AR_TF32X3) ? 1u : 2u;
    static constexpr uint32_t kBSbo = (kBMnMajor && ARITH == AR_TF32X3) ? 512u : 1024u;
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = BN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;    // one ring stage: [A | B] as TMA delivers them
    // 3xTF32: the raw fp32 tiles double as the hi operands (the tensor core reads only the top 19
    // bits of each word); the lo tiles live in a short ring of their own, [A_lo | B_lo] per slot.
    // fp32 tiles keep the A operand of the MMAs in tensor memory: the split warps read the raw A tile
    // once and write hi and lo straight into TMEM (tcgen05.st), so the three MMAs of a product read only
    // B from shared memory. TMEM: 2 * kAccBufs accumulators x BN columns (256 in all) + kLoSlots x (32 hi
    // + 32 lo) columns of A. The lo ring in shared memory then holds B tiles only.
#ifndef T2SP_ATMEM_MAX_BN
#define T2SP_ATMEM_MAX_BN 64
#endif
    static constexpr bool kATmem = kX3 && BN <= T2SP_ATMEM_MAX_BN;
    // accumulators per kind (main chunk / cross terms): two where TMEM has room, else one
    static constexpr int kAccBufs = (kATmem && BN > 64) ? 1 : 2;
    static constexpr int kLoSlots = kX3 ? (kATmem ? 4 : 3) : 0;
    static constexpr int kLoBytes = kATmem ? kBBytes : kStageBytes;  // one lo slot: [A_lo | B_lo], or B_lo alone
    static constexpr int kLoBOff = kATmem ? 0 : kABytes;             // where B_lo starts inside a lo slot
    static constexpr int kATmemCol0 = 256;                           // first TMEM column of the A slots
    // MTTKRP writes its partial slabs column-major and never stages an output tile: its staging
    // bytes go to a deeper lo ring instead.
    static constexpr int kCStage = (OP == OP_MTTKRP) ? 0 : kCStageBytes;
    static constexpr int kBoxBytesMn = AT::kBlockK * 128;           // one MN-major box: kBlockK rows of 128 B
    static constexpr int kBoxesMn = kBBytes / kBoxBytesMn;          // boxes per MN-major B tile
    static constexpr int kBoxElemsMn = 128 / AT::kElem;             // N elements per MN-major box
    // split warps: more of them shorten the time a k-block's lo tiles take (MTTKRP also builds its B tile there)
    // split warps: with A in TMEM a multiple of four (each warp reaches one TMEM lane quarter only); the
    // 128-wide tile keeps four so that its epilogue warps can hold 128 running sums in registers
    static constexpr int kSplitWarps = kX3 ? (kATmem ? (BN <= 64 ? 8 : 4) : (OP == OP_MTTKRP ? (BN <= 64 ? 8 : 4) : 6)) : 0;
    static constexpr int kSplitThreads = kSplitWarps * 32;
    static constexpr int kWarps = 2 + 4 + kSplitWarps;
    static constexpr int kThreads = kWarps * 32;
    // 16-bit / int8: two whole-tile accumulators (tile t+1 accumulates while tile t drains).
    // 3xTF32: two chunk accumulators for the hi*hi products plus two (one per tile in flight) for the
    // small cross terms.
    static constexpr int kTmemCols = kX3 ? ((4 * BN <= 256 && !kATmem) ? 256 : 512) : 2 * BN;
    static constexpr int kChunkKb = 8;  // 3xTF32: k-blocks summed inside TMEM before an fp32 drain
    static constexpr int kNumBars = 2 * STAGES + 14;
    static constexpr int kTailBytes = kNumBars * 8 + 16 + 4 * 256 * 8;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kLoSlots * kLoBytes + kCStage + kTailBytes + 1024;
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "TMEM columns must be a power of two");
    static_assert(!kX3 || 2 * kAccBufs * BN + (kATmem ? kLoSlots * 64 : 0) <= 512, "3xTF32 accumulators and A slots must fit TMEM");
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
    static_assert(!kX3 || STAGES >= kLoSlots, "the stage barriers double as lo-slot barriers: the raw ring must be at least as deep");
};

struct AbortCtx {
    volatile uint32_t* flag;  // shared memory, CTA-wide
    unsigned* status;         // global memory
    long long limit;          // SM cycles a wait may last
};

__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, const AbortCtx& ab, unsigned code) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    // the SM's own cycle counter: cheap to read, and roles that block at every k-block come here often
    const long long t0 = clock64();
    uint32_t polls = 0;
    while (true) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++polls & 0x3Fu) == 0) {
            if (*ab.flag) return false;
            if (clock64() - t0 > ab.limit) {
                *ab.flag = 1u;
                atomicOr(ab.status, code);
                return false;
            }
        }
    }
}

// Warp-wide form: lane 0 polls, every lane gets the verdict, so the warp stays converged
// for the .sync.aligned tcgen05 instructions that follow.
__device__ __forceinline__ bool bounded_wait_warp(uint64_t* bar, uint32_t parity, const AbortCtx& ab, unsigned code,
                                                  int lane) {
    int ok = 1;
    if (lane == 0) ok = bounded_wait(bar, parity, ab, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

__device__ __forceinline__ long long digits_offset(const Digits& d, int x) {
    long long off = 0;
#pragma unroll
    for (int i = 0; i < kMaxDigits; ++i)
        if (i < d.n) off += static_cast<long long>((((x / d.div[i]) % d.mod[i]) / d.div2[i]) % d.mod2[i]) * d.stride[i];
    return off;
}

// k-blocks the tile of split `nb` walks (all tiles walk num_kb except MTTKRP's last split).
template <int OP>
__device__ __forceinline__ int kb_count(const CoreParams& p, int nb) {
    if constexpr (OP == OP_MTTKRP) return max(0, min(p.num_kb, p.total_kb - nb * p.num_kb));
    else return p.num_kb;
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int G, int& mb, int& nb) {
    // Groups of G row-blocks sweep all column-blocks, rows fastest inside a group, so the
    // CTAs running at the same time share a small set of A and B panels in L2.
    const int per_group = G * tiles_n;
    const int g = t / per_group, r = t % per_group;
    const int gm = min(G, tiles_m - g * G);
    mb = g * G + r % gm;
    nb = r / gm;
}


// EPI_TMA: the warp's 32 rows x 32 columns go through a swizzled shared-memory tile and leave as
// one TMA store (full 128-byte lines instead of 32 scattered 16-byte pieces per instruction).
// `buf` is this warp's 4 KiB tile (1024-byte aligned); lane = row within the tile.
__device__ __forceinline__ void store_chunk_tma(const CoreParams& p, uint8_t* buf, int m_warp0, int nc,
                                                const uint32_t (&r)[32], int lane) {
    if (lane == 0) ptx::bulk_wait_read_all();  // the previous store has finished reading the tile
    __syncwarp();
    if (p.tma_t) {
        // column-major output (m contiguous): the tile is staged as [column][row], 128 bytes per column, and one
        // store writes 32 pieces of 128 contiguous bytes (plain stores of the same pieces, one instruction per
        // column with a column pitch between them, held the epilogue warps up for longer than the whole k-loop)
#pragma unroll
        for (int j = 0; j < 32; ++j) *reinterpret_cast<uint32_t*>(buf + j * 128 + lane * 4) = r[j];
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m_warp0 < p.M && nc < p.N) {
            ptx::tma_store_2d(&p.mapC, buf, m_warp0, nc);
            ptx::bulk_commit_group();
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && m_warp0 < p.M && nc < p.N) {
        ptx::tma_store_2d(&p.mapC, buf, nc, m_warp0);
        ptx::bulk_commit_group();
    }
}

// Writes 32 consecutive output columns [nc, nc+32) of row m held in r[] (raw 32-bit words).
__device__ __forceinline__ void store_row_chunk(const CoreParams& p, uint32_t* out32, int m, int nc,
                                                const uint32_t (&r)[32], long long offm, const long long* ntab) {
    if (nc >= p.N) return;
    if (p.epi == EPI_ROWMAJOR && p.use_ab) {
        float* dst = reinterpret_cast<float*>(out32) + static_cast<long long>(m) * p.ldo + nc;
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (nc + j < p.N) {
                const float v = p.alpha * __uint_as_float(r[j]);
                dst[j] = p.beta != 0.f ? v + p.beta * dst[j] : v;
            }
    } else if (p.epi == EPI_ROWMAJOR) {
        uint32_t* dst = out32 + static_cast<long long>(m) * p.ldo + nc;
        if (nc + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) dst[j] = r[j];
        }
    } else if (p.epi == EPI_COLMAJOR) {
        uint32_t* dst = out32 + static_cast<long long>(nc) * p.ldo + m;
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (nc + j < p.N) dst[static_cast<long long>(j) * p.ldo] = r[j];
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (nc + j < p.N) out32[offm + ntab[j]] = r[j];
    }
}

template <int ARITH, int OP, int BN, int STAGES>
__global__ void __launch_bounds__(CoreCfg<ARITH, OP, BN, STAGES>::kThreads, 1)
umma_contract_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = CoreCfg<ARITH, OP, BN, STAGES>;
    using AT = typename Cfg::AT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* lo_ring = smem + STAGES * Cfg::kStageBytes;     // 3xTF32: kLoSlots x [A_lo | B_lo]
    uint8_t* cstage = lo_ring + Cfg::kLoSlots * Cfg::kLoBytes;  // EPI_TMA staging tiles
    uint8_t* tail = cstage + Cfg::kCStage;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // TMA data landed
    uint64_t* empty_bar = full_bar + STAGES;                 // MMAs that read the stage retired
    uint64_t* ready_bar = empty_bar + STAGES;                // 3xTF32: lo slot written (2)
    uint64_t* tfull_bar = ready_bar + 4;                     // accumulator complete (2)
    uint64_t* tempty_bar = tfull_bar + 2;                    // accumulator drained (2)
    uint64_t* sempty_bar = tempty_bar + 2;                   // 3xTF32: cross-term accumulator drained (2)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sempty_bar + 2);
    uint32_t* abort_slot = tmem_slot + 1;
    long long* ntable = reinterpret_cast<long long*>(tmem_slot + 4);  // one 256-entry scatter table per epilogue warp

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 4; ++a) {
            ptx::mbar_init(&ready_bar[a], Cfg::kX3 ? Cfg::kSplitThreads : 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tfull_bar[a], 1);
            ptx::mbar_init(&tempty_bar[a], 4);
        }
        ptx::mbar_init(&sempty_bar[0], 4);
        ptx::mbar_init(&sempty_bar[1], 4);
        *abort_slot = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            if constexpr (OP == OP_CAPSULE) {
                for (int i = 0; i < 4; ++i) ptx::prefetch_tensormap(&p.mapA[i]);
            } else {
                ptx::prefetch_tensormap(&p.mapA[0]);
            }
            ptx::prefetch_tensormap(&p.mapB);
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int mb, nb;
                if constexpr (OP == OP_MTTKRP) { mb = t % p.tiles_m; nb = t / p.tiles_m; }
                else tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
                const int m0 = mb * p.tile_rows, n0 = nb * BN;
                const int nkb = kb_count<OP>(p, nb);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!bounded_wait(&empty_bar[s], ph ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    T2SP_TRACE(p, 0, it);
                    uint8_t* sa = smem + s * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    // Test hook for the bounded waits: this k-block's copies are left out, so its `full` barrier
                    // never completes, the consumer's wait runs out and the CTA takes the abort path.
                    if (p.skip_stage && it + 1 == p.skip_stage) continue;
                    ptx::mbar_expect_tx(&full_bar[s], p.a_tx_bytes + Cfg::kBBytes);
                    if constexpr (OP == OP_GEMM || OP == OP_TTM) {
                        ptx::tma_load_2d(sa, &p.mapA[0], &full_bar[s], kb * AT::kBlockK, m0);
                        if constexpr (OP == OP_TTM) {
                            ptx::tma_load_2d(sb, &p.mapB, &full_bar[s], kb * AT::kBlockK, n0);
                        } else {
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_2d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s],
                                                 n0 + j * Cfg::kBoxElemsMn, kb * AT::kBlockK);
                        }
                    } else if constexpr (OP == OP_CONV || OP == OP_CAPSULE) {
                        const int tap = kb / p.cblks, cb = kb % p.cblks;
                        const int ky = tap % p.KY, kx = tap / p.KY;
                        const int c0 = cb * AT::kBlockK;
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
                                // input tensor (ci, n, iy, ix); rows are (n, oy, ox)
                                ptx::tma_load_4d(dst, &p.mapA[0], &full_bar[s], c0, c[0], c[1] + ky, c[2] + kx);
                            } else {
                                // input tensor per stride parity (c', q, iy', ix', n); rows are (q, oy, ox, n)
                                const int sy = ky % p.stride, sx = kx % p.stride;
                                ptx::tma_load_5d(dst, &p.mapA[sy + 2 * sx], &full_bar[s], c0, c[0],
                                                 c[1] + ky / p.stride, c[2] + kx / p.stride, c[3]);
                            }
                        }
                        if constexpr (OP == OP_CONV) {
                            // weight tensor (co, kx, ci, ky)
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_4d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s],
                                                 n0 + j * Cfg::kBoxElemsMn, kx, c0, ky);
                        } else {
                            // weight tensor (n=(co,my), cii, tap, ci_outer, mk); c' = ci + CI*mk
                            const int mk0 = c0 / p.CI, ci0 = c0 % p.CI;
#pragma unroll
                            for (int j = 0; j < Cfg::kBoxesMn; ++j)
                                ptx::tma_load_5d(sb + j * Cfg::kBoxBytesMn, &p.mapB, &full_bar[s],
                                                 n0 + j * Cfg::kBoxElemsMn, ci0 % p.CII, tap, ci0 / p.CII, mk0);
                        }
                    } else {
                        // MTTKRP: tensor (l, i, k); this CTA's split walks k-blocks [nb*num_kb, (nb+1)*num_kb)
                        // with the l-block fastest, so consecutive stages fetch neighbouring 128-byte
                        // pieces of the same 128 rows. The factor slice c(l-block, all r) lands in the B
                        // region, already in the K-major swizzled layout of the Khatri-Rao tile.
                        const int g = nb * p.num_kb + kb;
                        const int k = g / p.lblks, lb = g % p.lblks;
                        ptx::tma_load_3d(sa, &p.mapA[0], &full_bar[s], lb * AT::kBlockK, m0, k);
                        ptx::tma_load_2d(sb, &p.mapB, &full_bar[s], lb * AT::kBlockK, 0);
                    }
                }
            }
            if (!ok) {
                // Give copies already in flight a bounded chance to land before the CTA exits.
                for (int s = 0; s < STAGES; ++s) {
                    const int last = it - 1 - ((it - 1 - s) % STAGES + STAGES) % STAGES;
                    if (last >= 0) {
                        for (int spin = 0; spin < 4000; ++spin)
                            if (ptx::mbar_try_wait(&full_bar[s], (last / STAGES) & 1)) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // With A in tensor memory the issue loop runs on the whole warp and an elected lane issues each
        // MMA and commit (measured faster there: MTTKRP 202 -> 187 us; with shared-memory descriptors for A
        // the same change was slower, capsule 103 -> 144 us); every other path runs it on lane 0.
        if (Cfg::kATmem || lane == 0) {
            int it = 0, lt = 0;
            bool ok = true;
            constexpr uint32_t kStepK = 32 >> 4;                                           // K-major: 32 B per UMMA
            constexpr uint32_t kStepMn = (AT::kUmmaK * 128) >> 4;                          // MN-major: kUmmaK rows
            constexpr uint32_t kStepB = Cfg::kBMnMajor ? kStepMn : kStepK;
            constexpr uint32_t kLboB = Cfg::kBMnMajor ? Cfg::kBoxBytesMn : 16;
            if constexpr (Cfg::kX3) {
                int gch = 0;
                auto wait_bar = [&](uint64_t* bar, uint32_t parity) {
                    if constexpr (Cfg::kATmem) return bounded_wait_warp(bar, parity, ab, ST_TIMEOUT_MMA, lane);
                    else return bounded_wait(bar, parity, ab, ST_TIMEOUT_MMA);
                };
                for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
                    const int cs = lt % Cfg::kAccBufs;
                    const uint32_t d_small = tmem_base + (Cfg::kAccBufs + cs) * BN;
                    const int nkb = kb_count<OP>(p, (OP == OP_MTTKRP) ? t / p.tiles_m : 0);
                    for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                        const int b = gch % Cfg::kAccBufs;
                        const uint32_t d_main = tmem_base + b * BN;
                        const int kend = min(kb0 + Cfg::kChunkKb, nkb);
                        for (int kb = kb0; kb < kend; ++kb, ++it) {
                            const int s = it % STAGES;
                            const int ls = it % Cfg::kLoSlots;
                            // the splitter arrives on ready[ls] after it has seen full[s], so this
                            // wait covers the raw tiles too
                            if (!wait_bar(&ready_bar[ls], (it / Cfg::kLoSlots) & 1)) { ok = false; break; }
                            ptx::tc_fence_after_sync();
                            if (lane == 0) T2SP_TRACE(p, 3, it);
                            const uint32_t sa = ptx::smem_u32(smem + s * Cfg::kStageBytes);
                            const uint32_t sb = sa + Cfg::kABytes;
                            const uint32_t la = ptx::smem_u32(lo_ring + ls * Cfg::kLoBytes);
                            const uint64_t db = ptx::make_smem_desc(sb, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                            const uint64_t dbl = ptx::make_smem_desc(la + Cfg::kLoBOff, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
                            const uint32_t a_hi = tmem_base + Cfg::kATmemCol0 + ls * 64, a_lo = a_hi + 32;  // kATmem only
                            const uint64_t da = ptx::make_smem_desc(sa, 16, 1024);
                            const uint64_t dal = ptx::make_smem_desc(la, 16, 1024);
                            auto issue_main = [&]() {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t acc = ((kb - kb0) | j) ? 1u : 0u;
                                    if constexpr (Cfg::kATmem) ptx::umma_tf32_a_tmem_warp(d_main, a_hi + 8 * j, db + j * kStepB, p.idesc, acc);
                                    else ptx::umma<AT::kKind, 1>(d_main, da + j * kStepK, db + j * kStepB, p.idesc, acc);
                                }
                            };
                            auto issue_cross = [&]() {
                                if (p.single_pass) return;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t acc = (kb | j) ? 1u : 0u;
                                    if constexpr (Cfg::kATmem) {
                                        ptx::umma_tf32_a_tmem_warp(d_small, a_lo + 8 * j, db + j * kStepB, p.idesc, acc);
                                        ptx::umma_tf32_a_tmem_warp(d_small, a_hi + 8 * j, dbl + j * kStepB, p.idesc, 1u);
                                    } else {
                                        ptx::umma<AT::kKind, 1>(d_small, dal + j * kStepK, db + j * kStepB, p.idesc, acc);
                                        ptx::umma<AT::kKind, 1>(d_small, da + j * kStepK, dbl + j * kStepB, p.idesc, 1u);
                                    }
                                }
                            };
                            // The main accumulator b is free once the epilogue drained the chunk that used
                            // it last (tempty), the cross-term accumulator once the tile that used it last
                            // was drained (sempty, which follows that tile's last tempty). Inside a tile the
                            // cross terms of a chunk's first k-block go out before the wait on tempty.
                            if (kb == 0) {
                                if (!wait_bar(&tempty_bar[b], ((gch / Cfg::kAccBufs) & 1) ^ 1)) { ok = false; break; }
                                ptx::tc_fence_after_sync();
                                issue_main();
                                if (!wait_bar(&sempty_bar[cs], ((lt / Cfg::kAccBufs) & 1) ^ 1)) { ok = false; break; }
                                ptx::tc_fence_after_sync();
                                issue_cross();
                            } else {
                                issue_cross();
                                if (kb == kb0) {
                                    if (!wait_bar(&tempty_bar[b], ((gch / Cfg::kAccBufs) & 1) ^ 1)) { ok = false; break; }
                                    ptx::tc_fence_after_sync();
                                }
                                issue_main();
                            }
                            if constexpr (Cfg::kATmem) ptx::umma_commit_warp(&empty_bar[s]);
                            else ptx::umma_commit(&empty_bar[s]);
                            if (lane == 0) T2SP_TRACE(p, 4, it);
                        }
                        if (ok) {
                            if constexpr (Cfg::kATmem) ptx::umma_commit_warp(&tfull_bar[b]);
                            else ptx::umma_commit(&tfull_bar[b]);
                        }
                    }
                }
            } else {
                for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
                    const int acc = lt & 1;
                    if (!bounded_wait(&tempty_bar[acc], ((lt >> 1) & 1) ^ 1, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int nkb = kb_count<OP>(p, 0);
                    for (int kb = 0; kb < nkb; ++kb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!bounded_wait(&full_bar[s], ph, ab, ST_TIMEOUT_MMA)) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                        const uint32_t sa = ptx::smem_u32(smem + s * Cfg::kStageBytes);
                        const uint32_t sb = sa + Cfg::kABytes;
                        const uint64_t da = ptx::make_smem_desc(sa, 16, 1024);
                        const uint64_t db = ptx::make_smem_desc(sb, kLboB, Cfg::kBSbo, Cfg::kBSwizzle);
#pragma unroll
                        for (int j = 0; j < AT::kBlockK / AT::kUmmaK; ++j)
                            ptx::umma<AT::kKind, 1>(d_tmem, da + j * kStepK, db + j * kStepB, p.idesc,
                                                    (kb | j) ? 1u : 0u);
                        ptx::umma_commit(&empty_bar[s]);
                    }
                    if (ok) ptx::umma_commit(&tfull_bar[acc]);
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (TMEM -> global)
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        int lt = 0, gch = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
            int mb, nb;
            if constexpr (OP == OP_MTTKRP) { mb = t % p.tiles_m; nb = t / p.tiles_m; }
            else tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, mb, nb);
            const int row = q * 32 + lane;
            const int m = mb * p.tile_rows + row;
            const int n0 = (OP == OP_MTTKRP) ? 0 : nb * BN;
            long long* ntab = ntable + (warp - 2) * 256;
            long long offm = 0;
            if (p.epi == EPI_SCATTER) {
                __syncwarp();
                for (int j = lane; j < BN; j += 32) ntab[j] = digits_offset(p.dn, n0 + j);
                offm = digits_offset(p.dm, m);
                __syncwarp();
            }
            uint32_t* out32 = reinterpret_cast<uint32_t*>(p.out);
            if constexpr (OP == OP_MTTKRP) out32 += static_cast<long long>(nb) * p.M * p.N;  // partial slab of this split
            const bool row_ok = row < p.tile_rows && m < p.M;
            if constexpr (Cfg::kX3) {
                uint32_t sum[BN];  // fp32 running sums of this thread's output row, kept as raw bits
                const int nkb = kb_count<OP>(p, nb);
                for (int kb0 = 0; kb0 < nkb && ok; kb0 += Cfg::kChunkKb, ++gch) {
                    const int b = gch % Cfg::kAccBufs;
                    if (!bounded_wait_warp(&tfull_bar[b], (gch / Cfg::kAccBufs) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (kb0 == 0) {
                        // first chunk of the tile: load straight into the sums, all loads in flight at once
#pragma unroll
                        for (int c = 0; c < BN / 32; ++c)
                            ptx::tmem_ld_32x32(lane_base + b * BN + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]));
                        ptx::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 32; ++c) {
                            uint32_t r[32];
                            ptx::tmem_ld_32x32(lane_base + b * BN + c * 32, r);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                        }
                    }
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&tempty_bar[b]);
                }
                if (!ok) break;
                // The last chunk's commit also covers every cross-term MMA of this tile.
                if (!p.single_pass) {
#pragma unroll
                    for (int c = 0; c < BN / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld_32x32(lane_base + (Cfg::kAccBufs + lt % Cfg::kAccBufs) * BN + c * 32, r);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[c * 32 + j] = __float_as_uint(__uint_as_float(sum[c * 32 + j]) + __uint_as_float(r[j]));
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sempty_bar[lt % Cfg::kAccBufs]);
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    if (p.epi == EPI_TMA)
                        store_chunk_tma(p, cstage + (warp - 2) * 4096, mb * p.tile_rows + q * 32, n0 + c * 32,
                                        *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]), lane);
                    else if (row_ok)
                        store_row_chunk(p, out32, m, n0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sum[c * 32]), offm, ntab + c * 32);
                }
            } else {
                const int acc = lt & 1;
                if (!bounded_wait_warp(&tfull_bar[acc], (lt >> 1) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(lane_base + acc * BN + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (p.epi == EPI_TMA) store_chunk_tma(p, cstage + (warp - 2) * 4096, mb * p.tile_rows + q * 32, n0 + c * 32, r, lane);
                    else if (row_ok) store_row_chunk(p, out32, m, n0 + c * 32, r, offm, ntab + c * 32);
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&tempty_bar[acc]);
            }
        }
    } else {
        // ------------------------------------------------------------ 3xTF32 splitter (and MTTKRP B generator)
        if constexpr (Cfg::kX3) {
            const int st = (warp - 6) * 32 + lane;
            int it = 0;
            bool ok = true;
            constexpr int kGenPos = BN * 8 / (Cfg::kBGenerated ? Cfg::kSplitThreads : 128);  // MTTKRP: 16-byte chunks of the generated tile per thread
            static_assert(!Cfg::kBGenerated || (BN * 8) % Cfg::kSplitThreads == 0, "the generated tile must divide among the split threads");
            float gen_b[kGenPos];
            int gen_k = -1;
            (void)gen_b; (void)gen_k;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int nb = (OP == OP_MTTKRP) ? t / p.tiles_m : 0;
                const int nkb = kb_count<OP>(p, nb);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const int ls = it % Cfg::kLoSlots;
                    uint8_t* hi = smem + s * Cfg::kStageBytes;
                    uint8_t* lo = lo_ring + ls * Cfg::kLoBytes;
                    uint8_t* lo_b = lo + Cfg::kLoBOff - Cfg::kABytes;  // lo_b + (offset inside the raw stage) = B_lo position
                    // the lo slot is free once the MMAs that read it last have retired
                    // the lo slot (and the TMEM A slot) is free once the MMAs of k-block it - kLoSlots retired:
                    // that is a completion of that k-block's stage barrier, so one commit per k-block serves
                    // the producer and the split warps alike
                    if (it >= Cfg::kLoSlots) {
                        const int jt = it - Cfg::kLoSlots;
                        if (!bounded_wait_warp(&empty_bar[jt % STAGES], (jt / STAGES) & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                    }
                    if (st == 0) T2SP_TRACE(p, 8, it);
                    if (!bounded_wait_warp(&full_bar[s], ph, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                    if (st == 0) T2SP_TRACE(p, 1, it);
                    if constexpr (Cfg::kBGenerated) {
                        // The B region holds c(l-block, r) as TMA delivered it: row r of the tile, 32
                        // consecutive l values, 128-byte swizzle. Scaling row r by b(k, r) in place turns
                        // it into the Khatri-Rao tile KR[(l,k), r] (the hi operand); lo goes to the lo
                        // slot. Each thread owns kGenPos 16-byte chunks; b(k, :) is constant while the
                        // l-block runs through its lblks values, so it is re-read only when k changes.
                        const int g = nb * p.num_kb + kb;
                        const int k = g / p.lblks;
                        if (k != gen_k) {
                            gen_k = k;
#pragma unroll
                            for (int i = 0; i < kGenPos; ++i) {
                                const int r = (st + Cfg::kSplitThreads * i) >> 3;
                                gen_b[i] = r < p.R ? __ldg(p.fb + static_cast<long long>(r) * p.ldfb + k) : 0.f;
                            }
                        }
#pragma unroll
                        for (int i = 0; i < kGenPos; ++i) {
                            const int off = Cfg::kABytes + (st + Cfg::kSplitThreads * i) * 16;  // chunk position as stored
                            const float4 c4 = *reinterpret_cast<const float4*>(hi + off);
                            const float bv = gen_b[i];
                            float4 h, l;
                            h.x = c4.x * bv; h.y = c4.y * bv; h.z = c4.z * bv; h.w = c4.w * bv;
                            l.x = h.x - __uint_as_float(__float_as_uint(h.x) & 0xFFFFE000u);
                            l.y = h.y - __uint_as_float(__float_as_uint(h.y) & 0xFFFFE000u);
                            l.z = h.z - __uint_as_float(__float_as_uint(h.z) & 0xFFFFE000u);
                            l.w = h.w - __uint_as_float(__float_as_uint(h.w) & 0xFFFFE000u);
                            *reinterpret_cast<float4*>(hi + off) = h;
                            *reinterpret_cast<float4*>(lo_b + off) = l;
                        }
                    }
                    // lo = x - trunc_tf32(x): exact in fp32, at most 13 significant bits. The raw
                    // tiles are left as they are: the tensor core ignores their low 13 mantissa bits.
                    constexpr int kSplitFrom = Cfg::kATmem ? Cfg::kABytes : 0;
                    constexpr int kSplitTo = Cfg::kBGenerated ? Cfg::kABytes : (Cfg::kABytes + Cfg::kBBytes);
                    if constexpr (Cfg::kATmem) {
                        // A goes to tensor memory: this thread owns one tile row (or half of it). The row's
                        // 16-byte chunks sit at
                        // chunk ^ (row & 7) in the swizzled tile, which also spreads a warp's reads over
                        // all banks.
                        const int q = warp & 3;
                        const int row = q * 32 + lane;
                        const uint8_t* rp = hi + row * 128;
                        // with eight split warps two of them share a lane quarter, 16 K values each
#pragma unroll
                        for (int h = (warp - 6) >> 2; h < 2; h += Cfg::kSplitWarps / 4) {
                            uint32_t vh[16], vl[16];
#pragma unroll
                            for (int cc = 0; cc < 4; ++cc) {
                                const float4 v = *reinterpret_cast<const float4*>(rp + (((4 * h + cc) ^ (row & 7)) << 4));
                                vh[4 * cc + 0] = __float_as_uint(v.x); vh[4 * cc + 1] = __float_as_uint(v.y);
                                vh[4 * cc + 2] = __float_as_uint(v.z); vh[4 * cc + 3] = __float_as_uint(v.w);
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                vl[j] = __float_as_uint(__uint_as_float(vh[j]) - __uint_as_float(vh[j] & 0xFFFFE000u));
                            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::kATmemCol0 + ls * 64 + 16 * h;
                            ptx::tmem_st_32x16(taddr, vh);
                            if (!p.single_pass) ptx::tmem_st_32x16(taddr + 32, vl);
                        }
                    }
                    if (!p.single_pass) {
#pragma unroll 4
                        for (int off = kSplitFrom + st * 16; off < kSplitTo; off += Cfg::kSplitThreads * 16) {
                            const float4 v = *reinterpret_cast<const float4*>(hi + off);
                            float4 l;
                            l.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
                            l.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
                            l.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
                            l.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
                            *reinterpret_cast<float4*>((off < Cfg::kABytes ? lo : lo_b) + off) = l;
                        }
                    }
                    if constexpr (Cfg::kATmem) {
                        ptx::tmem_st_wait();
                        ptx::tc_fence_before_sync();
                    }
                    ptx::fence_proxy_async_smem();
                    if (st == 0) T2SP_TRACE(p, 2, it);
                    ptx::mbar_arrive(&ready_bar[ls]);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (warp >= 2 && warp < 6 && lane == 0) ptx::bulk_wait_all();  // this warp's TMA stores are done
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_slot) __nanosleep(200000);  // let stray UMMAs / copies retire before TMEM goes away
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace t2sp
