// MTTKRP in the reference's own association (t2s/tests/correctness/util/util.h:470-477):
//   d(i,r) = sum_k ( sum_l a(l,i,k) c(l,r) ) b(k,r)
// The inner sum over l is a GEMM whose B operand is the factor c alone: E_k[i,r] = A_k[i,l] C[l,r],
// the same C for every k. So a CTA keeps its slice of c resident in shared memory, already split for
// the tensor cores, streams the tensor a through a TMA ring exactly once, accumulates E_k in tensor
// memory, and applies b(k,r) when E_k is drained: d += E_k * b(k,:) in fp32 registers. Neither the
// Khatri-Rao product nor E ever exists in global memory, and nothing but the 16 KB tiles of a moves
// per k-block.
//
// Work item = (128-row tile of i) x (range of up to 4 l-blocks of 32) x (range of up to 64 k); the items
// fill the SMs; every item writes a partial slab [item slab][r][i] and a second kernel adds the slabs
// in order (deterministic).
//
// fp32 accuracy from TF32/BF16 tensor-core passes, per product a*c:
//   a_hi * c_hi   kind::tf32 on the raw fp32 words (the tensor core reads the top 19 bits: truncation)
//   a_lo * c'     kind::f16, a_lo = bf16(a - trunc_tf32(a)), c' = bf16(c)
//   a'   * c_lo   kind::f16, a' = bf16(a), c_lo = bf16(c - trunc_tf32(c))
// |lo| <= 2^-10 |x| and a bf16 rounding is 2^-9 relative, so each cross term is off by at most
// 2^-19 |a||c|; the neglected a_lo c_lo is below 2^-20 |a||c|. All three accumulate in one fp32
// accumulator that lives for one k only (at most 4 l-blocks = 32 accumulate steps, so the tensor core's
// truncating adds stay far below the 1e-5 tolerance); the sum over k runs in fp32 registers, rounded
// to nearest.
//
// The A operand of all MMAs is in tensor memory: split warps read each raw tile of a once and write hi
// (fp32), bf16(a) and bf16(lo) into one of four 64-column A slots with tcgen05.st; two groups of four
// warps take the k-blocks in turn.
// Every mbarrier wait is bounded as in the other kernels.
#pragma once
#include <cuda_bf16.h>

#include "umma_core.cuh"

namespace t2sp {

struct Mttkrp2Cfg {
    static constexpr int kBN = 64;
    static constexpr int kStages = 8;
    static constexpr int kABytes = kBlockM * 128;                 // one raw tile of a: 128 rows x 32 l
    static constexpr int kMaxLb = 4;                              // l-blocks of c resident per item
    static constexpr int kMaxK = 64;                              // k values of b staged per item
    static constexpr int kCTile = kBN * 128;                      // one fp32 tile of c (64 r x 32 l), or one bf16 tile (64 r x 64 l)
    static constexpr int kCF32Bytes = kMaxLb * kCTile;
    static constexpr int kCB16Bytes = (kMaxLb / 2) * kCTile;
    static constexpr int kBvalBytes = kMaxK * kBN * 4;
    static constexpr int kSplitWarps = 8;
    static constexpr int kSplitThreads = kSplitWarps * 32;
    static constexpr int kWarps = 2 + 4 + kSplitWarps + 1;        // producer, issuer 0, 4 drain, split, issuer 1
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kAccBufs = 4, kASlots = 4;               // accumulators: [pipeline][2]; A slots: even ones pipeline 0, odd ones pipeline 1
    static constexpr int kATmemCol0 = kAccBufs * kBN;             // A slots behind the accumulators
    static constexpr int kTmemCols = 512;
    static constexpr int kNumBars = 2 * kStages + 2 * kASlots + 2 * kAccBufs + 5;
    static_assert(kStages % 2 == 0 && kASlots % 2 == 0, "the two split groups own the even and the odd stages / A slots");
    static constexpr int kSmemBytes = kStages * kABytes + kCF32Bytes + 2 * kCB16Bytes + kBvalBytes + kNumBars * 8 + 16 + 1024;
    static_assert(kAccBufs * kBN + kASlots * 64 <= kTmemCols, "accumulators and A slots must fit tensor memory");
    static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);  // .x (low half) = first argument
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float tf32_lo(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

__global__ void __launch_bounds__(Mttkrp2Cfg::kThreads, 1) umma_mttkrp2_kernel(const __grid_constant__ CoreParams p) {
    using Cfg = Mttkrp2Cfg;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* c_f32 = smem + S * Cfg::kABytes;            // raw fp32 tiles of c: the hi operand of the tf32 MMAs
    uint8_t* c_hb = c_f32 + Cfg::kCF32Bytes;             // bf16(c), two l-blocks per 128-byte row
    uint8_t* c_lb = c_hb + Cfg::kCB16Bytes;              // bf16(c - trunc_tf32(c))
    float* bvals = reinterpret_cast<float*>(c_lb + Cfg::kCB16Bytes);  // b(k0 + kk, r) at [kk * 64 + r]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(bvals) + Cfg::kBvalBytes);
    uint64_t* empty_bar = full_bar + S;                  // raw tile read by all split warps
    uint64_t* ready_bar = empty_bar + S;                 // A slot written
    uint64_t* afree_bar = ready_bar + Cfg::kASlots;      // MMAs that read the A slot retired
    uint64_t* tfull_bar = afree_bar + Cfg::kASlots;      // E_k complete
    uint64_t* tempty_bar = tfull_bar + Cfg::kAccBufs;    // E_k drained
    uint64_t* cfull_bar = tempty_bar + Cfg::kAccBufs;    // the item's tiles of c landed
    uint64_t* cfree_bar = cfull_bar + 1;                 // the item's MMAs retired: c may be replaced
    uint64_t* bready_bar = cfree_bar + 1;                // the item's values of b are staged (one arrival per drain warp)
    uint64_t* bdone_bar = bready_bar + 1;                // every drain warp is done with them
    uint64_t* cconv_bar = bdone_bar + 1;                 // every split warp has converted its share of c
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cconv_bar + 1);
    uint32_t* abort_slot = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const AbortCtx ab{abort_slot, p.status, p.wait_cycles > 0 ? p.wait_cycles : kWaitTimeoutCycles};
    const int slabs = p.mt_lranges * p.mt_kranges;
    const int num_items = p.tiles_m * slabs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], Cfg::kSplitWarps / 2);
        }
        for (int a = 0; a < Cfg::kASlots; ++a) {
            ptx::mbar_init(&ready_bar[a], Cfg::kSplitWarps / 2);
            ptx::mbar_init(&afree_bar[a], 1);
        }
        for (int a = 0; a < Cfg::kAccBufs; ++a) {
            ptx::mbar_init(&tfull_bar[a], 1);
            ptx::mbar_init(&tempty_bar[a], 4);
        }
        ptx::mbar_init(cfull_bar, 1);
        ptx::mbar_init(cfree_bar, 2);
        ptx::mbar_init(bready_bar, 4);
        ptx::mbar_init(bdone_bar, 4);
        ptx::mbar_init(cconv_bar, Cfg::kSplitWarps);
        *abort_slot = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before_sync();
    ptx::grid_dep_launch();  // the kernel that sums the partial slabs may be scheduled while this grid runs
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // item t -> row tile mb, l-blocks [lb0, lb0 + lb_cnt), k values [k0, k0 + k_cnt), partial slab `slab`
    auto decode = [&](int t, int& mb, int& slab, int& lb0, int& lb_cnt, int& k0, int& k_cnt) {
        mb = t % p.tiles_m;
        slab = t / p.tiles_m;
        const int lr = slab % p.mt_lranges, kr = slab / p.mt_lranges;
        lb0 = lr * p.mt_lb_per;
        lb_cnt = min(p.mt_lb_per, p.lblks - lb0);
        k0 = kr * p.mt_k_per;
        k_cnt = min(p.mt_k_per, p.Kdim - k0);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&p.mapA[0]);
            ptx::prefetch_tensormap(&p.mapB);
            int it = 0, n = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x, ++n) {
                int mb, slab, lb0, lb_cnt, k0, k_cnt;
                decode(t, mb, slab, lb0, lb_cnt, k0, k_cnt);
                if (n > 0 && !bounded_wait(cfree_bar, (n - 1) & 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                ptx::mbar_expect_tx(cfull_bar, lb_cnt * Cfg::kCTile);
                for (int j = 0; j < lb_cnt; ++j)
                    ptx::tma_load_2d(c_f32 + j * Cfg::kCTile, &p.mapB, cfull_bar, (lb0 + j) * 32, 0);
                for (int kc = 0; kc < k_cnt && ok; ++kc)
                    for (int j = 0; j < lb_cnt; ++j, ++it) {
                        const int s = it % S;
                        if (!bounded_wait(&empty_bar[s], ((it / S) & 1) ^ 1, ab, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                        T2SP_TRACE(p, 0, it);
                        ptx::mbar_expect_tx(&full_bar[s], Cfg::kABytes);
                        ptx::tma_load_3d(smem + s * Cfg::kABytes, &p.mapA[0], &full_bar[s], (lb0 + j) * 32, mb * kBlockM, k0 + kc);
                    }
            }
            if (!ok) {
                // Give copies already in flight a bounded chance to land before the CTA exits.
                for (int s = 0; s < S; ++s) {
                    const int last = it - 1 - ((it - 1 - s) % S + S) % S;
                    if (last >= 0)
                        for (int spin = 0; spin < 4000; ++spin)
                            if (ptx::mbar_try_wait(&full_bar[s], (last / S) & 1)) break;
                }
                for (int spin = 0; spin < 4000 && n > 0; ++spin)
                    if (ptx::mbar_try_wait(cfull_bar, (n - 1) & 1)) break;
            }
        }
    } else if (warp == 1 || warp == 6 + Cfg::kSplitWarps) {
        // ------------------------------------------------------------ MMA issuers (whole warp, one elected lane per instruction)
        // Two independent pipelines: the k-blocks with an even position in the stream of copies go from split group 0
        // through A slots 0 and 2 to issuer 0 (warp 1), the odd ones from group 1 through slots 1 and 3 to issuer 1,
        // and each pipeline sums its k-blocks of a k into accumulators of its own, which the drain warps add. An
        // issuing warp is held up for as long as its MMAs take to execute (about 53 cycles each at N = 64) and needs
        // about 630 cycles more per k-block for the barrier round (measured: 330 until the `ready` wait has returned,
        // 50 fence, 60 commit, 190 loop) plus 650 at every k: one issuer went round in 1170 cycles per k-block with the
        // tensor pipe busy a third of the time.
        const int pipe = warp == 1 ? 0 : 1;
        const uint32_t idesc32 = make_instr_desc(1, 2, false, false, kBlockM, Cfg::kBN);
        const uint32_t idesc16 = make_instr_desc(1, 1, false, false, kBlockM, Cfg::kBN);
        int it = 0, kcount = 0;  // kcount: the k values this pipeline has had a k-block of
        bool ok = true;
        for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
            int mb, slab, lb0, lb_cnt, k0, k_cnt;
            decode(t, mb, slab, lb0, lb_cnt, k0, k_cnt);
            for (int kc = 0; kc < k_cnt && ok; ++kc, it += lb_cnt) {
                const int first = it + ((it & 1) != pipe ? 1 : 0);  // this pipeline's first k-block of the k
                if (first >= it + lb_cnt) continue;
                const int acc = pipe * 2 + (kcount & 1);
                if (!bounded_wait_warp(&tempty_bar[acc], ((kcount >> 1) & 1) ^ 1, ab, ST_TIMEOUT_MMA, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kBN;
                for (int i = first; i < it + lb_cnt; i += 2) {
                    const int j = i - it, ls = i % Cfg::kASlots;
                    // the split warps arrive here after they have seen the tile land and (first k-block of an
                    // item) after they have converted c, so this wait covers both
                    if (!bounded_wait_warp(&ready_bar[ls], (i / Cfg::kASlots) & 1, ab, ST_TIMEOUT_MMA, lane)) { ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (lane == 0) T2SP_TRACE(p, 3, i);
                    const uint32_t a_hi = tmem_base + Cfg::kATmemCol0 + ls * 64, a_hb = a_hi + 32, a_lb = a_hi + 48;
                    const uint64_t db = ptx::make_smem_desc(ptx::smem_u32(c_f32 + j * Cfg::kCTile), 16, 1024);
                    const uint32_t off16 = (j >> 1) * Cfg::kCTile + (j & 1) * 64;
                    const uint64_t dhb = ptx::make_smem_desc(ptx::smem_u32(c_hb + off16), 16, 1024);
                    const uint64_t dlb = ptx::make_smem_desc(ptx::smem_u32(c_lb + off16), 16, 1024);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        ptx::umma_tf32_a_tmem_warp(d_tmem, a_hi + 8 * jj, db + jj * 2, idesc32, (i != first || jj) ? 1u : 0u);
                    if (!p.single_pass) {
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {
                            ptx::umma_f16_a_tmem_warp(d_tmem, a_lb + 8 * jj, dhb + jj * 2, idesc16, 1u);
                            ptx::umma_f16_a_tmem_warp(d_tmem, a_hb + 8 * jj, dlb + jj * 2, idesc16, 1u);
                        }
                    }
                    ptx::umma_commit_warp(&afree_bar[ls]);
                    if (lane == 0) T2SP_TRACE(p, 4, i);
                }
                if (ok) ptx::umma_commit_warp(&tfull_bar[acc]);
                ++kcount;
            }
            if (ok) ptx::umma_commit_warp(cfree_bar);  // tracks this warp's own MMAs: both issuers report
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ drain: d += E_k * b(k, :), then the partial slab
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        const int et = (warp - 2) * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        int g = 0, n = 0, it = 0;
        int kcount[2] = {0, 0};  // per pipeline: the k values it has had a k-block of (as the issuers count them)
        bool ok = true;
        for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x, ++n) {
            int mb, slab, lb0, lb_cnt, k0, k_cnt;
            decode(t, mb, slab, lb0, lb_cnt, k0, k_cnt);
            // (bounded mbarrier waits rather than bar.sync, so that a warp that gave up cannot strand the others)
            if (n > 0 && !bounded_wait_warp(bdone_bar, (n - 1) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
            for (int idx = et; idx < k_cnt * Cfg::kBN; idx += 128) {
                const int kk = idx >> 6, r = idx & 63;
                bvals[idx] = r < p.R ? __ldg(p.fb + static_cast<long long>(r) * p.ldfb + (k0 + kk)) : 0.f;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bready_bar);
            if (!bounded_wait_warp(bready_bar, n & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
            float d[Cfg::kBN];
            for (int kc = 0; kc < k_cnt; ++kc, ++g, it += lb_cnt) {
                // E_k is the sum of what the two pipelines accumulated; a pipeline has part in this k if one of the
                // k's k-blocks has its parity in the stream of copies (both whenever the k has two or more k-blocks)
                int acc[2];
                bool part[2];
#pragma unroll
                for (int pp = 0; pp < 2; ++pp) {
                    part[pp] = it + ((it & 1) != pp ? 1 : 0) < it + lb_cnt;
                    acc[pp] = pp * 2 + (kcount[pp] & 1);
                    if (part[pp]) {
                        if (!bounded_wait_warp(&tfull_bar[acc[pp]], (kcount[pp] >> 1) & 1, ab, ST_TIMEOUT_EPILOGUE, lane)) { ok = false; break; }
                    }
                }
                if (!ok) break;
                ptx::tc_fence_after_sync();
                if (et == 0) T2SP_TRACE(p, 5, g);
#pragma unroll
                for (int qt = 0; qt < 4; ++qt) {  // 16 columns at a time: two accumulators' worth of registers stay few
                    uint32_t e[16];
                    ptx::tmem_ld_32x16(lane_base + acc[part[0] ? 0 : 1] * Cfg::kBN + qt * 16, e);
                    if (part[0] && part[1]) {
                        uint32_t e2[16];
                        ptx::tmem_ld_32x16(lane_base + acc[1] * Cfg::kBN + qt * 16, e2);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int z = 0; z < 16; ++z) e[z] = __float_as_uint(__uint_as_float(e[z]) + __uint_as_float(e2[z]));
                    } else {
                        ptx::tmem_ld_wait();
                    }
                    const float4* bv = reinterpret_cast<const float4*>(bvals + kc * Cfg::kBN + qt * 16);
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        const float4 b4 = bv[j4];  // the same address in every lane: a broadcast read
                        float* dd = &d[qt * 16 + 4 * j4];
                        if (kc == 0) {
                            dd[0] = __uint_as_float(e[4 * j4 + 0]) * b4.x; dd[1] = __uint_as_float(e[4 * j4 + 1]) * b4.y;
                            dd[2] = __uint_as_float(e[4 * j4 + 2]) * b4.z; dd[3] = __uint_as_float(e[4 * j4 + 3]) * b4.w;
                        } else {
                            dd[0] = fmaf(__uint_as_float(e[4 * j4 + 0]), b4.x, dd[0]); dd[1] = fmaf(__uint_as_float(e[4 * j4 + 1]), b4.y, dd[1]);
                            dd[2] = fmaf(__uint_as_float(e[4 * j4 + 2]), b4.z, dd[2]); dd[3] = fmaf(__uint_as_float(e[4 * j4 + 3]), b4.w, dd[3]);
                        }
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
#pragma unroll
                for (int pp = 0; pp < 2; ++pp)
                    if (part[pp]) {
                        if (lane == 0) ptx::mbar_arrive(&tempty_bar[acc[pp]]);
                        ++kcount[pp];
                    }
                if (et == 0) T2SP_TRACE(p, 6, g);
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bdone_bar);
            const int m = mb * kBlockM + q * 32 + lane;
            if (m < p.M) {
                float* out = static_cast<float*>(p.out) + static_cast<long long>(slab) * p.M * p.N + m;
#pragma unroll
                for (int j = 0; j < Cfg::kBN; ++j)
                    if (j < p.N) out[static_cast<long long>(j) * p.M] = d[j];
            }
        }
    } else {
        // ------------------------------------------------------------ split warps: c once per item, then every tile of a into tensor memory
        // Two groups of four warps (one warp per TMEM lane quarter) take the k-blocks in turn, so two tiles are
        // being converted at any time: one warp's chain of waits, shared-memory loads, conversions and TMEM stores
        // for a k-block is longer than the k-block period the memory system allows.
        const int sw = warp - 6;
        const int st = sw * 32 + lane;
        const int q = warp & 3;    // TMEM lane quarter this warp may write
        const int grp = sw >> 2;   // this warp's group takes the k-blocks with (it & 1) == grp
        const int row = q * 32 + lane;
        int it = 0, n = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x, ++n) {
            int mb, slab, lb0, lb_cnt, k0, k_cnt;
            decode(t, mb, slab, lb0, lb_cnt, k0, k_cnt);
            if (!bounded_wait_warp(cfull_bar, n & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
            if (!p.single_pass) {
                // c(l-block j, r) as TMA delivered it: row r of tile j, 16-byte chunk c stored at c ^ (r & 7).
                // The bf16 tiles hold two l-blocks per 128-byte row (l-block j in the half (j & 1)), same swizzle.
                for (int qi = st; qi < lb_cnt * 512; qi += Cfg::kSplitThreads) {
                    const int j = qi >> 9, r = (qi & 511) >> 3, cs = qi & 7, c = cs ^ (r & 7);
                    const float4 v = *reinterpret_cast<const float4*>(c_f32 + j * Cfg::kCTile + r * 128 + cs * 16);
                    const int c16 = (j & 1) * 4 + (c >> 1);
                    const int off = (j >> 1) * Cfg::kCTile + r * 128 + ((c16 ^ (r & 7)) << 4) + (c & 1) * 8;
                    *reinterpret_cast<uint2*>(c_hb + off) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                    *reinterpret_cast<uint2*>(c_lb + off) =
                        make_uint2(pack_bf16(tf32_lo(v.x), tf32_lo(v.y)), pack_bf16(tf32_lo(v.z), tf32_lo(v.w)));
                }
                ptx::fence_proxy_async_smem();
            }
            // every split warp has converted its share before any of them reports a tile of a as ready
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(cconv_bar);
            if (!bounded_wait_warp(cconv_bar, n & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
            const int total = k_cnt * lb_cnt;
            const int it_end = it + total;
            for (int i = it + ((it & 1) != grp ? 1 : 0); i < it_end; i += 2) {
                const int s = i % S, ls = i % Cfg::kASlots;
                if (sw == 0 || sw == 4) T2SP_TRACE(p, 20 + grp, i >> 1);
                if (!bounded_wait_warp(&full_bar[s], (i / S) & 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                if (st == 0) T2SP_TRACE(p, 1, i >> 1);
                // This thread's tile row: 16-byte chunk c sits at c ^ (row & 7), which also spreads a warp's reads
                // over all banks. The row is converted in registers and the stage handed back to the producer
                // BEFORE the wait for a free A slot: at full memory bandwidth a copy takes about as long as eight
                // k-blocks, so every stage has to be back in flight as soon as its data has been read.
                const uint8_t* rp = smem + s * Cfg::kABytes + row * 128;
                uint32_t vh[32], vb[16], vl[16];
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const float4 v = *reinterpret_cast<const float4*>(rp + ((cc ^ (row & 7)) << 4));
                    vh[4 * cc + 0] = __float_as_uint(v.x); vh[4 * cc + 1] = __float_as_uint(v.y);
                    vh[4 * cc + 2] = __float_as_uint(v.z); vh[4 * cc + 3] = __float_as_uint(v.w);
                    vb[2 * cc + 0] = pack_bf16(v.x, v.y); vb[2 * cc + 1] = pack_bf16(v.z, v.w);
                    vl[2 * cc + 0] = pack_bf16(tf32_lo(v.x), tf32_lo(v.y)); vl[2 * cc + 1] = pack_bf16(tf32_lo(v.z), tf32_lo(v.w));
                }
                // the conversions above consumed every loaded value, so the loads have completed
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty_bar[s]);
                if (st == 0) T2SP_TRACE(p, 7, i >> 1);
                if (!bounded_wait_warp(&afree_bar[ls], ((i / Cfg::kASlots) & 1) ^ 1, ab, ST_TIMEOUT_SPLITTER, lane)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::kATmemCol0 + ls * 64;
                ptx::tmem_st_32x32(taddr, vh);
                if (!p.single_pass) {
                    ptx::tmem_st_32x16(taddr + 32, vb);
                    ptx::tmem_st_32x16(taddr + 48, vl);
                }
                if (st == 0) T2SP_TRACE(p, 9, i >> 1);
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ready_bar[ls]);
                if (lane == 0) T2SP_TRACE(p, 10 + sw, i >> 1);
            }
            it = it_end;
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_slot) __nanosleep(200000);  // let stray UMMAs / copies retire before TMEM goes away
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace t2sp
