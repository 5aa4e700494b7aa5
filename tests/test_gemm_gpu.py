"""GEMM parity on the GPU through the C ABI (host buffers in, host buffers out) against the CPU
oracle: known-answer cases with the reference's deterministic fixtures, seeded random cases for
every arithmetic, ragged sizes, and the tiled 6-D output layout of the FPGA drivers."""
import numpy as np
import pytest

from tests import oracle_lib as O
from tests.util import TOL_BF16, TOL_FP32, call_gemm, componentwise, library_env, normwise

pytestmark = pytest.mark.gpu


def test_bf16_known_answer_single_tile(lib):
    # ina(k,i) = k + i, inb(j,k) = j - k pattern of t2s/tests/correctness/aot/gemm-run.cpp:50-59,
    # reduced mod 8 so every product and partial sum is an integer that bf16/fp32 hold exactly.
    M, N, K = 128, 256, 64
    i, k, j = np.arange(M)[:, None], np.arange(K)[None, :], np.arange(N)[None, :]
    A = ((k + i) % 8).astype(np.float32)
    B = ((j - np.arange(K)[:, None]) % 8 - 4).astype(np.float32)
    rc, C = call_gemm(O.to_bf16(A), O.to_bf16(B), "bf16")
    assert rc == 0
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bad = np.argwhere(C != ref)
    assert bad.size == 0, f"{len(bad)} mismatches, first {bad[:5].tolist()} got {C[tuple(bad[0])]} want {ref[tuple(bad[0])]}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (256, 512, 1024), (200, 136, 72), (1024, 1024, 1024)])
def test_bf16_random(lib, M, N, K):
    A = O.to_bf16(O.uniform(0, 1, (M, K)))
    B = O.to_bf16(O.uniform(0, 2, (K, N)))
    rc, C = call_gemm(A, B, "bf16")
    assert rc == 0
    truth = O.gemm_h16(A, B, 0, acc64=True)
    err = normwise(C, truth)
    spec = normwise(O.gemm_h16(A, B, 0), truth)
    print(f"bf16 {M}x{N}x{K}: kernel vs truth {err:.3e}; spec-order oracle vs truth {spec:.3e}")
    assert err <= TOL_BF16
    absprod = O.gemm_f32(np.abs(O.bf16_to_f32(A)), np.abs(O.bf16_to_f32(B)), acc64=True)
    assert componentwise(C, truth, absprod) <= TOL_BF16


def test_f16_random(lib):
    M, N, K = 256, 256, 256
    A = O.uniform(3, 1, (M, K)).astype(np.float16)
    B = O.uniform(3, 2, (K, N)).astype(np.float16)
    rc, C = call_gemm(A, B, "f16")
    assert rc == 0
    truth = O.gemm_h16(A.view(np.uint16), B.view(np.uint16), 1, acc64=True)
    assert normwise(C, truth) <= TOL_BF16


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 1024), (136, 144, 80), (1024, 1024, 2048)])
def test_int8_bit_exact(lib, M, N, K):
    A = O.int8(1, 1, (M, K))
    B = O.int8(1, 2, (K, N))
    rc, C = call_gemm(A, B, "i8", out_dtype=np.int32)
    assert rc == 0
    ref = O.gemm_i8(A, B)
    bad = np.argwhere(C != ref)
    assert bad.size == 0, f"{len(bad)} mismatches, first {bad[:5].tolist()}"


def test_fp32_known_answer(lib):
    # SEQUENTIAL fixture of t2s/tests/correctness/util/util.h:52-65 (value i + j + 1): integers,
    # so the 3xTF32 product must be exact.
    M, N, K = 64, 64, 64
    A = (np.arange(M)[:, None] + np.arange(K)[None, :] + 1).astype(np.float32)
    B = (np.arange(K)[:, None] + np.arange(N)[None, :] + 1).astype(np.float32)
    rc, C = call_gemm(A, B, "f32")
    assert rc == 0
    ref = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
    assert np.array_equal(C, ref)


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (1024, 1024, 1024), (100, 68, 36)])
def test_fp32_random(lib, M, N, K):
    A = O.uniform(2, 1, (M, K))
    B = O.uniform(2, 2, (K, N))
    rc, C = call_gemm(A, B, "f32")
    assert rc == 0
    truth = O.gemm_f32(A, B, acc64=True)
    absprod = O.gemm_f32(np.abs(A), np.abs(B), acc64=True)
    spec_c = O.gemm_f32(A, B)
    err, cw = normwise(C, truth), componentwise(C, truth, absprod)
    print(f"fp32 {M}x{N}x{K}: kernel vs truth normwise {err:.3e} componentwise {cw:.3e}; "
          f"spec-order oracle vs truth {normwise(spec_c, truth):.3e} / {componentwise(spec_c, truth, absprod):.3e}; "
          f"kernel vs spec-order oracle {normwise(C, spec_c):.3e}")
    assert err <= TOL_FP32 and cw <= TOL_FP32
    assert normwise(C, spec_c) <= TOL_FP32


def test_fp32_positive_inputs_strict(lib):
    # The reference drivers fill inputs with non-negative random() values
    # (gemm-run-fpga.cpp:60,65), where the strict elementwise relative error is well behaved.
    M, N, K = 256, 256, 512
    A = np.abs(O.uniform(4, 1, (M, K))) * 1000.0
    B = np.abs(O.uniform(4, 2, (K, N))) * 1000.0
    rc, C = call_gemm(A, B, "f32")
    assert rc == 0
    truth = O.gemm_f32(A, B, acc64=True)
    assert O.rel_err(C, truth, 0.0) <= TOL_FP32


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_tiled_output_layout(lib, dtype):
    # 6-D output c(JJJ,III,JJ,II,J,I) of the FPGA driver (gemm-run-fpga.cpp:69), GPU-variant
    # tile extents (const-parameters.h:24-29) on a 256 x 256 x 128 problem.
    JJJ, III, JJ, II = 8, 16, 2, 4
    M, N, K = III * II * 4, JJJ * JJ * 16, 128
    A = O.uniform(5, 1, (M, K))
    B = O.uniform(5, 2, (K, N))
    if dtype == "bf16":
        Ab, Bb = O.to_bf16(A), O.to_bf16(B)
        rc, C6 = call_gemm(Ab, Bb, "bf16", tiled=(JJJ, III, JJ, II))
        plain = O.gemm_h16(Ab, Bb, 0, acc64=True)
    else:
        rc, C6 = call_gemm(A, B, "f32", tiled=(JJJ, III, JJ, II))
        plain = O.gemm_f32(A, B, acc64=True)
    assert rc == 0
    ref6 = O.gemm_tile_layout(plain, JJJ, III, JJ, II)
    assert not np.isnan(C6).any(), "some tiled output elements were never written"
    assert normwise(C6, ref6) <= (TOL_BF16 if dtype == "bf16" else TOL_FP32)


def test_repeatable_and_deterministic(lib):
    M, N, K = 256, 256, 256
    A = O.to_bf16(O.uniform(6, 1, (M, K)))
    B = O.to_bf16(O.uniform(6, 2, (K, N)))
    rc1, C1 = call_gemm(A, B, "bf16")
    rc2, C2 = call_gemm(A, B, "bf16")
    assert rc1 == 0 and rc2 == 0
    assert np.array_equal(C1, C2)


def test_empty_contraction_and_empty_output(lib):
    A = np.zeros((64, 0), np.float32)
    B = np.zeros((0, 64), np.float32)
    rc, C = call_gemm(A, B, "f32")
    assert rc == 0 and np.array_equal(C, np.zeros((64, 64), np.float32))
    rc, C = call_gemm(np.zeros((0, 32), np.float32), np.zeros((32, 64), np.float32), "f32")
    assert rc == 0 and C.size == 0


@pytest.mark.parametrize("dtype,M,N,K,trans_b", [
    ("bf16", 1024, 1024, 512, 0), ("bf16", 640, 768, 256, 0), ("bf16", 1000, 520, 136, 0), ("bf16", 768, 512, 320, 1),
    ("i8", 1024, 768, 512, 0), ("i8", 520, 1040, 144, 0), ("i8", 512, 512, 256, 1),
])
def test_cta_pair_kernel(lib, dtype, M, N, K, trans_b):
    """Problems of at least 512 x 512 outputs run on CTA pairs (256 x 256 tiles, cta_group::2);
    ragged edges are zero-filled by TMA on the way in and masked on the way out."""
    import t2sp_b200
    from t2sp_b200 import Buffer, GemmDesc
    if dtype == "i8":
        A, B = O.int8(7, 1, (M, K)), O.int8(7, 2, (K, N))
        ref = O.gemm_i8(A, B)
        C = np.full((M, N), -1, np.int32)
    else:
        A, B = O.to_bf16(O.uniform(7, 1, (M, K))), O.to_bf16(O.uniform(7, 2, (K, N)))
        ref = O.gemm_h16(A, B, 0, acc64=True)
        C = np.full((M, N), np.nan, np.float32)
    d = GemmDesc()
    d.trans_b = trans_b
    cb = Buffer.from_numpy(C)
    rc = t2sp_b200.gemm(Buffer.from_numpy(A, dtype=dtype),
                        Buffer.from_numpy(np.ascontiguousarray(B.T) if trans_b else B, dtype=dtype), cb, d)
    assert rc == 0
    if dtype == "i8":
        bad = np.argwhere(cb.keepalive != ref)
        assert bad.size == 0, f"{len(bad)} mismatches, first {bad[:5].tolist()}"
    else:
        assert not np.isnan(cb.keepalive).any()
        assert normwise(cb.keepalive, ref) <= TOL_BF16
        assert normwise(cb.keepalive, ref) <= 1e-5   # bf16 products are exact; only the fp32 summation order differs


@pytest.mark.parametrize("M,N,K,trans_b", [(2048, 2048, 512, 0), (2560, 1300, 200, 0), (4096, 128, 320, 0), (2304, 1024, 256, 1)])
def test_fp32_cta_pair_kernel(lib, M, N, K, trans_b):
    """fp32 problems with enough 256-row tiles run the 3xTF32 kernel on CTA pairs."""
    import t2sp_b200
    from t2sp_b200 import Buffer, GemmDesc
    A, B = O.uniform(8, 1, (M, K)), O.uniform(8, 2, (K, N))
    C = np.full((M, N), np.nan, np.float32)
    cb = Buffer.from_numpy(C)
    d = GemmDesc()
    d.trans_b = trans_b
    rc = t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(np.ascontiguousarray(B.T) if trans_b else B), cb, d)
    assert rc == 0
    assert not np.isnan(cb.keepalive).any()
    truth = O.gemm_f32(A, B, acc64=True)
    err = normwise(cb.keepalive, truth)
    print(f"fp32 pair {M}x{N}x{K}: normwise {err:.3e}")
    assert err <= TOL_FP32
    assert componentwise(cb.keepalive, truth, O.gemm_f32(np.abs(A), np.abs(B), acc64=True)) <= TOL_FP32


@pytest.mark.parametrize("M,N,K,trans_b,force", [(1024, 1024, 1024, 0, None), (1024, 1000, 2048, 1, "3"), (2048, 300, 520, 0, "5")])
def test_fp32_split_k(lib, M, N, K, trans_b, force):
    """fp32 problems with fewer 256-row tiles than SM pairs cut the contraction into ranges (work items of
    their own) and sum the partial tiles in range order in a second kernel; uneven ranges included."""
    import t2sp_b200
    from t2sp_b200 import Buffer, GemmDesc
    A, B = O.uniform(12, 1, (M, K)), O.uniform(12, 2, (K, N))
    d = GemmDesc()
    d.trans_b = trans_b
    Bin = np.ascontiguousarray(B.T) if trans_b else B
    outs = []
    for no_split in (False, True):
        env = {"T2SP_B200_NO_SPLITK": "1"} if no_split else ({"T2SP_B200_SPLITK": force} if force else {})
        with library_env(**env):
            C = np.full((M, N), np.nan, np.float32)
            cb = Buffer.from_numpy(C)
            before = lib.t2sp_b200_kernel_launches()
            assert t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(Bin), cb, d) == 0
            outs.append((cb.keepalive.copy(), lib.t2sp_b200_kernel_launches() - before))
    (split, n_split), (whole, n_whole) = outs
    assert n_split == n_whole + 1, "the split path launches the summing kernel as well"
    truth = O.gemm_f32(A, B, acc64=True)
    assert not np.isnan(split).any()
    assert normwise(split, truth) <= TOL_FP32 and normwise(whole, truth) <= TOL_FP32
    assert componentwise(split, truth, O.gemm_f32(np.abs(A), np.abs(B), acc64=True)) <= TOL_FP32


@pytest.mark.parametrize("M,N,K,trans_b", [(9728, 256, 96, 0), (9728, 264, 200, 0), (9728, 256, 100, 1), (5120, 500, 640, 1),
                                           (9728, 128, 200, 0), (9600, 128, 96, 1)])  # the last two: 256 x 128 tiles
def test_fp32_pair_prepacked_b(lib, M, N, K, trans_b):
    """With many 256-row tiles over one B, the fp32 pair kernel with its A operand in tensor memory runs: a pre-pass
    writes B's shared-memory tile images (raw fp32 and the bf16 operands of the cross-term MMAs) once, the kernel
    fetches them with one bulk copy per k-block and carries the cross terms at bf16 rate. Same tolerance as the
    all-TF32 kernel, which the same call uses when the pre-pass is switched off; one launch more.
    K = 100 / 200 end inside a k-block, N = 264 / 500 inside a tile."""
    import t2sp_b200
    from t2sp_b200 import Buffer, GemmDesc
    A, B = O.uniform(21, 1, (M, K)), O.uniform(21, 2, (K, N))
    d = GemmDesc()
    d.trans_b = trans_b
    Bin = np.ascontiguousarray(B.T) if trans_b else B
    outs = []
    for env in ({"T2SP_B200_NO_SPLITK": "1"}, {"T2SP_B200_NO_SPLITK": "1", "T2SP_B200_NO_PRESPLIT": "1"}):
        with library_env(**env):
            cb = Buffer.from_numpy(np.full((M, N), np.nan, np.float32))
            before = lib.t2sp_b200_kernel_launches()
            assert t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(Bin), cb, d) == 0
            outs.append((cb.keepalive.copy(), lib.t2sp_b200_kernel_launches() - before))
    (pre, n_pre), (plain, n_plain) = outs
    assert n_pre == n_plain + 1, "the pre-pass is a launch of its own"
    truth = O.gemm_f32(A, B, acc64=True)
    absprod = O.gemm_f32(np.abs(A), np.abs(B), acc64=True)
    assert not np.isnan(pre).any()
    for got in (pre, plain):
        assert normwise(got, truth) <= TOL_FP32
        assert componentwise(got, truth, absprod) <= TOL_FP32
    print(f"fp32 pair, pre-packed B {M}x{N}x{K}: componentwise {componentwise(pre, truth, absprod):.3e} "
          f"(all-TF32 kernel {componentwise(plain, truth, absprod):.3e})")


@pytest.mark.parametrize("dist", ["uniform", "positive"])
def test_fp32_bf16_cross_terms_bound_k8192(lib, dist):
    """Known-answer check of the error bound of the bf16 cross terms (a = hi + lo: hi_a hi_b in TF32, bf16(lo_a) bf16(b)
    and bf16(a) bf16(lo_b) in bf16; each product off by at most about 2^-18 |a||b|): a long contraction, K = 8192,
    against the fp64-accumulated oracle, elementwise relative to sum_k |a||b|, on inputs of mixed sign and on the
    positive distribution of the reference's own drivers (where every rounding error has the same sign and nothing
    cancels in the result either). The all-TF32 kernel on the same inputs is printed beside it."""
    import t2sp_b200
    from t2sp_b200 import Buffer
    M, N, K = 4864, 256, 8192
    A, B = O.uniform(31, 1, (M, K)), O.uniform(31, 2, (K, N))
    if dist == "positive":
        A, B = np.abs(A), np.abs(B)
    truth = O.gemm_f32(A, B, acc64=True)
    absprod = O.gemm_f32(np.abs(A), np.abs(B), acc64=True)
    errs = []
    for env in ({}, {"T2SP_B200_NO_PRESPLIT": "1"}):
        with library_env(**env):
            cb = Buffer.from_numpy(np.full((M, N), np.nan, np.float32))
            before = lib.t2sp_b200_kernel_launches()
            assert t2sp_b200.gemm(Buffer.from_numpy(A), Buffer.from_numpy(B), cb) == 0
            launches = lib.t2sp_b200_kernel_launches() - before
            got = cb.keepalive
            assert not np.isnan(got).any()
            errs.append((componentwise(got, truth, absprod), normwise(got, truth), launches))
    (cw, nw, n_pre), (cw_tf32, nw_tf32, n_plain) = errs
    print(f"K=8192 {dist}: bf16 cross terms componentwise {cw:.3e} normwise {nw:.3e}; all TF32 {cw_tf32:.3e} / {nw_tf32:.3e}")
    assert n_pre == n_plain + 1, "the first call ran the pre-pass and the tensor-memory kernel"
    assert cw <= TOL_FP32 and nw <= TOL_FP32
    assert cw_tf32 <= TOL_FP32 and nw_tf32 <= TOL_FP32


def test_fp32_split_k_tiled_layout_and_blas_epilogue(lib):
    """The summing kernel applies the call's own epilogue: the 6-D tiled layout and alpha/beta.
    (Split-K is forced: by itself the library avoids it for tiled layouts, whose summing pass is dear.)"""
    with library_env(T2SP_B200_SPLITK="4"):
        JJJ, III, JJ, II = 8, 16, 2, 4
        M, N, K = III * II * 32, JJJ * JJ * 32, 1024
        A, B = O.uniform(13, 1, (M, K)), O.uniform(13, 2, (K, N))
        rc, C6 = call_gemm(A, B, "f32", tiled=(JJJ, III, JJ, II))
        assert rc == 0
        ref6 = O.gemm_tile_layout(O.gemm_f32(A, B, acc64=True), JJJ, III, JJ, II)
        assert not np.isnan(C6).any()
        assert normwise(C6, ref6) <= TOL_FP32
        m = n = k = 1024
        a, b, c0 = O.uniform(13, 3, (m, k)), O.uniform(13, 4, (k, n)), O.uniform(13, 5, (m, n))
        c = c0.copy()
        assert lib.t2sp_b200_sgemm(b"N", b"N", m, n, k, 1.75, a.ctypes.data, 0, b.ctypes.data, 0, -0.5, c.ctypes.data, 0) == 0
        truth = 1.75 * (a.astype(np.float64) @ b.astype(np.float64)) - 0.5 * c0.astype(np.float64)
        assert normwise(c, truth) <= TOL_FP32


@pytest.mark.parametrize("ta,tb,m,n,k", [("N", "N", 256, 192, 128), ("T", "N", 300, 200, 100), ("N", "T", 128, 260, 64),
                                         ("T", "T", 520, 516, 90), ("N", "N", 2048, 1024, 256),
                                         # many row tiles over one B: the tensor-memory pair kernel, 256- and 128-column tiles
                                         ("N", "N", 9728, 300, 96), ("T", "T", 9728, 128, 70)])
def test_blas_sgemm(lib, ta, tb, m, n, k):
    """BLAS-style entry (reference: t2s/peppers/blas/level3/gemm/release/a10/blas-gemm.cpp): row-major arrays,
    transposes, alpha/beta. transa = 'T' exercises the on-device transpose, including K not a multiple of 4."""
    import ctypes
    a = O.uniform(9, 1, (k, m) if ta == "T" else (m, k))
    b = O.uniform(9, 2, (n, k) if tb == "T" else (k, n))
    c0 = O.uniform(9, 3, (m, n))
    c = c0.copy()
    alpha, beta = 1.75, -0.5
    rc = lib.t2sp_b200_sgemm(ta.encode(), tb.encode(), m, n, k, alpha, a.ctypes.data, 0, b.ctypes.data, 0, beta,
                             c.ctypes.data, 0)
    assert rc == 0
    opa = a.T if ta == "T" else a
    opb = b.T if tb == "T" else b
    truth = alpha * (opa.astype(np.float64) @ opb.astype(np.float64)) + beta * c0.astype(np.float64)
    assert normwise(c, truth) <= TOL_FP32


@pytest.mark.parametrize("dtype,M,N,K", [("bf16", 1024, 512, 4096), ("bf16", 1500, 700, 4104), ("i8", 1024, 768, 8192)])
def test_cta_pair_kernel_512_row_tiles(lib, dtype, M, N, K):
    """Long-K problems (64 or more k-blocks) with M >= 1024 use 512 x 256 pair tiles: two 128-row
    sub-tiles per CTA, both TMEM accumulators in one tile."""
    if dtype == "i8":
        A, B = O.int8(11, 1, (M, K)), O.int8(11, 2, (K, N))
        rc, C = call_gemm(A, B, "i8", out_dtype=np.int32)
        assert rc == 0 and np.array_equal(C, O.gemm_i8(A, B))
    else:
        A, B = O.to_bf16(O.uniform(11, 1, (M, K))), O.to_bf16(O.uniform(11, 2, (K, N)))
        rc, C = call_gemm(A, B, "bf16")
        assert rc == 0 and not np.isnan(C).any()
        assert normwise(C, O.gemm_h16(A, B, 0, acc64=True)) <= 1e-5


def test_large_host_gemm_is_pipelined_and_identical(lib):
    """Host-buffer GEMMs of ~100 MB and more stream their operands in slabs and overlap copies with
    the block computes; the result must be bit-identical to the plain path (same kernel, same
    per-element accumulation order) and right against the oracle on a row slab."""
    import os
    M, N, K = 4096, 4096, 2048
    A, B = O.to_bf16(O.uniform(12, 1, (M, K))), O.to_bf16(O.uniform(12, 2, (K, N)))
    rc, C1 = call_gemm(A, B, "bf16")
    assert rc == 0 and not np.isnan(C1).any()
    with library_env(T2SP_B200_NO_PIPELINE="1"):
        rc, C2 = call_gemm(A, B, "bf16")
    assert rc == 0
    assert np.array_equal(C1, C2)
    rows = slice(1000, 1064)
    assert normwise(C1[rows], O.gemm_h16(np.ascontiguousarray(A[rows]), B, 0, acc64=True)) <= 1e-5


def test_concurrent_host_threads(lib):
    """The library is re-entrant (every host thread works on its own stream, event pair and status word;
    reference: single-shot globals in t2s/src/AOT-OpenCL-Runtime.cpp:25-34): two host threads issue
    different contractions at once."""
    import threading
    import t2sp_b200
    from t2sp_b200 import Buffer
    jobs = [("f32", 384, 320, 520, 41), ("bf16", 512, 768, 1024, 42)]
    errors = []

    def work(dtype, M, N, K, seed):
        try:
            A, B = O.uniform(seed, 1, (M, K)), O.uniform(seed, 2, (K, N))
            if dtype == "bf16":
                A, B = O.to_bf16(A), O.to_bf16(B)
                truth = O.bf16_to_f32(A).astype(np.float64) @ O.bf16_to_f32(B).astype(np.float64)
            else:
                truth = A.astype(np.float64) @ B.astype(np.float64)
            for _ in range(8):
                rc, C = call_gemm(A, B, dtype)
                if rc != 0 or normwise(C, truth) > (TOL_BF16 if dtype == "bf16" else TOL_FP32):
                    errors.append((dtype, rc, normwise(C, truth)))
        except Exception as e:  # surfaced by the assertion below
            errors.append((dtype, repr(e)))

    threads = [threading.Thread(target=work, args=j) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_sgemm_padded_output_keeps_its_padding(lib):
    """ldc > n with beta == 0: only the m x n region of the host array may change; the elements between
    the rows belong to the caller (they are NaN here and must stay NaN)."""
    m, n, k, ldc = 300, 200, 96, 232
    a, b = O.uniform(21, 1, (m, k)), O.uniform(21, 2, (k, n))
    c = np.full((m, ldc), np.nan, np.float32)
    assert lib.t2sp_b200_sgemm(b"N", b"N", m, n, k, 1.0, a.ctypes.data, 0, b.ctypes.data, 0, 0.0, c.ctypes.data, ldc) == 0
    assert np.isnan(c[:, n:]).all()
    assert not np.isnan(c[:, :n]).any()
    assert normwise(c[:, :n], a.astype(np.float64) @ b.astype(np.float64)) <= TOL_FP32


def test_host_column_slab_output_leaves_other_columns_alone(lib):
    """C given as a column slab of a wider host matrix (row pitch = the full width), as a column-sharded
    caller passes it: the other slabs' columns must not be touched."""
    import t2sp_b200
    from t2sp_b200 import Buffer
    M, K, NT, c0, cols = 256, 128, 640, 256, 128
    A, B = O.to_bf16(O.uniform(22, 1, (M, K))), O.to_bf16(O.uniform(22, 2, (K, NT)))
    C = np.full((M, NT), np.nan, np.float32)
    a = Buffer.from_numpy(A, dtype="bf16")
    b = Buffer((cols, K), "bf16", host=B.ctypes.data + 2 * c0, strides=(1, NT), keepalive=B)
    c = Buffer((cols, M), "f32", host=C.ctypes.data + 4 * c0, strides=(1, NT), keepalive=C)
    assert t2sp_b200.gemm(a, b, c) == 0
    assert np.isnan(C[:, :c0]).all() and np.isnan(C[:, c0 + cols:]).all()
    ref = O.gemm_h16(A, np.ascontiguousarray(B[:, c0:c0 + cols]), 0, acc64=True)
    assert normwise(C[:, c0:c0 + cols], ref) <= 1e-5


def test_empty_contraction_zeroes_only_the_region(lib):
    """K == 0: C becomes zero inside its extents; a device-resident C with padded rows keeps its padding."""
    import torch
    import t2sp_b200
    from t2sp_b200 import Buffer
    M, N, ld = 64, 48, 80
    t = torch.full((M, ld), float("nan"), dtype=torch.float32, device="cuda")
    a = Buffer((0, M), "f32", host=None)
    b = Buffer((N, 0), "f32", host=None)
    c = Buffer((N, M), "f32", strides=(1, ld))
    za = torch.zeros(16, device="cuda")
    for x, ptr in ((a, za.data_ptr()), (b, za.data_ptr()), (c, t.data_ptr())):
        assert t2sp_b200.wrap_device(x, ptr) == 0
    torch.cuda.synchronize()
    assert t2sp_b200.gemm(a, b, c) == 0
    assert lib.t2sp_b200_sync() == 0
    out = t.cpu().numpy()
    assert np.all(out[:, :N] == 0) and np.isnan(out[:, N:]).all()


def test_two_threads_on_their_own_streams(lib):
    """Each host thread has its own stream, timing events and status word, and cached device blocks are
    ordered by events when they change streams: two threads, one on a stream it set itself and one on
    the library's per-thread stream, run host-buffer calls of different sizes at once (scratch, staging
    and split-K blocks keep moving between the two streams through the cache)."""
    import threading
    import torch
    import t2sp_b200
    errors = []

    def work(seed, own_stream, shapes):
        try:
            lib.t2sp_b200_set_device(0)
            stream = torch.cuda.Stream() if own_stream else None
            if stream is not None:
                lib.t2sp_b200_set_stream(ctypes.c_void_p(stream.cuda_stream))
            for it in range(6):
                M, N, K = shapes[it % len(shapes)]
                A, B = O.uniform(seed + it, 1, (M, K)), O.uniform(seed + it, 2, (K, N))
                rc, C = call_gemm(A, B, "f32")
                err = normwise(C, A.astype(np.float64) @ B.astype(np.float64)) if rc == 0 else None
                if rc != 0 or err > TOL_FP32:
                    errors.append((seed, it, rc, err))
            if stream is not None:
                lib.t2sp_b200_set_stream(None)
        except Exception as e:  # surfaced by the assertion below
            errors.append((seed, repr(e)))

    import ctypes
    shapes_a = [(1024, 1024, 1024), (384, 320, 520), (512, 512, 2048)]
    shapes_b = [(512, 512, 2048), (1024, 1024, 1024), (200, 136, 72)]
    threads = [threading.Thread(target=work, args=(50, True, shapes_a)), threading.Thread(target=work, args=(60, False, shapes_b))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_bounded_wait_runs_out_and_the_library_stays_usable(lib):
    """A wait inside a kernel that can never be satisfied ends by itself: the producer of a small
    single-tile GEMM leaves out one k-block's copies (a test hook), the tensor-core warp's wait on that
    stage runs out after the shortened limit, every role leaves its loop, the CTA frees its tensor memory
    and returns, and the host reports halide_error_code_device_run_failed. The next call works."""
    A = O.to_bf16(O.uniform(23, 1, (128, 512)))
    B = O.to_bf16(O.uniform(23, 2, (512, 128)))
    with library_env(T2SP_B200_WAIT_CYCLES="20000000", T2SP_B200_TEST_SKIP_STAGE="3"):
        rc, _ = call_gemm(A, B, "bf16")
    assert rc == -23
    rc, C = call_gemm(A, B, "bf16")
    assert rc == 0
    assert normwise(C, O.gemm_h16(A, B, 0, acc64=True)) <= 1e-5
