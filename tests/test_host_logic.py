"""Host-side behaviour of the C ABI that needs no GPU: argument validation in the reference's
order with the reference's error codes (HalideRuntime.h:957-1143), bounds queries, and the
loud failure when no CUDA device exists (there is no CPU path)."""
import ctypes

import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer, CapsuleDesc, ConvDesc, GemmDesc

F = np.float32


def bufs(M=64, N=64, K=64, dtype=F):
    return (Buffer.from_numpy(np.ones((M, K), dtype)), Buffer.from_numpy(np.ones((K, N), dtype)),
            Buffer.from_numpy(np.zeros((M, N), F)))


def test_null_arguments(lib):
    A, B, C = bufs()
    assert lib.t2sp_b200_gemm(A.ptr, B.ptr, None, None) == -12
    assert lib.t2sp_b200_gemm(None, B.ptr, C.ptr, None) == -12
    assert lib.t2sp_b200_ttm(None, None, None, None) == -12
    assert lib.t2sp_b200_mttkrp(A.ptr, B.ptr, C.ptr, None, None) == -12


def test_bad_type_and_dimensions(lib):
    A, B, C = bufs(dtype=np.float64)
    assert t2sp_b200.gemm(A, B, C) == -3
    A, B, C = bufs()
    A3 = Buffer.from_numpy(np.ones((4, 64, 64), F))
    assert t2sp_b200.gemm(A3, B, C) == -43
    Ci = Buffer.from_numpy(np.zeros((64, 64), np.int32))
    assert t2sp_b200.gemm(A, B, Ci) == -3                       # fp32 inputs need an fp32 output
    Ai, Bi, _ = bufs(dtype=np.int8)
    assert t2sp_b200.gemm(Ai, Bi, C) == -3                      # int8 inputs need an int32 output
    assert t2sp_b200.gemm(Ai, B, Ci) == -3                      # A and B must share a type


def test_extents_constraints_and_coverage(lib):
    A, B, C = bufs()
    A.dims[1].extent = -1
    assert t2sp_b200.gemm(A, B, C) == -28
    A, B, C = bufs(K=64)
    B2 = Buffer.from_numpy(np.ones((32, 64), F))                # K mismatch
    assert t2sp_b200.gemm(A, B2, C) == -8
    small = Buffer.from_numpy(np.zeros((32, 64), F))            # output does not cover M
    assert t2sp_b200.gemm(A, B, small) == -4
    C.dims[0].min = 1                                           # output starts after column 0
    assert t2sp_b200.gemm(A, B, C) == -4
    A, B, C = bufs()
    A.dims[0].stride = 2
    assert t2sp_b200.gemm(A, B, C) == -8                        # stride.0 must be 1
    A, B, C = bufs()
    A.raw.host = None
    B.raw.host = None                                           # A and B are both bounds queries now
    assert t2sp_b200.gemm(A, B, C) == 0
    A, B, C = bufs()
    B.raw.host = None
    B.raw.device = 1234                                         # a device handle of someone else, no host
    assert t2sp_b200.gemm(A, B, C) == -34


def test_tiled_gemm_output_validation(lib):
    A = Buffer.from_numpy(np.ones((64, 32), F))
    B = Buffer.from_numpy(np.ones((32, 64), F))
    C6 = Buffer.from_numpy(np.zeros((4, 4, 4, 4, 4, 4), F))     # JJJ=III=JJ=II=4, J=I=4
    d = GemmDesc()
    d.layout = 1
    assert t2sp_b200.gemm(A, B, C6, d) == -36                    # valid arguments: only the device is missing here
    d.JJJ = 5                                                    # 64 columns are not a multiple of JJJ*JJ
    assert t2sp_b200.gemm(A, B, C6, d) == -8
    Cbad = Buffer.from_numpy(np.zeros((4, 4, 4, 4, 4, 2), F))   # I extent too small
    assert t2sp_b200.gemm(A, B, Cbad) == -4


def test_bounds_query_fills_shapes(lib):
    A, B, _ = bufs(M=48, N=80, K=32)
    q = Buffer.query(2)
    assert t2sp_b200.gemm(A, B, q) == 0
    assert q.shape() == [(0, 80, 1), (0, 48, 80)]
    a = Buffer.from_numpy(np.ones((6, 5, 16), F))
    b = Buffer.from_numpy(np.ones((7, 16), F))
    q3 = Buffer.query(3)
    assert t2sp_b200.ttm(a, b, q3) == 0
    assert [e for _, e, _ in q3.shape()] == [5, 6, 7]
    d = ConvDesc()
    d.CI, d.CO, d.KY, d.KX, d.OY, d.OX = 16, 32, 3, 3, 4, 4
    I2 = Buffer.from_numpy(np.ones((36, 16 * 2), F))
    qk, qo = Buffer.query(2), Buffer.query(2)
    assert t2sp_b200.conv(I2, qk, qo, d) == 0
    assert [e for _, e, _ in qk.shape()] == [32 * 3, 16 * 3]
    assert [e for _, e, _ in qo.shape()] == [32 * 2, 16]


def test_conv_and_capsule_descriptor_checks(lib):
    I2 = Buffer.from_numpy(np.ones((36, 32), F))
    K2 = Buffer.from_numpy(np.ones((48, 96), F))
    O2 = Buffer.from_numpy(np.zeros((16, 64), F))
    assert t2sp_b200.lib().t2sp_b200_conv(I2.ptr, K2.ptr, O2.ptr, None) == -1      # descriptor is mandatory
    d = ConvDesc()
    d.CI, d.CO, d.KY, d.KX, d.OY, d.OX = 16, 32, 3, 3, 4, 4
    assert t2sp_b200.conv(I2, K2, O2, d) == -36                                    # consistent: reaches the device step
    d.OY = 5                                                                      # input plane no longer IY*IX
    assert t2sp_b200.conv(I2, K2, O2, d) == -8
    c = CapsuleDesc()
    c.CI, c.CII, c.CO, c.KY, c.KX, c.OY, c.OX = 16, 4, 16, 3, 3, 7, 7
    c.MY = c.MX = c.MK = 4
    c.NN, c.stride = 1, 3
    P = Buffer.from_numpy(np.ones((15 * 15 * 2, 16 * 16), F))
    W = Buffer.from_numpy(np.ones((16 * 9 * 4, 64), F))
    V = Buffer.from_numpy(np.zeros((49 * 2, 16 * 16), F))
    assert t2sp_b200.capsule(P, W, V, c) == -8                                     # stride must be 1 or 2
    c.stride = 2
    assert t2sp_b200.capsule(P, W, V, c) == -36


def test_mttkrp_validation(lib):
    a = Buffer.from_numpy(np.ones((8, 16, 32), F))      # (L=32, I=16, K=8)
    b = Buffer.from_numpy(np.ones((4, 8), F))           # (K=8, R=4)
    c = Buffer.from_numpy(np.ones((4, 32), F))          # (L=32, R=4)
    d = Buffer.from_numpy(np.zeros((4, 16), F))
    assert t2sp_b200.mttkrp(a, b, c, d) == -36
    cbad = Buffer.from_numpy(np.ones((4, 16), F))
    assert t2sp_b200.mttkrp(a, b, cbad, d) == -8
    dsmall = Buffer.from_numpy(np.zeros((4, 8), F))
    assert t2sp_b200.mttkrp(a, b, c, dsmall) == -4


def test_no_device_means_loud_failure_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    A, B, C = bufs()
    before = lib.t2sp_b200_kernel_launches()
    assert t2sp_b200.gemm(A, B, C) == -36
    assert lib.t2sp_b200_kernel_launches() == before
    assert np.all(C.keepalive == 0)                       # nothing computed anywhere
    assert lib.t2sp_b200_mttkrp_noalloc(256, 32, 512, 256, 8, 256, 32, 256, 16, 32, 16, 8, 4, None, 1) != 0


def test_device_helpers_without_device(lib):
    A, _, _ = bufs()
    assert lib.t2sp_b200_wrap_device_ptr(A.ptr, 4096) == 0
    assert A.raw.device == 4096 and A.raw.device_interface == lib.t2sp_b200_device_interface()
    assert lib.t2sp_b200_wrap_device_ptr(A.ptr, 8192) == -32     # already wrapped
    assert lib.t2sp_b200_detach_device_ptr(A.ptr) == 0 and A.raw.device == 0
    assert lib.t2sp_b200_set_device(99) == -36
    assert lib.t2sp_b200_set_device(0) == 0


def test_nd_fronts_and_syrk_validation(lib):
    """conv_nd / capsule_nd / syrk read every constant from the extents; inconsistent shapes are
    rejected on the host with the reference's codes before any device work."""
    z = lambda *shape: Buffer.from_numpy(np.zeros(shape, F))
    assert lib.t2sp_b200_conv_nd(None, None, None, 0) == -12
    assert lib.t2sp_b200_capsule_nd(None, None, None, 0) == -12
    assert lib.t2sp_b200_syrk(0, ctypes.c_float(1), ctypes.c_float(0), None, None, None) == -12
    # conv: I(IY,IX,CI,N) numpy (N,CI,IX,IY); K (CO,CI,KX,KY); O 10-D
    I, K = z(2, 8, 6, 6), z(8, 8, 3, 3)
    assert t2sp_b200.conv_nd(I, K, z(2, 1, 1, 1, 1, 1, 2, 4, 4, 4)) == -36   # consistent: only the missing device stops it
    assert t2sp_b200.conv_nd(I, K, z(2, 1, 1, 1, 1, 1, 2, 4, 5, 4)) == -8    # OY = 5 but IY - KY + 1 = 4
    assert t2sp_b200.conv_nd(I, z(8, 4, 3, 3), z(2, 1, 1, 1, 1, 1, 2, 4, 4, 4)) == -8   # channel counts differ
    assert t2sp_b200.conv_nd(I, K, z(3, 1, 1, 1, 1, 1, 2, 4, 4, 4)) == -8    # batch differs
    assert t2sp_b200.conv_nd(z(8, 6, 6), K, z(2, 1, 1, 1, 1, 1, 2, 4, 4, 4)) == -43  # 3-D input: bad dimensions
    assert t2sp_b200.conv_nd(Buffer.from_numpy(np.zeros((2, 8, 6, 6), np.float64)), K, z(2, 1, 1, 1, 1, 1, 2, 4, 4, 4)) == -3
    # capsule: P (N,IX,IY,CI,MX,MK), W (KX,KY,CO,CI,MK,MY), V (N,CO_o,COO,MX,MY,Y_X,YY_XX,YYY_XXX,COOO)
    P, W = z(2, 5, 5, 4, 4, 4), z(3, 3, 8, 4, 4, 4)
    assert t2sp_b200.capsule_nd(P, W, z(2, 1, 2, 4, 4, 1, 1, 4, 4)) == -36   # stride 2: 5 -> 2 x 2 outputs = 4 slots
    assert t2sp_b200.capsule_nd(P, W, z(2, 1, 2, 4, 4, 1, 1, 9, 4)) == -36   # stride 1: 3 x 3 outputs = 9 slots
    assert t2sp_b200.capsule_nd(P, W, z(2, 1, 2, 4, 4, 1, 1, 3, 4)) == -8    # 3 pixel slots hold neither 2 x 2 nor 3 x 3 outputs
    assert t2sp_b200.capsule_nd(P, z(3, 3, 8, 4, 2, 4), z(2, 1, 2, 4, 4, 1, 1, 4, 4)) == -8  # MK differs
    # syrk: A (N,K), C (N,N), O (I, I+1, II, II, III, III) with N = III*II*I
    A, C = z(16, 8), z(16, 16)
    assert t2sp_b200.syrk(0, 1.0, 0.0, A, C, z(4, 5, 2, 2, 2, 2)) == -36
    assert t2sp_b200.syrk(0, 1.0, 0.0, A, C, z(4, 5, 2, 2, 2, 3)) == -8      # the two innermost extents must agree
    assert t2sp_b200.syrk(0, 1.0, 0.0, A, C, z(2, 4, 2, 2, 2, 2)) == -8      # I = 3 is odd
    assert t2sp_b200.syrk(0, 1.0, 0.0, z(12, 8), C, z(4, 5, 2, 2, 2, 2)) == -8   # N != III*II*I
    # ger: A (TI,TK), X (TI,), Y (TK,), O (I, K, KK, II, III, KKK)
    assert lib.t2sp_b200_ger(None, None, None, None) == -12
    A, X, Y = z(8, 16), z(8), z(16)
    assert t2sp_b200.ger(A, X, Y, z(2, 2, 2, 2, 2, 4)) == -36
    assert t2sp_b200.ger(A, X, Y, z(2, 2, 2, 2, 2, 2)) == -8     # KKK*KK*K = 8, A has 16 columns
    assert t2sp_b200.ger(A, X, Y, z(2, 2, 2, 2, 3, 4)) == -8     # III*II*I = 12, A has 8 rows
    assert t2sp_b200.ger(A, z(4), Y, z(2, 2, 2, 2, 2, 4)) == -4  # X shorter than A's row count
    assert t2sp_b200.ger(A, X, z(2, 8), z(2, 2, 2, 2, 2, 4)) == -43  # Y must be 1-D


def test_bf16_cross_term_formulation_bound():
    """The arithmetic of the fp32 pair kernel with bf16 cross terms, restated in numpy (no GPU): a = hi + lo with
    hi = a truncated to TF32 (what the tensor core reads from a raw fp32 word) and lo = a - hi (exact in fp32);
    a b ~ hi_a hi_b + bf16(lo_a) bf16(b) + bf16(a) bf16(lo_b), products and sums exact here (fp64), so that only the
    formulation's own error shows: the dropped lo_a lo_b (2^-22) and the four bf16 roundings of terms that are
    2^-11 of the product. Bound per product: 2 x 2^-9 x 2^-11 x (1 + 2^-9) + 2^-22 < 2^-18.
    K = 8192 on mixed-sign and on positive inputs, elementwise relative to sum_k |a||b|."""
    import numpy as np
    from tests import oracle_lib as O

    def tf32_trunc(x):
        return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)

    def bf16(x):
        return O.bf16_to_f32(O.to_bf16(x))

    M, N, K = 48, 40, 8192
    for positive in (False, True):
        A, B = O.uniform(41, 1, (M, K)), O.uniform(41, 2, (K, N))
        if positive:
            A, B = np.abs(A), np.abs(B)
        hi_a, hi_b = tf32_trunc(A), tf32_trunc(B)
        lo_a, lo_b = A - hi_a, B - hi_b
        assert np.array_equal(hi_a.astype(np.float64) + lo_a.astype(np.float64), A.astype(np.float64)), "the split is exact"
        f = np.float64
        got = hi_a.astype(f) @ hi_b.astype(f) + bf16(lo_a).astype(f) @ bf16(B).astype(f) + bf16(A).astype(f) @ bf16(lo_b).astype(f)
        truth = A.astype(f) @ B.astype(f)
        absprod = np.abs(A).astype(f) @ np.abs(B).astype(f)
        err = float(np.max(np.abs(got - truth) / absprod))
        assert err < 2.0 ** -18, err
        # on positive inputs nothing cancels: the typical error is far below the bound
        if positive:
            assert err < 2.0 ** -20, err
