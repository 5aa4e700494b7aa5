"""Parity at the full sizes of the published configurations (the other GPU tests run scaled-down
shapes so that the CPU oracle finishes quickly):

 * GEMM 8192^3 and 16384^3 (bf16 and int8): 64 random 64 x 64 output tiles each, recomputed on the CPU in fp64 from
   the K-length rows and columns they need (exact for the bf16 and int8 products); int8 bit-exact;
 * GEMM 4096^3: the whole matrix, against an fp64 BLAS product (exact for int8: |sum| < 2^53);
 * conv (64 x 256 x 14 x 14, 3x3), TTM (512.512.256 -> 256), MTTKRP (512^3, R = 64) and capsule
   (batch 32, 32 -> 32 channels, 4x4 poses, 16 x 16, 3x3, stride 1) at their full sizes, against
   fp64 references (numpy BLAS for TTM / MTTKRP, the oracle's fp64-accumulated form for conv / capsule), in the
   normwise form and element by element against sum |a||b| (the same reference run on the absolute values).
"""
import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer, CapsuleDesc, ConvDesc
from tests import oracle_lib as O
from tests.util import TOL_BF16, TOL_FP32, call_gemm, componentwise, normwise

pytestmark = pytest.mark.gpu


def _gemm_inputs(dtype, n, seed):
    if dtype == "i8":
        return O.int8(seed, 1, (n, n)), O.int8(seed, 2, (n, n))
    A, B = O.to_bf16(O.uniform(seed, 1, (n, n))), O.to_bf16(O.uniform(seed, 2, (n, n)))
    return A, B


def _as_f64(x, dtype):
    return x.astype(np.float64) if dtype == "i8" else O.bf16_to_f32(x).astype(np.float64)


@pytest.mark.parametrize("dtype,n", [("bf16", 8192), ("i8", 8192), ("bf16", 16384), ("i8", 16384)])
def test_gemm_large_sampled_tiles(lib, dtype, n):
    A, B = _gemm_inputs(dtype, n, 31)
    rc, C = call_gemm(A, B, dtype, out_dtype=np.int32 if dtype == "i8" else np.float32)
    assert rc == 0
    pick = O.rng(31, 9)
    worst = 0.0
    for _ in range(64):
        r0, c0 = (int(v) * 64 for v in pick.integers(0, n // 64, size=2))
        truth = _as_f64(A[r0:r0 + 64], dtype) @ _as_f64(np.ascontiguousarray(B[:, c0:c0 + 64]), dtype)
        got = C[r0:r0 + 64, c0:c0 + 64]
        if dtype == "i8":
            assert np.array_equal(got.astype(np.int64), truth.astype(np.int64)), (r0, c0)
        else:
            worst = max(worst, float(np.max(np.abs(got - truth)) / np.max(np.abs(truth))))
    if dtype != "i8":
        print(f"{dtype} {n}^3: worst tile error {worst:.2e}")
        # bf16 products are exact in fp32, so all of the error is the tensor core's fp32 accumulation
        # (about 1e-5 of a tile's largest element at K = 8192), far inside the bf16 tolerance
        assert worst <= TOL_BF16
        assert worst <= 1e-4


@pytest.mark.parametrize("dtype", ["bf16", "i8"])
def test_gemm_4096_full_matrix(lib, dtype):
    n = 4096
    A, B = _gemm_inputs(dtype, n, 32)
    rc, C = call_gemm(A, B, dtype, out_dtype=np.int32 if dtype == "i8" else np.float32)
    assert rc == 0
    truth = _as_f64(A, dtype) @ _as_f64(B, dtype)
    if dtype == "i8":
        assert np.array_equal(C.astype(np.int64), np.rint(truth).astype(np.int64))
    else:
        assert normwise(C, truth) <= 1e-4 and normwise(C, truth) <= TOL_BF16


def test_conv_published_size(lib):
    N, CI, CO, KY, KX, OY, OX = 64, 256, 256, 3, 3, 14, 14
    IY, IX = OY + KY - 1, OX + KX - 1
    I2 = O.uniform(33, 1, (IY * IX, CI * N))
    K2 = O.normal(33, 2, (CI * KY, CO * KX), (1.0 / (KY * KX * CI)) ** 0.5)
    d = ConvDesc()
    d.CI, d.CO, d.KY, d.KX, d.OY, d.OX = CI, CO, KY, KX, OY, OX
    out = np.full((OY * OX, CO * N), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    assert t2sp_b200.conv(Buffer.from_numpy(I2), Buffer.from_numpy(K2), ob, d) == 0
    truth = O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=True)
    assert not np.isnan(ob.keepalive).any()
    assert normwise(ob.keepalive, truth) <= TOL_FP32
    # and element by element against sum |input| |weight|: one more oracle pass on the absolute values
    absprod = O.conv_f32(np.abs(I2), np.abs(K2), N, CI, CO, KY, KX, OY, OX, acc64=True)
    assert componentwise(ob.keepalive, truth, absprod) <= TOL_FP32


def test_ttm_published_size(lib):
    L, I, J, K = 256, 512, 512, 256
    a = O.uniform(34, 1, (J, I, L))
    b = O.uniform(34, 2, (K, L))
    c = np.full((K, J, I), np.nan, np.float32)
    cb = Buffer.from_numpy(c)
    assert t2sp_b200.ttm(Buffer.from_numpy(a), Buffer.from_numpy(b), cb) == 0
    truth = b.astype(np.float64) @ a.reshape(J * I, L).astype(np.float64).T  # [k, (j, i)]
    assert normwise(cb.keepalive.reshape(K, J * I), truth) <= TOL_FP32
    absprod = np.abs(b).astype(np.float64) @ np.abs(a).reshape(J * I, L).astype(np.float64).T
    assert componentwise(cb.keepalive.reshape(K, J * I), truth, absprod) <= TOL_FP32


def test_mttkrp_published_size(lib):
    L, I, K, R = 512, 512, 512, 64
    a = O.uniform(35, 1, (K, I, L))
    b = O.uniform(35, 2, (R, K))
    c = O.uniform(35, 3, (R, L))
    d = np.full((R, I), np.nan, np.float32)
    db = Buffer.from_numpy(d)
    assert t2sp_b200.mttkrp(Buffer.from_numpy(a), Buffer.from_numpy(b), Buffer.from_numpy(c), db) == 0
    truth, absprod = np.zeros((R, I)), np.zeros((R, I))
    c64, b64 = c.astype(np.float64), b.astype(np.float64)
    for k in range(K):  # d(i, r) = sum_k (sum_l a(l, i, k) c(l, r)) b(k, r), one k-slice at a time
        ak = a[k].astype(np.float64).T
        truth += (c64 @ ak) * b64[:, k:k + 1]
        absprod += (np.abs(c64) @ np.abs(ak)) * np.abs(b64[:, k:k + 1])
    assert normwise(db.keepalive, truth) <= TOL_FP32
    assert componentwise(db.keepalive, truth, absprod) <= TOL_FP32


def test_capsule_published_size(lib):
    N, NN, CI, CO, KY, KX, OY, OX, M, s = 1, 32, 32, 32, 3, 3, 16, 16, 4, 1  # batch = NN * N = 32
    IY, IX = s * OY + KY - s, s * OX + KX - s
    P2 = O.normal(36, 1, (IY * IX * N, CI * M * M * NN), 0.1)
    W2 = O.normal(36, 2, (CI * KY * KX * M, CO * M), 0.1)
    d = CapsuleDesc()
    d.CI, d.CII, d.CO, d.KY, d.KX, d.OY, d.OX = CI, CI, CO, KY, KX, OY, OX
    d.MY = d.MX = d.MK = M
    d.NN, d.stride = NN, s
    out = np.full((OY * OX * N, CO * M * M * NN), np.nan, np.float32)
    vb = Buffer.from_numpy(out)
    assert t2sp_b200.capsule(Buffer.from_numpy(P2), Buffer.from_numpy(W2), vb, d) == 0
    truth = O.capsule_f32(P2, W2, N, NN, CI, CI, CO, KY, KX, OY, OX, M, M, M, s, acc64=True)
    assert not np.isnan(vb.keepalive).any()
    assert normwise(vb.keepalive, truth) <= TOL_FP32
    absprod = O.capsule_f32(np.abs(P2), np.abs(W2), N, NN, CI, CI, CO, KY, KX, OY, OX, M, M, M, s, acc64=True)
    assert componentwise(vb.keepalive, truth, absprod) <= TOL_FP32
