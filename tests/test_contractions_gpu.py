"""TTM and MTTKRP parity on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer
from tests import oracle_lib as O
from tests.util import TOL_FP32, componentwise, normwise

pytestmark = pytest.mark.gpu


def run_ttm(a, b, tiled=None):
    J, I, L = a.shape
    K = b.shape[0]
    if tiled is None:
        c = np.full((K, J, I), np.nan, np.float32)
    else:
        JJ, KK, II, KKK, JJJ, III = tiled
        c = np.full((I // (III * II), J // (JJJ * JJ), K // (KKK * KK), III, JJJ, KKK, II, KK, JJ), np.nan, np.float32)
    cb = Buffer.from_numpy(c)
    rc = t2sp_b200.ttm(Buffer.from_numpy(a), Buffer.from_numpy(b), cb)
    return rc, cb.keepalive


def test_ttm_known_answer(lib):
    # SEQUENTIAL fixtures of t2s/tests/correctness/buffer/tmm_small.cpp:131-132 at its 8x8x8x8
    # size: a(l,i,j) = l + i + j, b(l,k) = l + k + 1 (util.h:52-65,100-114); exact integers.
    L = I = J = K = 8
    l = np.arange(L)
    a = (np.arange(J)[:, None, None] + np.arange(I)[None, :, None] + l[None, None, :]).astype(np.float32)
    b = (np.arange(K)[:, None] + l[None, :] + 1).astype(np.float32)
    rc, c = run_ttm(a, b)
    assert rc == 0
    ref = np.einsum("jil,kl->kji", a.astype(np.float64), b.astype(np.float64))
    assert np.array_equal(c, ref.astype(np.float32))
    # and the 9-D device layout of the same test (tmm_small.cpp:116-129), all tile extents 2
    rc, c9 = run_ttm(a, b, tiled=(2, 2, 2, 2, 2, 2))
    assert rc == 0
    assert np.array_equal(c9, O.ttm_tile_layout(ref.astype(np.float32), 2, 2, 2, 2, 2, 2))


@pytest.mark.parametrize("L,I,J,K", [(256, 64, 48, 256), (100, 24, 10, 72), (64, 128, 128, 64),
                                     (96, 128, 100, 256), (64, 256, 64, 128),  # these two run on CTA pairs
                                     (100, 128, 96, 256), (72, 100, 99, 250)])  # pairs; L, rows and K ending inside blocks / tiles
def test_ttm_random(lib, L, I, J, K):
    a = O.uniform(0, 1, (J, I, L))
    b = O.uniform(0, 2, (K, L))
    rc, c = run_ttm(a, b)
    assert rc == 0
    assert not np.isnan(c).any()
    truth = O.ttm_f32(a, b, acc64=True)
    absprod = O.ttm_f32(np.abs(a), np.abs(b), acc64=True)
    print(f"ttm L{L} I{I} J{J} K{K}: normwise {normwise(c, truth):.3e} componentwise {componentwise(c, truth, absprod):.3e}")
    assert normwise(c, truth) <= TOL_FP32 and componentwise(c, truth, absprod) <= TOL_FP32
    assert normwise(c, O.ttm_f32(a, b)) <= TOL_FP32


def test_ttm_tiled_output_many_row_tiles(lib):
    """The 9-D tiled output through the scatter epilogue of the tensor-memory pair kernel (12288 rows i + I*j over a
    256-column factor: 48 row tiles)."""
    L, I, J, K = 96, 128, 96, 256
    tiles = (2, 4, 2, 8, 2, 4)  # JJ, KK, II, KKK, JJJ, III
    a = O.uniform(5, 1, (J, I, L))
    b = O.uniform(5, 2, (K, L))
    rc, c9 = run_ttm(a, b, tiled=tiles)
    assert rc == 0
    assert not np.isnan(c9).any()
    ref9 = O.ttm_tile_layout(O.ttm_f32(a, b, acc64=True).astype(np.float32), *tiles)
    assert normwise(c9, ref9) <= TOL_FP32


def run_mttkrp(a, b, c, splits=0):
    K, I, L = a.shape
    R = b.shape[0]
    d = np.full((R, I), np.nan, np.float32)
    db = Buffer.from_numpy(d)
    desc = t2sp_b200.MttkrpDesc(0, splits)
    rc = t2sp_b200.mttkrp(Buffer.from_numpy(a), Buffer.from_numpy(b), Buffer.from_numpy(c), db, desc)
    return rc, db.keepalive


def test_mttkrp_known_answer(lib):
    # SEQUENTIAL-style integer data: exact under any association of the sums.
    L, I, K, R = 8, 8, 8, 8
    a = (np.arange(K)[:, None, None] + np.arange(I)[None, :, None] + np.arange(L)[None, None, :]).astype(np.float32)
    b = (np.arange(R)[:, None] + np.arange(K)[None, :] + 1).astype(np.float32)
    c = (np.arange(R)[:, None] + np.arange(L)[None, :] + 1).astype(np.float32)
    rc, d = run_mttkrp(a, b, c)
    assert rc == 0
    ref = np.einsum("kil,rl,rk->ri", a.astype(np.float64), c.astype(np.float64), b.astype(np.float64))
    assert np.array_equal(d, ref.astype(np.float32))


@pytest.mark.parametrize("L,I,K,R,splits", [(64, 128, 32, 64, 0), (96, 200, 17, 40, 5), (128, 256, 64, 64, 1), (32, 64, 8, 128, 3)])
def test_mttkrp_random(lib, L, I, K, R, splits):
    a = O.uniform(0, 1, (K, I, L))
    b = O.uniform(0, 2, (R, K))
    c = O.uniform(0, 3, (R, L))
    rc, d = run_mttkrp(a, b, c, splits)
    assert rc == 0
    assert not np.isnan(d).any()
    truth = O.mttkrp_f32(a, b, c, acc64=True)
    absprod = O.mttkrp_f32(np.abs(a), np.abs(b), np.abs(c), acc64=True)
    print(f"mttkrp L{L} I{I} K{K} R{R}: normwise {normwise(d, truth):.3e} componentwise {componentwise(d, truth, absprod):.3e}")
    assert normwise(d, truth) <= TOL_FP32 and componentwise(d, truth, absprod) <= TOL_FP32
    assert normwise(d, O.mttkrp_f32(a, b, c)) <= TOL_FP32
    # deterministic: the split partial sums are added in a fixed order
    rc2, d2 = run_mttkrp(a, b, c, splits)
    assert rc2 == 0 and np.array_equal(d, d2)


@pytest.mark.parametrize("splits", [1, 5])
def test_mttkrp_padded_output_pitch(lib, splits):
    """d with a row pitch wider than I (d.stride.1 = I + 12): the ordered sum over the split slabs must
    address slab s of column r, and the 12 elements between the columns are the caller's (NaN stays NaN)."""
    L, I, K, R, pad = 96, 200, 17, 40, 12
    a, b, c = O.uniform(5, 1, (K, I, L)), O.uniform(5, 2, (R, K)), O.uniform(5, 3, (R, L))
    d = np.full((R, I + pad), np.nan, np.float32)
    db = Buffer((I, R), "f32", host=d.ctypes.data, strides=(1, I + pad), keepalive=d)
    rc = t2sp_b200.mttkrp(Buffer.from_numpy(a), Buffer.from_numpy(b), Buffer.from_numpy(c), db, t2sp_b200.MttkrpDesc(0, splits))
    assert rc == 0
    assert np.isnan(d[:, I:]).all()
    assert not np.isnan(d[:, :I]).any()
    assert normwise(d[:, :I], O.mttkrp_f32(a, b, c, acc64=True)) <= TOL_FP32


@pytest.mark.parametrize("III,II,I,K", [(12, 8, 8, 1024), (4, 2, 4, 40), (8, 4, 2, 100)])
def test_syrk_folded_output(lib, III, II, I, K):
    """O(jjj,iii,jj,ii,j,i) = Alpha * (A A^T)(r,c) + Beta * C(r,c) with the fold of
    t2s/tests/performance/syrk/syrk.cpp:38-73: (r,c) = (N-1-ti, N-1-tj) for i >= j, else (ti, tj - III*II)."""
    N = III * II * I
    A = O.uniform(14, 1, (N, K))
    Cs = O.uniform(14, 2, (N, N))
    Cs = ((Cs + Cs.T) * 0.5).astype(np.float32)
    alpha, beta = 1.5, -0.25
    out = np.full((I, I + 1, II, II, III, III), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    assert t2sp_b200.syrk(0, alpha, beta, Buffer.from_numpy(A), Buffer.from_numpy(Cs), ob) == 0
    R = alpha * (A.astype(np.float64) @ A.astype(np.float64).T) + beta * Cs.astype(np.float64)
    got = ob.keepalive
    t = III * II
    want = np.full(got.shape, np.nan)
    i, j, ii, jj, iii, jjj = np.meshgrid(np.arange(I // 2), np.arange(I + 1), np.arange(II), np.arange(II),
                                         np.arange(III), np.arange(III), indexing="ij")
    ti, tj = iii + III * ii + t * i, jjj + III * jj + t * j
    bot = i >= j
    r = np.where(bot, N - 1 - ti, ti)
    c = np.where(bot, N - 1 - tj, tj - t)
    want[:I // 2] = R[r, c]
    assert not np.isnan(got[:I // 2]).any()
    assert np.isnan(got[I // 2:]).all(), "rows i >= I/2 of the folded buffer are not part of the design's output"
    assert normwise(got[:I // 2], want[:I // 2]) <= TOL_FP32
    assert normwise(got[:I // 2], O.syrk_f32(A, Cs, III, II, I, alpha, beta, acc64=True)[:I // 2]) <= TOL_FP32


@pytest.mark.parametrize("KKK,III,II,KK,K,I", [(16, 10, 4, 4, 3, 2), (2, 2, 2, 2, 2, 2), (6, 3, 2, 5, 2, 3), (8, 7, 5, 6, 2, 2),
                                               (4, 3, 3, 3, 2, 2), (12, 5, 2, 2, 2, 2)])
def test_ger_tiled_output_bit_exact(lib, KKK, III, II, KK, K, I):
    """O(kkk,iii,ii,kk,k,i) = A(tk,ti) + X(ti) * Y(tk) (t2s/tests/performance/ger/ger.cpp:34-62): one
    rounded product and one rounded sum per element, so the result equals the oracle's bit for bit
    (KKK = 16, 8, 4: the row-tiled 16-byte kernel with 4, 2 and 1 kk per row group; KKK = 12: the generic
    16-byte kernel, as 3 x 2 threads per row do not divide a CTA; KKK = 2 and 6: the scalar kernel)."""
    TI, TK = III * II * I, KKK * KK * K
    A, X, Y = O.uniform(15, 1, (TI, TK)), O.uniform(15, 2, (TI,)), O.uniform(15, 3, (TK,))
    out = np.full((I, K, KK, II, III, KKK), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    assert t2sp_b200.ger(Buffer.from_numpy(A), Buffer.from_numpy(X), Buffer.from_numpy(Y), ob) == 0
    want = O.ger_f32(A, X, Y, KKK, III, II, KK, K, I)
    assert np.array_equal(ob.keepalive.view(np.uint32), want.view(np.uint32))
    # and the oracle's layout against plain numpy
    plain = A + (X[:, None] * Y[None, :]).astype(np.float32)
    assert np.array_equal(want, plain.reshape(I, II, III, K, KK, KKK).transpose(0, 3, 4, 1, 2, 5))


def test_ger_published_size_a10(lib):
    """The A10 design constants with its 32 x 32 outer loops (const-parameters.h:45-50, ger-run-fpga.cpp:29-30):
    10240 x 16384 elements, checked in full against numpy (same two roundings)."""
    KKK, III, II, KK, K, I = 16, 10, 32, 32, 32, 32
    TI, TK = III * II * I, KKK * KK * K
    A, X, Y = O.uniform(16, 1, (TI, TK)), O.uniform(16, 2, (TI,)), O.uniform(16, 3, (TK,))
    ob = Buffer.from_numpy(np.empty((I, K, KK, II, III, KKK), np.float32))
    assert t2sp_b200.ger(Buffer.from_numpy(A), Buffer.from_numpy(X), Buffer.from_numpy(Y), ob) == 0
    plain = A + (X[:, None] * Y[None, :]).astype(np.float32)
    assert np.array_equal(ob.keepalive, plain.reshape(I, II, III, K, KK, KKK).transpose(0, 3, 4, 1, 2, 5))
