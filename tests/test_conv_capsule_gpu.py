"""2-D convolution and capsule convolution parity on the GPU through the C ABI against the
CPU oracle, at the reference's TINY and GPU design constants
(t2s/tests/performance/{conv,capsule}/const-parameters.h) and at scaled-down BASELINE shapes."""
import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer, CapsuleDesc, ConvDesc
from tests import oracle_lib as O
from tests.util import TOL_FP32, componentwise, normwise

pytestmark = pytest.mark.gpu


def conv_inputs(seed, N, CI, CO, KY, KX, OY, OX):
    IY, IX = OY + KY - 1, OX + KX - 1
    I2 = O.uniform(seed, 1, (IY * IX, CI * N))
    K2 = O.normal(seed, 2, (CI * KY, CO * KX), (1.0 / (KY * KX * CI)) ** 0.5)
    return I2, K2


def run_conv(I2, K2, N, CI, CO, KY, KX, OY, OX, tiles=None):
    d = ConvDesc()
    d.CI, d.CO, d.KY, d.KX, d.OY, d.OX = CI, CO, KY, KX, OY, OX
    if tiles is None:
        out = np.full((OY * OX, CO * N), np.nan, np.float32)
    else:
        COOO, YYY, XXX, COO, YY, XX, Y, X = tiles
        d.layout = 1
        d.COOO, d.YYY, d.XXX, d.COO, d.YY, d.XX, d.Y, d.X = tiles
        out = np.full((N, CO // (COOO * COO), X, Y, XX, YY, COO, XXX, YYY, COOO), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    rc = t2sp_b200.conv(Buffer.from_numpy(I2), Buffer.from_numpy(K2), ob, d)
    return rc, ob.keepalive


CONV_CASES = [
    # N, CI, CO, KY, KX, OY, OX
    (4, 16, 64, 3, 3, 4, 4),      # TINY constants (CII*CI = 16, COOO*COO*CO = 64, 4x4 output)
    (8, 64, 128, 3, 3, 14, 14),   # BASELINE config 2 scaled down in batch and channels
    (64, 32, 64, 3, 3, 6, 4),     # batch 64: one TMA box = 64 images x 2 rows
    (3, 40, 72, 3, 2, 5, 7),      # ragged: channel counts not multiples of the tile sizes
    (2, 32, 32, 1, 1, 8, 8),      # 1x1 filter
    (64, 32, 256, 3, 3, 14, 14),  # BASELINE config 2 with fewer input channels: CTA-pair kernel, 256-wide tiles
    (64, 64, 128, 3, 3, 14, 12),  # CTA-pair kernel, 128-wide tiles
    (64, 40, 256, 3, 2, 14, 14),  # tensor-memory pair kernel with a channel count that ends inside a 32-channel block
    (64, 72, 200, 2, 3, 14, 14),  # ... and an output channel count that ends inside a tile
]


@pytest.mark.parametrize("N,CI,CO,KY,KX,OY,OX", CONV_CASES)
def test_conv_plain(lib, N, CI, CO, KY, KX, OY, OX):
    I2, K2 = conv_inputs(0, N, CI, CO, KY, KX, OY, OX)
    rc, out = run_conv(I2, K2, N, CI, CO, KY, KX, OY, OX)
    assert rc == 0
    assert not np.isnan(out).any(), "unwritten output elements"
    truth = O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=True)
    absprod = O.conv_f32(np.abs(I2), np.abs(K2), N, CI, CO, KY, KX, OY, OX, acc64=True)
    print(f"conv N{N} CI{CI} CO{CO} {KY}x{KX} {OY}x{OX}: normwise {normwise(out, truth):.3e} componentwise {componentwise(out, truth, absprod):.3e}")
    assert normwise(out, truth) <= TOL_FP32 and componentwise(out, truth, absprod) <= TOL_FP32
    assert normwise(out, O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, CII=min(CI, 8) if CI % 8 == 0 else 0)) <= TOL_FP32


def test_conv_tiled_output_tiny(lib):
    # 10-D output of conv-run-fpga.cpp:68 with the TINY constants (const-parameters.h:38-49)
    N, CI, CO, KY, KX, OY, OX = 4, 16, 64, 3, 3, 4, 4
    tiles = (4, 4, 4, 4, 1, 1, 1, 1)
    I2, K2 = conv_inputs(1, N, CI, CO, KY, KX, OY, OX)
    rc, out = run_conv(I2, K2, N, CI, CO, KY, KX, OY, OX, tiles)
    assert rc == 0 and not np.isnan(out).any()
    truth = O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=True)
    ref10 = O.conv_tile_layout(truth, N, 4, 4, 4, 4, 1, 1, 1, 1, 4)
    assert normwise(out, ref10) <= TOL_FP32


def test_conv_tiled_output_general(lib):
    # every tile extent > 1 so each digit of the 10-D address map is exercised
    N, CI, CO, KY, KX = 2, 32, 32, 3, 3
    COOO, YYY, XXX, COO, YY, XX, Y, X = 4, 2, 3, 2, 2, 2, 3, 2
    OY, OX = YYY * YY * Y, XXX * XX * X
    I2, K2 = conv_inputs(2, N, CI, CO, KY, KX, OY, OX)
    rc, out = run_conv(I2, K2, N, CI, CO, KY, KX, OY, OX, (COOO, YYY, XXX, COO, YY, XX, Y, X))
    assert rc == 0 and not np.isnan(out).any()
    truth = O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=True)
    ref10 = O.conv_tile_layout(truth, N, COOO, YYY, XXX, COO, YY, XX, Y, X, CO // (COOO * COO))
    assert normwise(out, ref10) <= TOL_FP32


def capsule_inputs(seed, N, NN, CI, CO, KY, KX, OY, OX, MY, MX, MK, s):
    IY, IX = s * OY + KY - s, s * OX + KX - s
    P2 = O.normal(seed, 1, (IY * IX * N, CI * MK * MX * NN), 0.1)
    W2 = O.normal(seed, 2, (CI * KY * KX * MK, CO * MY), 0.1)
    return P2, W2


def run_capsule(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, s, tiles=None, M=4):
    d = CapsuleDesc()
    d.CI, d.CII, d.CO, d.KY, d.KX, d.OY, d.OX = CI, CII, CO, KY, KX, OY, OX
    d.MY = d.MX = d.MK = M
    d.NN, d.stride = NN, s
    if tiles is None:
        out = np.full((OY * OX * N, CO * M * M * NN), np.nan, np.float32)
    else:
        COOO, YYY_XXX, YY_XX, Y_X, COO = tiles
        d.layout = 1
        d.COOO, d.YYY_XXX, d.YY_XX, d.Y_X, d.COO = tiles
        out = np.full((N, CO // (COOO * COO), NN, COO, M, M, Y_X, YY_XX, YYY_XXX, COOO), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    rc = t2sp_b200.capsule(Buffer.from_numpy(P2), Buffer.from_numpy(W2), ob, d)
    return rc, ob.keepalive


CAPSULE_CASES = [
    # N, NN, CI, CII, CO, KY, KX, OY, OX, stride
    (4, 1, 16, 4, 16, 3, 3, 7, 7, 2),    # TINY constants (capsule/const-parameters.h:46-55)
    (2, 16, 32, 4, 32, 3, 3, 7, 7, 2),   # GPU constants with a smaller batch
    (2, 4, 32, 32, 32, 3, 3, 8, 8, 1),   # BASELINE config 4 (stride 1) scaled down
    (2, 4, 32, 16, 32, 3, 3, 7, 7, 2),   # A10 constants (CII 16)
    (1, 2, 16, 4, 8, 2, 3, 3, 5, 1),     # ragged spatial extents, non-square filter
    (2, 32, 32, 32, 32, 3, 3, 8, 10, 1), # BASELINE config 4 with fewer pixels: CTA-pair kernel (M = 20480 rows)
    (8, 16, 16, 4, 32, 3, 3, 7, 7, 2),   # stride 2 on CTA pairs (two 64-row boxes per CTA)
]


@pytest.mark.parametrize("N,NN,CI,CII,CO,KY,KX,OY,OX,s", CAPSULE_CASES)
def test_capsule_plain(lib, N, NN, CI, CII, CO, KY, KX, OY, OX, s):
    P2, W2 = capsule_inputs(0, N, NN, CI, CO, KY, KX, OY, OX, 4, 4, 4, s)
    rc, out = run_capsule(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, s)
    assert rc == 0
    assert not np.isnan(out).any(), "unwritten output elements"
    truth = O.capsule_f32(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, 4, 4, 4, s, acc64=True)
    absprod = O.capsule_f32(np.abs(P2), np.abs(W2), N, NN, CI, CII, CO, KY, KX, OY, OX, 4, 4, 4, s, acc64=True)
    print(f"capsule N{N} NN{NN} CI{CI}/{CII} CO{CO} s{s}: normwise {normwise(out, truth):.3e} componentwise {componentwise(out, truth, absprod):.3e}")
    assert normwise(out, truth) <= TOL_FP32 and componentwise(out, truth, absprod) <= TOL_FP32
    assert normwise(out, O.capsule_f32(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, 4, 4, 4, s)) <= TOL_FP32


@pytest.mark.parametrize("tiles,NN,CI,CII,CO", [((4, 7, 1, 7, 4), 1, 16, 4, 16), ((8, 10, 1, 5, 4), 4, 32, 16, 32)])
def test_capsule_tiled_output(lib, tiles, NN, CI, CII, CO):
    # 10-D output of capsule-run-fpga.cpp:73: TINY constants, and the A10 constants whose
    # 10*1*5 = 50 pixel slots exceed the 49 pixels (slot 49 must be written as 0).
    N, KY, KX, OY, OX, s = 2, 3, 3, 7, 7, 2
    P2, W2 = capsule_inputs(3, N, NN, CI, CO, KY, KX, OY, OX, 4, 4, 4, s)
    rc, out = run_capsule(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, s, tiles)
    assert rc == 0 and not np.isnan(out).any()
    truth = O.capsule_f32(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, 4, 4, 4, s, acc64=True)
    COOO, YYY_XXX, YY_XX, Y_X, COO = tiles
    ref10 = O.capsule_tile_layout(truth, N, NN, COOO, COO, CO // (COOO * COO), YYY_XXX, YY_XX, Y_X, 4, 4, OY, OX)
    assert normwise(out, ref10) <= TOL_FP32


# ---------------------------------------------------------------- oneAPI-flow N-D operand layouts
def _tile10(out, COOO, YYY, XXX, COO, YY, XX, Y, X):
    """out[n, co, ox, oy] -> the 10-D o(COOO,YYY,XXX,COO,YY,XX,Y,X,CO,N) (numpy axes reversed)."""
    N, CO = out.shape[:2]
    t = out.reshape(N, CO // (COOO * COO), COO, COOO, X, XX, XXX, Y, YY, YYY)
    #               n  co_o               coo  cooo  x  xx  xxx  y  yy  yyy
    return np.ascontiguousarray(t.transpose(0, 1, 4, 7, 5, 8, 2, 6, 9, 3))


@pytest.mark.parametrize("N,CI,CO,KY,KX,tiles", [
    (4, 16, 64, 3, 3, (4, 4, 4, 4, 1, 1, 1, 1)),      # oneapi-target-5-parameters.h, TINY
    (3, 10, 24, 3, 2, (4, 2, 3, 2, 2, 1, 2, 2)),      # channels not a multiple of 4: zero-padded in the device copy
    (16, 64, 256, 3, 3, (8, 7, 7, 4, 2, 2, 1, 1)),    # wide enough for the CTA-pair kernel
])
def test_conv_nd_layout(lib, N, CI, CO, KY, KX, tiles):
    """I(IY,IX,CI,N), K(KY,KX,CI,CO) as the oneAPI flow passes them
    (t2s/tests/correctness/oneapi-integration/oneapi-target-5-run.cpp:92-117)."""
    COOO, YYY, XXX, COO, YY, XX, Y, X = tiles
    OY, OX = YYY * YY * Y, XXX * XX * X
    IY, IX = OY + KY - 1, OX + KX - 1
    I = O.uniform(21, 1, (N, CI, IX, IY))
    K = O.normal(21, 2, (CO, CI, KX, KY), (1.0 / (KY * KX * CI)) ** 0.5)
    out = np.full((N, CO // (COOO * COO), X, Y, XX, YY, COO, XXX, YYY, COOO), np.nan, np.float32)
    ob = Buffer.from_numpy(out)
    assert t2sp_b200.conv_nd(Buffer.from_numpy(I), Buffer.from_numpy(K), ob) == 0
    truth = np.zeros((N, CO, OX, OY))
    I64, K64 = I.astype(np.float64), K.astype(np.float64)
    for kx in range(KX):
        for ky in range(KY):
            truth += np.einsum("ncxy,oc->noxy", I64[:, :, kx:kx + OX, ky:ky + OY], K64[:, :, kx, ky])
    want = _tile10(truth, *tiles)
    got = ob.keepalive
    assert not np.isnan(got).any()
    assert normwise(got, want) <= TOL_FP32
    assert normwise(got, O.conv_nd_f32(I, K, tiles, acc64=True)) <= TOL_FP32   # the pinned oracle agrees


def test_conv_nd_rejects_inconsistent_extents(lib):
    I = np.zeros((2, 8, 6, 6), np.float32)
    K = np.zeros((8, 8, 3, 3), np.float32)
    out = np.zeros((2, 1, 1, 1, 1, 1, 2, 4, 5, 4), np.float32)  # OY = 5 but IY - KY + 1 = 4
    assert t2sp_b200.conv_nd(Buffer.from_numpy(I), Buffer.from_numpy(K), Buffer.from_numpy(out)) == -8
    assert t2sp_b200.lib().t2sp_b200_conv_nd(None, None, None, 0) == -12


@pytest.mark.parametrize("N,CI,CO,OY,OX,s,vt", [
    (4, 16, 16, 7, 7, 2, (4, 7, 1, 7, 4)),    # oneapi-target-6-parameters.h, TINY (COOO, YYY_XXX, YY_XX, Y_X, COO)
    (2, 8, 32, 6, 5, 1, (8, 6, 5, 1, 2)),     # stride 1, as BASELINE's capsule configuration
])
def test_capsule_nd_layout(lib, N, CI, CO, OY, OX, s, vt):
    """P(MK,MX,CI,IY,IX,N), W(MY,MK,CI,CO,KY,KX), 9-D V as the oneAPI flow passes them
    (t2s/tests/correctness/oneapi-integration/oneapi-target-6-run.cpp:92-173)."""
    MY = MX = MK = 4
    KY = KX = 3
    COOO, YYY_XXX, YY_XX, Y_X, COO = vt
    IY, IX = s * OY + KY - s, s * OX + KX - s
    P = O.normal(22, 1, (N, IX, IY, CI, MX, MK), 0.1)
    W = O.normal(22, 2, (KX, KY, CO, CI, MK, MY), 0.1)
    V = np.full((N, CO // (COOO * COO), COO, MX, MY, Y_X, YY_XX, YYY_XXX, COOO), np.nan, np.float32)
    vb = Buffer.from_numpy(V)
    assert t2sp_b200.capsule_nd(Buffer.from_numpy(P), Buffer.from_numpy(W), vb) == 0
    P64, W64 = P.astype(np.float64), W.astype(np.float64)
    truth = np.zeros((N, CO, OX, OY, MX, MY))  # [n, co, ox, oy, mx, my]
    for kx in range(KX):
        for ky in range(KY):
            Ps = P64[:, kx:kx + s * OX:s, ky:ky + s * OY:s]  # [n, ox, oy, ci, mx, mk]
            truth += np.einsum("nxycmk,ockj->noxymj", Ps, W64[kx, ky])  # m = mx, k = mk, j = my
    got = vb.keepalive
    assert not np.isnan(got).any()
    # pixel slot p = yyy_xxx + YYY_XXX*yy_xx + YYY_XXX*YY_XX*y_x holds (oy, ox) = (p % OY, p / OY)
    want = np.zeros_like(got, dtype=np.float64)
    for p in range(YYY_XXX * YY_XX * Y_X):
        if p >= OY * OX:
            continue
        oy, ox = p % OY, p // OY
        a, b, c = p % YYY_XXX, (p // YYY_XXX) % YY_XX, p // (YYY_XXX * YY_XX)
        blk = truth[:, :, ox, oy].reshape(N, CO // (COOO * COO), COO, COOO, MX, MY)  # [n, co_o, coo, cooo, mx, my]
        want[:, :, :, :, :, c, b, a, :] = blk.transpose(0, 1, 2, 4, 5, 3)
    assert normwise(got, want) <= TOL_FP32
    assert normwise(got, O.capsule_nd_f32(P, W, vt, s, acc64=True)) <= TOL_FP32   # the pinned oracle agrees
