"""The CPU oracle against everything that pins it (no GPU needed):
 - the reference's own, unmodified host drivers, linked against the oracle exposed under the
   interface symbols (oracle/ref_interface.cpp); they need the mounted reference tree to build;
 - the golden loops of the reference's test helper for TTM and MTTKRP (correctness/util/util.h:428-441,
   464-481), compiled unmodified into oracle/_ref/pin_contractions, which must give the oracle's bits;
 - the reference's deterministic fixtures evaluated exactly (tests/golden/kat.npz);
 - independent numpy formulations of conv and capsule."""
import os
import subprocess

import numpy as np
import pytest

from tests import oracle_lib as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("T2SP_REFERENCE", "/root/reference")
KAT = np.load(os.path.join(ROOT, "tests", "golden", "kat.npz"))


@pytest.mark.parametrize("name", ["pin_gemm_tiny", "pin_conv_tiny", "pin_capsule_tiny", "pin_aot_gemm", "pin_syrk_tiny", "pin_ger_tiny",
                                  "pin_oneapi_conv_tiny", "pin_oneapi_capsule_tiny", "pin_contractions"])
def test_reference_driver_accepts_oracle(name):
    exe = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(exe):
        if not os.path.isdir(REF):
            pytest.skip("reference tree not mounted and pin binaries not built")
        subprocess.run(["bash", os.path.join(ROOT, "oracle", "build_ref_drivers.sh")], check=True, capture_output=True)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-500:]
    assert res.stdout.strip().splitlines()[-1].startswith("Success")


def test_golden_aot_gemm_fixture():
    # |c| reaches ~2.9e9 with K = 2048 terms of up to ~4e6: not exact in fp32, so compare like the
    # reference does (aot/gemm-run.cpp:78: 0.5 % relative), and exactly with the fp64 variant.
    a, b, exact = KAT["aot_gemm_a"], KAT["aot_gemm_b"], KAT["aot_gemm_c_exact"].astype(np.float64)
    c64 = O.gemm_f32(a, b, acc64=True).astype(np.float64)
    assert np.max(np.abs(c64 - exact) / np.maximum(np.abs(exact), 1)) < 1e-6
    c32 = O.gemm_f32(a, b).astype(np.float64)
    nz = np.abs(exact) > 0
    assert np.all(np.abs(c32 - exact)[nz] < 0.005 * np.abs(exact)[nz])


def test_golden_sequential_fixtures_exact():
    assert np.array_equal(O.gemm_f32(KAT["seq_gemm_a"], KAT["seq_gemm_b"]), KAT["seq_gemm_c_exact"].astype(np.float32))
    assert np.array_equal(O.ttm_f32(KAT["seq_ttm_a"], KAT["seq_ttm_b"]), KAT["seq_ttm_c_exact"].astype(np.float32))
    assert np.array_equal(O.mttkrp_f32(KAT["seq_mttkrp_a"], KAT["seq_mttkrp_b"], KAT["seq_mttkrp_c"]),
                          KAT["seq_mttkrp_d_exact"].astype(np.float32))


def test_constant_conv_fixture():
    N, CI, CO, KY, KX, OY, OX = 2, 16, 8, 3, 3, 4, 4
    I2 = np.ones(((OY + 2) * (OX + 2), CI * N), np.float32)
    K2 = np.ones((CI * KY, CO * KX), np.float32)
    assert np.all(O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX) == float(KAT["const_conv_expected"][0]))


def test_int8_and_bf16_variants_against_numpy():
    A, B = O.int8(0, 1, (37, 50)), O.int8(0, 2, (50, 41))
    assert np.array_equal(O.gemm_i8(A, B), A.astype(np.int64) @ B.astype(np.int64))
    Af, Bf = O.uniform(0, 1, (33, 64)), O.uniform(0, 2, (64, 40))
    Ab, Bb = O.to_bf16(Af), O.to_bf16(Bf)
    ref = O.bf16_to_f32(Ab).astype(np.float64) @ O.bf16_to_f32(Bb).astype(np.float64)
    assert np.allclose(O.gemm_h16(Ab, Bb, 0, acc64=True), ref, rtol=1e-6, atol=1e-6)
    Ah, Bh = Af.astype(np.float16), Bf.astype(np.float16)
    ref16 = Ah.astype(np.float64) @ Bh.astype(np.float64)
    assert np.allclose(O.gemm_h16(Ah.view(np.uint16), Bh.view(np.uint16), 1, acc64=True), ref16, rtol=1e-6, atol=1e-6)
    # bf16 rounding helper: round to nearest even, checked against the C helper
    L = O.load()
    for v in (1.0, 1.00390625, 1.01171875, -3.14159, 1e-30, 65504.0):
        assert int(O.to_bf16(np.array([v], np.float32))[0]) == int(L.oracle_f32_to_bf16(v))


def test_conv_against_numpy():
    N, CI, CO, KY, KX, OY, OX = 3, 8, 6, 3, 2, 4, 5
    IY, IX = OY + KY - 1, OX + KX - 1
    I2, K2 = O.uniform(1, 1, (IY * IX, CI * N)), O.uniform(1, 2, (CI * KY, CO * KX))
    I4 = I2.reshape(IX, IY, N, CI).astype(np.float64)      # [ix][iy][n][ci]
    K4 = K2.reshape(KY, CI, KX, CO).astype(np.float64)     # [ky][ci][kx][co]
    ref = np.zeros((OX, OY, N, CO))
    for kx in range(KX):
        for ky in range(KY):
            ref += np.einsum("xync,co->xyno", I4[kx:kx + OX, ky:ky + OY], K4[ky, :, kx, :])
    got = O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=True).reshape(OX, OY, N, CO)
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-5)
    assert np.allclose(O.conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, CII=4).reshape(OX, OY, N, CO), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("s", [1, 2])
def test_capsule_against_numpy(s):
    N, NN, CI, CII, CO, KY, KX, OY, OX, M = 2, 2, 8, 4, 4, 3, 3, 3, 4, 4
    IY, IX = s * OY + KY - s, s * OX + KX - s
    P2 = O.uniform(2, 1, (IY * IX * N, CI * M * M * NN))
    W2 = O.uniform(2, 2, (CI * KY * KX * M, CO * M))
    P = P2.reshape(N, IX, IY, NN, M, M, CI).astype(np.float64)              # [n][ix][iy][nn][mx][mk][ci]
    W = W2.reshape(M, CI // CII, KX, KY, CII, M, CO).astype(np.float64)      # [mk][ci_o][kx][ky][cii][my][co]
    ref = np.zeros((N, OX, OY, NN, M, M, CO))                                # [n][ox][oy][nn][mx][my][co]
    for kx in range(KX):
        for ky in range(KY):
            Pw = P[:, kx:kx + s * OX:s, ky:ky + s * OY:s]                    # [n][ox][oy][nn][mx][mk][ci]
            Wk = W[:, :, kx, ky].transpose(0, 1, 2, 3, 4)                    # [mk][ci_o][cii][my][co]
            Wk = Wk.reshape(M, CI, M, CO)                                    # ci = cii + CII*ci_o
            ref += np.einsum("nxyqmkc,kcuo->nxyqmuo", Pw, Wk)
    got = O.capsule_f32(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, M, M, M, s, acc64=True)
    assert np.allclose(got.reshape(N, OX, OY, NN, M, M, CO), ref, rtol=1e-5, atol=1e-5)


def test_tiled_layout_maps_are_permutations():
    C = np.arange(24 * 32, dtype=np.float32).reshape(24, 32)
    t = O.gemm_tile_layout(C, 2, 3, 4, 2)
    assert sorted(t.ravel().tolist()) == sorted(C.ravel().tolist())
    # element (jjj,iii,jj,ii,j,i) of the tiled buffer is C[iii + III*ii + III*II*i, jjj + JJJ*jj + JJJ*JJ*j]
    assert t[1, 2, 1, 3, 2, 1] == C[2 + 3 * 1 + 6 * 1, 1 + 2 * 3 + 8 * 2]
    c = np.arange(8 * 12 * 4, dtype=np.float32).reshape(8, 12, 4)            # [k][j][i]
    t9 = O.ttm_tile_layout(c, 2, 2, 2, 2, 3, 2)
    assert sorted(t9.ravel().tolist()) == sorted(c.ravel().tolist())
