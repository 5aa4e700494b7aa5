"""The allocation-free MTTKRP entry point, for hosts that may not call cudaMalloc while they
run (fixed memory pools, latency-critical loops, frameworks that own all device memory).
It must give what the regular entry gives. Two calls in a row share the library's built-in
scratch array, so the second one runs over whatever the first left behind; the second problem
is smaller on purpose, leaving stale partial sums beyond its own slabs.

This file sorts last so that a run stopping at the first failure has already run the rest."""
import ctypes

import numpy as np
import pytest

import t2sp_b200
from t2sp_b200 import Buffer
from tests import oracle_lib as O
from tests.util import TOL_FP32, normwise

pytestmark = pytest.mark.gpu


def regular(a, b, c):
    K, I, L = a.shape
    R = b.shape[0]
    d = np.full((R, I), np.nan, np.float32)
    db = Buffer.from_numpy(d)
    rc = t2sp_b200.mttkrp(Buffer.from_numpy(a), Buffer.from_numpy(b), Buffer.from_numpy(c), db)
    assert rc == 0
    return db.keepalive


def no_alloc(lib, a, b, c):
    import torch
    K, I, L = a.shape
    R = b.shape[0]
    ta, tb, tc = (torch.from_numpy(x).cuda() for x in (a, b, c))
    td = torch.full((R, I), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.t2sp_b200_mttkrp_noalloc(ta.data_ptr(), L, L * I, tb.data_ptr(), K, tc.data_ptr(), L, td.data_ptr(), I,
                                      L, I, K, R, None, 1)
    assert rc == 0
    return td.cpu().numpy()


def test_no_alloc_matches_regular_entry_twice(lib):
    for seed, (L, I, K, R) in enumerate([(128, 256, 48, 64), (64, 128, 16, 40)]):
        a, b, c = O.uniform(seed, 1, (K, I, L)), O.uniform(seed, 2, (R, K)), O.uniform(seed, 3, (R, L))
        want = regular(a, b, c)
        got = no_alloc(lib, a, b, c)
        assert not np.isnan(got).any()
        assert normwise(got, want) <= TOL_FP32
        assert normwise(got, O.mttkrp_f32(a, b, c, acc64=True)) <= TOL_FP32


def test_no_alloc_padded_output_pitch(lib):
    """d_stride_r > I: the columns of d are I + 12 elements apart; what lies between them is the caller's."""
    import torch
    L, I, K, R, pad = 96, 200, 17, 40, 12
    a, b, c = O.uniform(6, 1, (K, I, L)), O.uniform(6, 2, (R, K)), O.uniform(6, 3, (R, L))
    ta, tb, tc = (torch.from_numpy(x).cuda() for x in (a, b, c))
    td = torch.full((R, I + pad), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.t2sp_b200_mttkrp_noalloc(ta.data_ptr(), L, L * I, tb.data_ptr(), K, tc.data_ptr(), L, td.data_ptr(), I + pad,
                                      L, I, K, R, None, 1)
    assert rc == 0
    got = td.cpu().numpy()
    assert np.isnan(got[:, I:]).all() and not np.isnan(got[:, :I]).any()
    assert normwise(got[:, :I], O.mttkrp_f32(a, b, c, acc64=True)) <= TOL_FP32


def test_no_alloc_rejects_oversized_problem(lib):
    # one partial slab of 4*I*R bytes beyond the 16 MiB array: refused before anything is launched
    I, R = 40000, 128
    assert 4 * I * R > 16 << 20
    rc = lib.t2sp_b200_mttkrp_noalloc(ctypes.c_void_p(256), 32, 32 * I, ctypes.c_void_p(256), 8, ctypes.c_void_p(256), 32,
                                      ctypes.c_void_p(256), I, 32, I, 8, R, None, 1)
    assert rc == -5  # halide_error_code_buffer_allocation_too_large
