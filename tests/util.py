"""Shared helpers for the parity tests: the error metric and C-ABI call wrappers."""
import contextlib
import os

import numpy as np

import t2sp_b200
from t2sp_b200 import Buffer
from tests import oracle_lib as O

# Tolerances. "Max relative error" for a contraction with inputs of mixed sign is taken in the
# two standard forms of rounding-error analysis, because an elementwise |got-ref|/|ref| is
# unbounded wherever the exact sum cancels to ~0 (two correct fp32 summation orders already
# differ by more than 1e-5 there):
#   normwise       max_ij |got - truth|_ij / max_ij |truth|_ij                      <= tol
#   componentwise  max_ij |got - truth|_ij / (sum_k |a_ik| |b_kj|)                  <= tol
# with `truth` the fp64-accumulated oracle. On non-negative inputs (what the reference's own
# drivers use) the two collapse into the strict elementwise relative error, tested as such.
TOL_FP32 = 1e-5
TOL_BF16 = 1e-2


def normwise(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-300))


def componentwise(got, ref, absprod):
    """absprod_ij = sum_k |a_ik||b_kj| (the oracle run on |A|, |B|)."""
    num = np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64))
    den = np.maximum(np.asarray(absprod, np.float64), 1e-300)
    return float(np.max(num / den))


def call_gemm(A, B, dtype_in, out_dtype=np.float32, tiled=None):
    """A: (M,K) array, B: (K,N) array (bf16 as uint16 bits). Returns (rc, C)."""
    M, K = A.shape
    N = B.shape[1]
    a = Buffer.from_numpy(A, dtype=dtype_in)
    b = Buffer.from_numpy(B, dtype=dtype_in)
    if tiled is None:
        C = np.full((M, N), np.nan if out_dtype == np.float32 else -1, dtype=out_dtype)
        c = Buffer.from_numpy(C)
        rc = t2sp_b200.gemm(a, b, c)
    else:
        JJJ, III, JJ, II = tiled
        C = np.full((M // (III * II), N // (JJJ * JJ), II, JJ, III, JJJ), np.nan, dtype=out_dtype)
        c = Buffer.from_numpy(C)
        rc = t2sp_b200.gemm(a, b, c)
    return rc, c.keepalive


@contextlib.contextmanager
def library_env(**values):
    """Sets T2SP_B200_* variables for the duration of a block. The library reads its environment
    once, so it is told to read it again on the way in and on the way out."""
    L = t2sp_b200.lib()
    L.t2sp_b200_reload_env.restype = None
    old = {k: os.environ.get(k) for k in values}
    try:
        for k, v in values.items():
            os.environ[k] = str(v)
        L.t2sp_b200_reload_env()
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        L.t2sp_b200_reload_env()
