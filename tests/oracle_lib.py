"""ctypes access to the CPU oracle (oracle/oracle.cpp) plus seeded input generators.
Test infrastructure: only tests, smoke() and the bench's CPU-baseline legs import this."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_ref", "liboracle.so")

_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    src = os.path.join(ORACLE_DIR, "oracle.cpp")
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
    L = ctypes.CDLL(ORACLE_SO)
    L.oracle_max_rel_err.restype = ctypes.c_double
    L.oracle_max_abs.restype = ctypes.c_double
    L.oracle_f32_to_bf16.restype = ctypes.c_uint16
    L.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
    _lib = L
    return L


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def rng(seed, tensor_id=0):
    """Counter-based generator keyed by (seed, tensor id): any shard can be regenerated alone."""
    return np.random.Generator(np.random.Philox(key=[seed, tensor_id]))


def uniform(seed, tid, shape):
    return rng(seed, tid).uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal(seed, tid, shape, sigma):
    return (rng(seed, tid).standard_normal(size=shape) * sigma).astype(np.float32)


def int8(seed, tid, shape):
    return rng(seed, tid).integers(-127, 128, size=shape, dtype=np.int8)


def to_bf16(x):
    """fp32 -> bf16 bits (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(h):
    return (h.astype(np.uint32) << 16).view(np.float32)


# ---- oracle calls; numpy arrays are C-contiguous with the LAST axis = Halide dimension 0
def gemm_f32(A, B, acc64=False):
    """A: (M,K), B: (K,N) -> C: (M,N)."""
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), np.float32)
    load().oracle_gemm_f32(_p(A), _p(B), _p(C), M, N, K, int(acc64))
    return C


def gemm_h16(A, B, kind, acc64=False):
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), np.float32)
    load().oracle_gemm_h16(_p(A), _p(B), _p(C), M, N, K, int(kind), int(acc64))
    return C


def gemm_i8(A, B):
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), np.int32)
    load().oracle_gemm_i8(_p(A), _p(B), _p(C), M, N, K)
    return C


def gemm_tile_layout(C, JJJ, III, JJ, II):
    M, N = C.shape
    J, I = N // (JJJ * JJ), M // (III * II)
    out = np.empty((I, J, II, JJ, III, JJJ), np.float32)
    load().oracle_gemm_tile_layout(_p(np.ascontiguousarray(C)), _p(out), JJJ, III, JJ, II, J, I)
    return out


def conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, CII=0, acc64=False):
    """I2: (IY*IX, CI*N), K2: (CI*KY, CO*KX) -> O2: (OY*OX, CO*N)."""
    O2 = np.empty((OY * OX, CO * N), np.float32)
    load().oracle_conv_f32(_p(I2), _p(K2), _p(O2), N, CI, CO, KY, KX, OY, OX, CII, int(acc64))
    return O2


def conv_tile_layout(O2, N, COOO, YYY, XXX, COO, YY, XX, Y, X, COout):
    out = np.empty((N, COout, X, Y, XX, YY, COO, XXX, YYY, COOO), np.float32)
    load().oracle_conv_tile_layout(_p(np.ascontiguousarray(O2)), _p(out), N, COOO, YYY, XXX, COO, YY, XX, Y, X, COout)
    return out


def capsule_f32(P2, W2, N, NN, CI, CII, CO, KY, KX, OY, OX, MY, MX, MK, s, acc64=False):
    V2 = np.empty((OY * OX * N, CO * MY * MX * NN), np.float32)
    load().oracle_capsule_f32(_p(P2), _p(W2), _p(V2), N, NN, CI, CII, CO, KY, KX, OY, OX, MY, MX, MK, s, int(acc64))
    return V2


def capsule_tile_layout(V2, N, NN, COOO, COO, COout, YYY_XXX, YY_XX, Y_X, MY, MX, OY, OX):
    out = np.empty((N, COout, NN, COO, MX, MY, Y_X, YY_XX, YYY_XXX, COOO), np.float32)
    load().oracle_capsule_tile_layout(_p(np.ascontiguousarray(V2)), _p(out), N, NN, COOO, COO, COout, YYY_XXX, YY_XX,
                                      Y_X, MY, MX, OY, OX)
    return out


def syrk_f32(A, C, III, II, I, alpha, beta, acc64=False):
    """A: (N,K), C: (N,N) -> folded O: (I, I+1, II, II, III, III) (rows i >= I/2 stay NaN: the design
    does not write them)."""
    N, K = A.shape
    Ofold = np.full((I, I + 1, II, II, III, III), np.nan, np.float32)
    L = load()
    L.oracle_syrk_f32.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 6 + [ctypes.c_float] * 2 + [ctypes.c_int]
    L.oracle_syrk_f32(_p(A), _p(C), _p(Ofold), K, III, II, I, I, C.shape[1], alpha, beta, int(acc64))
    return Ofold


def ger_f32(A, X, Y, KKK, III, II, KK, K, I):
    """A: (TI, TK), X: (TI,), Y: (TK,) -> tiled O: (I, K, KK, II, III, KKK)."""
    out = np.empty((I, K, KK, II, III, KKK), np.float32)
    L = load()
    L.oracle_ger_f32.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 7
    L.oracle_ger_f32(_p(A), _p(X), _p(Y), _p(out), KKK, III, II, KK, K, I, A.shape[1])
    return out


def conv_nd_f32(I4, K4, tiles, acc64=False):
    """I4: (N,CI,IX,IY), K4: (CO,CI,KX,KY) -> the 10-D tiled output of the oneAPI flow."""
    N, CI, IX, IY = I4.shape
    CO, _, KX, KY = K4.shape
    COOO, YYY, XXX, COO, YY, XX, Y, X = tiles
    OY, OX = IY - KY + 1, IX - KX + 1
    I2 = np.empty((IY * IX, CI * N), np.float32)
    K2 = np.empty((CI * KY, CO * KX), np.float32)
    load().oracle_conv_nd_to_2d(_p(I4), _p(K4), _p(I2), _p(K2), N, CI, CO, KY, KX, IY, IX)
    return conv_tile_layout(conv_f32(I2, K2, N, CI, CO, KY, KX, OY, OX, acc64=acc64), N, COOO, YYY, XXX, COO, YY, XX, Y, X,
                            CO // (COOO * COO))


def capsule_nd_f32(P6, W6, vt, s, acc64=False):
    """P6: (N,IX,IY,CI,MX,MK), W6: (KX,KY,CO,CI,MK,MY) -> the 9-D tiled output of the oneAPI flow."""
    N, IX, IY, CI, MX, MK = P6.shape
    KX, KY, CO, _, _, MY = W6.shape
    COOO, YYY_XXX, YY_XX, Y_X, COO = vt
    OY, OX = (IY - KY + s) // s, (IX - KX + s) // s
    P2 = np.empty((IY * IX * N, CI * MK * MX), np.float32)
    W2 = np.empty((CI * KY * KX * MK, CO * MY), np.float32)
    load().oracle_capsule_nd_to_2d(_p(P6), _p(W6), _p(P2), _p(W2), N, CI, CO, KY, KX, IY, IX, MY, MX, MK)
    V2 = capsule_f32(P2, W2, N, 1, CI, CI, CO, KY, KX, OY, OX, MY, MX, MK, s, acc64=acc64)
    V10 = capsule_tile_layout(V2, N, 1, COOO, COO, CO // (COOO * COO), YYY_XXX, YY_XX, Y_X, MY, MX, OY, OX)
    return V10.reshape(N, CO // (COOO * COO), COO, MX, MY, Y_X, YY_XX, YYY_XXX, COOO)  # the unit NN axis dropped


def ttm_f32(a, b, acc64=False):
    """a: (J,I,L), b: (K,L) -> c: (K,J,I)."""
    J, I, L = a.shape
    K = b.shape[0]
    c = np.empty((K, J, I), np.float32)
    load().oracle_ttm_f32(_p(a), _p(b), _p(c), L, I, J, K, int(acc64))
    return c


def ttm_tile_layout(c, JJ, KK, II, KKK, JJJ, III):
    K, J, I = c.shape
    OK, OJ, OI = K // (KKK * KK), J // (JJJ * JJ), I // (III * II)
    out = np.empty((OI, OJ, OK, III, JJJ, KKK, II, KK, JJ), np.float32)
    load().oracle_ttm_tile_layout(_p(np.ascontiguousarray(c)), _p(out), JJ, KK, II, KKK, JJJ, III, OK, OJ, OI)
    return out


def mttkrp_f32(a, b, c, acc64=False):
    """a: (K,I,L), b: (R,K), c: (R,L) -> d: (R,I)."""
    K, I, L = a.shape
    R = b.shape[0]
    d = np.empty((R, I), np.float32)
    load().oracle_mttkrp_f32(_p(a), _p(b), _p(c), _p(d), L, I, K, R, int(acc64))
    return d


def rel_err(got, ref, floor_abs=0.0):
    """max |got-ref| / max(|ref|, floor_abs)."""
    got = np.ascontiguousarray(got, np.float32)
    ref = np.ascontiguousarray(ref, np.float32)
    return float(load().oracle_max_rel_err(_p(got), _p(ref), ctypes.c_size_t(got.size), ctypes.c_double(floor_abs)))
