"""B200-native replacement for the host interface and device kernels that T2SP generates for
its dense-tensor workloads (GEMM, 2-D convolution, capsule convolution, TTM, MTTKRP).

The product is the C ABI in include/t2sp_b200/runtime.h, served by libt2sp_b200.so (CUDA,
sm_100a). This package only loads that library and mirrors its entry points for Python
callers; there is no CPU path, and importing the library raises if it has not been built."""
import ctypes
import os

from . import halide
from .halide import Buffer

_HERE = os.path.dirname(os.path.abspath(__file__))
# $T2SP_B200_LIBRARY selects another build of the same library (e.g. an instrumented one).
LIB_PATH = os.environ.get("T2SP_B200_LIBRARY") or os.path.join(_HERE, "libt2sp_b200.so")
_lib = None


class GemmDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("layout", "JJJ", "III", "JJ", "II", "precision", "trans_b", "trans_a",
                                               "scale")] + [("alpha", ctypes.c_float), ("beta", ctypes.c_float)]


class ConvDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "layout", "CI", "CO", "KY", "KX", "OY", "OX", "COOO", "YYY", "XXX", "COO", "YY", "XX", "Y", "X", "precision")]


class CapsuleDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "layout", "CI", "CII", "CO", "KY", "KX", "OY", "OX", "MY", "MX", "MK", "NN", "stride",
        "COOO", "YYY_XXX", "YY_XX", "Y_X", "COO", "precision")]


class TtmDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("layout", "precision")]


class MttkrpDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("precision", "splits")]


ERROR_NAMES = {
    0: "success", -1: "generic_error", -3: "bad_type", -4: "access_out_of_bounds",
    -5: "buffer_allocation_too_large", -6: "buffer_extents_too_large", -8: "constraint_violated",
    -11: "out_of_memory", -12: "buffer_argument_is_null", -14: "copy_to_host_failed",
    -15: "copy_to_device_failed", -16: "device_malloc_failed", -17: "device_sync_failed",
    -23: "device_run_failed", -28: "buffer_extents_negative", -32: "device_wrap_native_failed",
    -34: "host_is_null", -36: "device_interface_no_device", -43: "bad_dimensions",
}


def lib():
    """The loaded C-ABI library. Raises if libt2sp_b200.so is missing: nothing falls back."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libt2sp_b200.so is not built (run `python -m t2sp_b200.build`); "
                "t2sp_b200 has no CPU or PyTorch fallback")
        L = ctypes.CDLL(LIB_PATH)
        P = ctypes.c_void_p
        for name, nargs in (("t2sp_b200_gemm", 4), ("t2sp_b200_conv", 4), ("t2sp_b200_capsule", 4),
                            ("t2sp_b200_ttm", 4), ("t2sp_b200_mttkrp", 5)):
            fn = getattr(L, name)
            fn.argtypes = [P] * nargs
            fn.restype = ctypes.c_int
        L.t2sp_b200_syrk.argtypes = [ctypes.c_int32, ctypes.c_float, ctypes.c_float, P, P, P]
        L.t2sp_b200_syrk.restype = ctypes.c_int
        L.t2sp_b200_ger.argtypes = [P, P, P, P]
        L.t2sp_b200_ger.restype = ctypes.c_int
        for name in ("t2sp_b200_conv_nd", "t2sp_b200_capsule_nd"):
            getattr(L, name).argtypes = [P, P, P, ctypes.c_int]
            getattr(L, name).restype = ctypes.c_int
        for name in ("t2sp_b200_device_malloc", "t2sp_b200_device_free", "t2sp_b200_copy_to_device",
                     "t2sp_b200_copy_to_host", "t2sp_b200_detach_device_ptr"):
            getattr(L, name).argtypes = [P]
            getattr(L, name).restype = ctypes.c_int
        L.t2sp_b200_sgemm.argtypes = [ctypes.c_char, ctypes.c_char, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                      P, ctypes.c_int, P, ctypes.c_int, ctypes.c_float, P, ctypes.c_int]
        L.t2sp_b200_sgemm.restype = ctypes.c_int
        i64, i32 = ctypes.c_int64, ctypes.c_int32
        L.t2sp_b200_mttkrp_noalloc.argtypes = [P, i64, i64, P, i64, P, i64, P, i64, i32, i32, i32, i32, P, i32]
        L.t2sp_b200_mttkrp_noalloc.restype = ctypes.c_int
        L.t2sp_b200_wrap_device_ptr.argtypes = [P, ctypes.c_uint64]
        L.t2sp_b200_wrap_device_ptr.restype = ctypes.c_int
        L.t2sp_b200_device_interface.restype = P
        L.t2sp_b200_set_device.argtypes = [ctypes.c_int]
        L.t2sp_b200_set_stream.argtypes = [P]
        L.t2sp_b200_set_async.argtypes = [ctypes.c_int]
        L.t2sp_b200_sync.restype = ctypes.c_int
        L.t2sp_b200_kernel_launches.restype = ctypes.c_uint64
        L.t2sp_b200_last_kernel_ns.restype = ctypes.c_double
        L.t2sp_b200_version.restype = ctypes.c_char_p
        L.t2sp_b200_device_info.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        _lib = L
    return _lib


def _opt(desc):
    return ctypes.byref(desc) if desc is not None else None


def gemm(A, B, C, desc=None):
    """int gemm(A, B, C): C = A x B. Mirrors the generated `gemm(halide_buffer_t*...)`
    (t2s/tests/performance/gemm/gemm.cpp:95). Returns the halide error code (0 = success)."""
    return lib().t2sp_b200_gemm(A.ptr, B.ptr, C.ptr, _opt(desc))


def conv(I, K, O, desc):
    """int conv(I, K, O) (t2s/tests/performance/conv/conv.cpp:101)."""
    return lib().t2sp_b200_conv(I.ptr, K.ptr, O.ptr, _opt(desc))


def capsule(P, W, V, desc):
    """int capsule(P, W, V) (t2s/tests/performance/capsule/capsule.cpp:104)."""
    return lib().t2sp_b200_capsule(P.ptr, W.ptr, V.ptr, _opt(desc))


def conv_nd(I, K, O, precision=0):
    """conv on the oneAPI flow's N-D operands I(IY,IX,CI,N), K(KY,KX,CI,CO), 10-D O
    (t2s/tests/correctness/oneapi-integration/oneapi-target-5-conv.cpp:58-62)."""
    return lib().t2sp_b200_conv_nd(I.ptr, K.ptr, O.ptr, precision)


def capsule_nd(P, W, V, precision=0):
    """capsule on the oneAPI flow's N-D operands P(MK,MX,CI,IY,IX,N), W(MY,MK,CI,CO,KY,KX), 9-D V
    (t2s/tests/correctness/oneapi-integration/oneapi-target-6-capsule.cpp:57-61)."""
    return lib().t2sp_b200_capsule_nd(P.ptr, W.ptr, V.ptr, precision)


def ger(A, X, Y, O):
    """int ger(A, X, Y, deserializer): the tiled 6-D output of the GER design
    (t2s/tests/performance/ger/ger.cpp:34-62, ger-run-fpga.cpp:66)."""
    return lib().t2sp_b200_ger(A.ptr, X.ptr, Y.ptr, O.ptr)


def syrk(opa, alpha, beta, A, C, O):
    """int syrk(OpA, Alpha, Beta, A, C, deserializer): the folded 6-D output of the SYRK design
    (t2s/peppers/blas/level3/syrk/release/s10/syrk-interface.h:12, t2s/tests/performance/syrk/syrk.cpp:52-73)."""
    return lib().t2sp_b200_syrk(opa, alpha, beta, A.ptr, C.ptr, O.ptr)


def ttm(a, b, c, desc=None):
    """c(i,j,k) = sum_l a(l,i,j) b(l,k) (t2s/tests/correctness/buffer/tmm_small.cpp:60-64)."""
    return lib().t2sp_b200_ttm(a.ptr, b.ptr, c.ptr, _opt(desc))


def mttkrp(a, b, c, d, desc=None):
    """d(i,r) = sum_k (sum_l a(l,i,k) c(l,r)) b(k,r) (t2s/tests/correctness/util/util.h:464-481)."""
    return lib().t2sp_b200_mttkrp(a.ptr, b.ptr, c.ptr, d.ptr, _opt(desc))


def wrap_device(buf, device_ptr):
    """Marks `buf` as resident at CUDA device address `device_ptr` (no copy is made)."""
    return lib().t2sp_b200_wrap_device_ptr(buf.ptr, ctypes.c_uint64(int(device_ptr)))
