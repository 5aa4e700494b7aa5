"""ctypes mirror of Halide's buffer ABI (Halide/src/runtime/HalideRuntime.h:1338-1420) and
helpers that describe numpy arrays or raw device pointers as halide_buffer_t, with
dimension 0 innermost exactly as Halide::Runtime::Buffer lays tensors out."""
import ctypes

import numpy as np

TYPE_INT, TYPE_UINT, TYPE_FLOAT, TYPE_HANDLE, TYPE_BFLOAT = 0, 1, 2, 3, 4


class HalideType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class HalideDimension(ctypes.Structure):
    _fields_ = [("min", ctypes.c_int32), ("extent", ctypes.c_int32), ("stride", ctypes.c_int32),
                ("flags", ctypes.c_uint32)]


class HalideBuffer(ctypes.Structure):
    _fields_ = [("device", ctypes.c_uint64), ("device_interface", ctypes.c_void_p),
                ("host", ctypes.c_void_p), ("flags", ctypes.c_uint64), ("type", HalideType),
                ("dimensions", ctypes.c_int32), ("dim", ctypes.POINTER(HalideDimension)),
                ("padding", ctypes.c_void_p)]


assert ctypes.sizeof(HalideBuffer) == 56 and ctypes.sizeof(HalideDimension) == 16

DTYPES = {
    "f32": (TYPE_FLOAT, 32), "bf16": (TYPE_BFLOAT, 16), "f16": (TYPE_FLOAT, 16),
    "i8": (TYPE_INT, 8), "i32": (TYPE_INT, 32), "f64": (TYPE_FLOAT, 64),
}
_NP = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int8): "i8",
       np.dtype(np.int32): "i32", np.dtype(np.float64): "f64"}


class Buffer:
    """A halide_buffer_t plus the Python objects that keep its memory alive.

    `extents` are listed innermost first (Halide order). Strides default to dense."""

    def __init__(self, extents, dtype, host=None, device=0, strides=None, mins=None, keepalive=None):
        code, bits = DTYPES[dtype]
        n = len(extents)
        self.dims = (HalideDimension * max(n, 1))()
        stride = 1
        for d, e in enumerate(extents):
            s = strides[d] if strides is not None else stride
            self.dims[d] = HalideDimension(mins[d] if mins else 0, int(e), int(s), 0)
            stride *= int(e)
        self.raw = HalideBuffer()
        self.raw.device = int(device)
        self.raw.device_interface = None
        self.raw.host = host
        self.raw.flags = 0
        self.raw.type = HalideType(code, bits, 1)
        self.raw.dimensions = n
        self.raw.dim = ctypes.cast(self.dims, ctypes.POINTER(HalideDimension))
        self.raw.padding = None
        self.keepalive = keepalive
        self.dtype = dtype
        self.extents = tuple(int(e) for e in extents)

    @property
    def ptr(self):
        return ctypes.byref(self.raw)

    @classmethod
    def from_numpy(cls, arr, dtype=None, extents=None):
        """Wraps a C-contiguous numpy array: numpy's LAST axis is Halide's dimension 0.
        `dtype` overrides the element type for views numpy cannot name (bf16 stored as uint16)."""
        arr = np.ascontiguousarray(arr)
        if dtype is None:
            dtype = _NP[arr.dtype]
        if extents is None:
            extents = tuple(reversed(arr.shape))
        return cls(extents, dtype, host=arr.ctypes.data, keepalive=arr)

    @classmethod
    def query(cls, ndims, dtype="f32"):
        """A bounds-query buffer (host == NULL, device == 0) with room for `ndims` dimensions."""
        return cls([0] * ndims, dtype)

    def shape(self):
        return [(self.dims[d].min, self.dims[d].extent, self.dims[d].stride) for d in range(self.raw.dimensions)]
