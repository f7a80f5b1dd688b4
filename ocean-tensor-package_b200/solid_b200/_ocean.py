"""ctypes binding of libocean_gpu_b200.so, the Ocean-level dispatch declared in
include/ocean_gpu_b200.h (OcTensorGPU_<op> over plain tensor descriptions).  No fallback:
a missing library is an import error."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import dtypes as dt
from ._lib import Scalar, scalar_from_bytes, get as _solid

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libocean_gpu_b200.so"


class OceanError(RuntimeError):
    """An OcTensorGPU_* function returned -1; the message is OcGPU_errorMessage()."""


class TensorView(C.Structure):
    _fields_ = [("dtype", C.c_int), ("ndims", C.c_int), ("size", C.c_size_t * 8), ("strides", C.c_ssize_t * 8),
                ("data", C.c_void_p), ("device", C.c_int), ("byteswapped", C.c_int),
                ("stream", C.c_void_p), ("event", C.c_void_p)]


class IndexView(C.Structure):
    """OcIndexView: the indexed tensor, the shape of the selection and per dimension NULL or an offset table."""
    _fields_ = [("view", TensorView), ("ndims", C.c_int), ("size", C.c_size_t * 8),
                ("offsets", C.POINTER(TensorView) * 8)]


class ScalarView(C.Structure):
    _fields_ = [("dtype", C.c_int), ("value", Scalar)]


_SPECIAL = {"multiply": "scale", "min": "elemwiseMin", "max": "elemwiseMax", "fmin": "elemwiseFMin",
            "fmax": "elemwiseFMax", "lt": "elemwiseLT", "le": "elemwiseLE", "eq": "elemwiseEQ", "ne": "elemwiseNE",
            "ge": "elemwiseGE", "gt": "elemwiseGT"}
_UPPER = {"nan": "NaN", "inf": "Inf", "lt": "LT", "le": "LE", "gt": "GT", "ge": "GE",
          "gtlt": "GTLT", "gtle": "GTLE", "gelt": "GELT", "gele": "GELE"}


def ocean_name(solid_name: str) -> str:
    """Solid table name -> Ocean function name (bitwise_not -> bitwiseNot, sum_nan -> sumNaN,
    multiply -> scale, lt -> elemwiseLT, axis_norm2_nan -> axisNorm2NaN)."""
    if solid_name in _SPECIAL:
        return _SPECIAL[solid_name]
    parts = solid_name.split("_")
    out = parts[0]
    for p in parts[1:]:
        out += _UPPER.get(p, p[:1].upper() + p[1:])
    return out


class OceanGPU:
    def __init__(self, path=LIB_PATH):
        path = Path(path)
        if not path.exists():
            raise ImportError("%s is missing: build it with ocean-tensor-package_b200/build.py" % path)
        _solid()                                           # the Solid library first (RTLD_GLOBAL)
        self.dll = C.CDLL(str(path))
        self.dll.OcGPU_errorMessage.restype = C.c_char_p

    def _check(self, status, what):
        if status != 0:
            raise OceanError("%s: %s" % (what, (self.dll.OcGPU_errorMessage() or b"").decode(errors="replace")))

    def fn(self, name):
        f = getattr(self.dll, "OcTensorGPU_" + name)
        f.restype = C.c_int
        return f

    def has(self, name):
        return hasattr(self.dll, "OcTensorGPU_" + name)

    def init(self):
        self._check(self.dll.OcInitGPU_B200(), "OcInitGPU_B200")

    @staticmethod
    def view(t, stream: int, event: int = 0) -> TensorView:
        v = TensorView()
        v.dtype, v.ndims = dt.INDEX[t.dtype], len(t.size)
        for i, (s, st) in enumerate(zip(t.size, t.strides)):
            v.size[i], v.strides[i] = s, st
        v.data, v.device, v.byteswapped = t.ptr, t.device_index, int(t.byteswapped)
        v.stream, v.event = stream or None, event or None
        return v

    @staticmethod
    def scalar(raw: bytes, dtype: str) -> ScalarView:
        s = ScalarView()
        s.dtype, s.value = dt.INDEX[dtype], scalar_from_bytes(raw)
        return s

    def result_type(self, solid_name: str, dtype: str) -> str:
        f = self.dll.OcGPU_reductionResultType
        f.restype = C.c_int
        return dt.NAMES[f(solid_name.encode(), dt.INDEX[dtype])]


_instance = None


def get() -> OceanGPU:
    global _instance
    if _instance is None:
        _instance = OceanGPU()
    return _instance
