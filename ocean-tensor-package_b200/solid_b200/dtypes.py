"""The fifteen Solid element types: table index, byte size, numpy carrier.

Index order and sizes are the ABI of the function tables
(solid/include/solid/base/generic/dtype.h:23-38, solid/src/core/gpu/template_dtype.cu:21-55).
bool travels as uint8 holding 0/1, half as raw uint16 bits, chalf as two raw
uint16 (real, imag).
"""
from __future__ import annotations

import numpy as np

NAMES = ["bool", "uint8", "uint16", "uint32", "uint64", "int8", "int16", "int32", "int64",
         "half", "float", "double", "chalf", "cfloat", "cdouble"]
INDEX = {n: i for i, n in enumerate(NAMES)}
SIZE = dict(zip(NAMES, [1, 1, 2, 4, 8, 1, 2, 4, 8, 2, 4, 8, 4, 8, 16]))
WORKSIZE = dict(zip(NAMES, [1, 1, 2, 4, 8, 1, 2, 4, 8, 4, 4, 8, 8, 8, 16]))

CHALF_NP = np.dtype([("real", "<u2"), ("imag", "<u2")])
NUMPY = {"bool": np.dtype(np.uint8), "uint8": np.dtype(np.uint8), "uint16": np.dtype(np.uint16),
         "uint32": np.dtype(np.uint32), "uint64": np.dtype(np.uint64), "int8": np.dtype(np.int8),
         "int16": np.dtype(np.int16), "int32": np.dtype(np.int32), "int64": np.dtype(np.int64),
         "half": np.dtype(np.uint16), "float": np.dtype(np.float32), "double": np.dtype(np.float64),
         "chalf": CHALF_NP, "cfloat": np.dtype(np.complex64), "cdouble": np.dtype(np.complex128)}

BOOL = ["bool"]
UINT = ["uint8", "uint16", "uint32", "uint64"]
SINT = ["int8", "int16", "int32", "int64"]
REAL = ["half", "float", "double"]
COMPLEX = ["chalf", "cfloat", "cdouble"]
GROUPS = {
    "bool": BOOL, "uint": UINT, "sint": SINT, "real": REAL, "complex": COMPLEX,
    "integer": UINT + SINT, "float": REAL + COMPLEX, "integer_bool": BOOL + UINT + SINT,
    "all": BOOL + UINT + SINT + REAL + COMPLEX, "all_nobool": UINT + SINT + REAL + COMPLEX,
    "all_nouint": BOOL + SINT + REAL + COMPLEX, "all_nocomplex": BOOL + UINT + SINT + REAL,
}


def is_complex(name: str) -> bool:
    return name in COMPLEX


def elem_type(name: str) -> str:
    """Component type of a complex type (the type itself otherwise)."""
    return {"chalf": "half", "cfloat": "float", "cdouble": "double"}.get(name, name)


def sum_type(name: str) -> str:
    """Result type of sum/prod (reduce_ops.h:607-617)."""
    if name in BOOL or name in UINT:
        return "uint64"
    if name in SINT:
        return "int64"
    return name


def abs_type(name: str) -> str:
    """SDTYPE_ABSTYPE: signed -> unsigned of the same width, complex -> component."""
    if name in SINT:
        return "u" + name
    return elem_type(name)


def norm_type(name: str) -> str:
    """Result type of norm/norm2 (reduce_ops.h:1132-1175,1221-1255)."""
    if name in BOOL or name in UINT or name in SINT:
        return "double"
    return elem_type(name)
