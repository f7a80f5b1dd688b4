"""The C-ABI library on a machine without a GPU: it loads, exports every symbol that
include/solid_core_gpu.h declares, its function tables have the entries (and the holes) the
header's type groups say, and argument errors come back as -1 with a message."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from solid_b200 import _lib, dtypes as dt, oplist as ol

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "solid_core_gpu.h"


@pytest.fixture(scope="module")
def declared():
    """Function and table names declared by the header, from the preprocessor output."""
    cuda_inc = "/usr/local/cuda/include"
    out = subprocess.run(["gcc", "-E", "-P", "-I", str(ROOT / "include"), "-I", cuda_inc, str(HEADER)],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert out.returncode == 0, out.stderr[-2000:]
    text = out.stdout
    functions = set(re.findall(r"\bint\s+(solid_gpu_\w+)\s*\(", text))
    functions |= set(re.findall(r"\bvoid\s+(solid_gpu_\w+)\s*\(", text))
    functions |= set(re.findall(r"\bsolid_gpu_properties\s*\*\s*(solid_gpu_\w+)\s*\(", text))
    tables = set(re.findall(r"solid_funptr_gpu_\w+\s+(solid_gpu_\w+)\s*\[", text))
    return functions, tables


def test_library_exports_every_declared_symbol(declared):
    lib = _lib.get()
    functions, tables = declared
    assert len(functions) > 2000 and len(tables) > 120
    missing = sorted(n for n in functions | tables if not lib.has(n))
    assert not missing, "declared but not exported: %s" % missing[:20]
    for name in ("solid_errmsg", "solid_gpu_type_size", "solid_gpu_worktype_size"):
        assert lib.has(name)


def expected_functions():
    names = set()
    families = [ol.FILL_OPS, {"masked_fill": "all", "byteswap": "all", "axpy": "real"}, ol.UNARY_OPS, ol.BINARY_OPS,
                {op + "_scalar": group for op, group in ol.SCALAR_OPS.items()}, ol.STEPS_OPS, ol.GEMM_OPS, ol.INDEX_OPS, {op + "_checked": g for op, g in ol.CHECKED_OPS.items()}, ol.REDUCE_BOOL_OPS, ol.REDUCE_BOUND1_OPS, ol.REDUCE_BOUND2_OPS, ol.REDUCE_U64_OPS,
                ol.REDUCE_VOID_OPS, ol.REDUCE_NORM_OPS, ol.AXIS_OPS, ol.AXIS_NORM_OPS]
    for fam in families:
        for op, group in fam.items():
            for t in dt.GROUPS[group]:
                names.add("solid_gpu_%s_%s" % (op, t))
    for s in dt.NAMES:
        for d in dt.NAMES:
            for v in ("copy", "copy_regular", "byteswap_copy"):
                names.add("solid_gpu_%s_%s_%s" % (v, s, d))
    return names


def test_python_operation_lists_match_the_header(declared):
    functions, _ = declared
    per_type = {f for f in functions if re.search(r"_(%s)$" % "|".join(dt.NAMES), f)}
    per_type -= {"solid_gpu_axpy_sums_float", "solid_gpu_axpy_sums_double", "solid_gpu_axis_sum_float_noalloc",
                 "solid_gpu_peer_sum_float"}
    exp = expected_functions()
    assert per_type - exp == set(), sorted(per_type - exp)[:10]
    assert exp - per_type == set(), sorted(exp - per_type)[:10]


def test_function_tables_have_entries_and_holes():
    lib = _lib.get()
    families = [ol.FILL_OPS, {"masked_fill": "all", "byteswap": "all", "axpy": "real"}, ol.UNARY_OPS, ol.BINARY_OPS,
                {op + "_scalar": group for op, group in ol.SCALAR_OPS.items()}, ol.STEPS_OPS, ol.GEMM_OPS, ol.INDEX_OPS, {op + "_checked": g for op, g in ol.CHECKED_OPS.items()}, ol.REDUCE_BOOL_OPS, ol.REDUCE_BOUND1_OPS, ol.REDUCE_BOUND2_OPS, ol.REDUCE_U64_OPS,
                ol.REDUCE_VOID_OPS, ol.REDUCE_NORM_OPS, ol.AXIS_OPS, ol.AXIS_NORM_OPS]
    for fam in families:
        for op, group in fam.items():
            table = (C.c_void_p * 15).in_dll(lib.dll, "solid_gpu_" + op)
            for i, t in enumerate(dt.NAMES):
                if t in dt.GROUPS[group]:
                    fn = C.cast(getattr(lib.dll, "solid_gpu_%s_%s" % (op, t)), C.c_void_p).value
                    assert table[i] == fn, (op, t)
                else:
                    assert table[i] is None, (op, t)
    for v in ("copy", "copy_regular", "byteswap_copy"):
        table = ((C.c_void_p * 15) * 15).in_dll(lib.dll, "solid_gpu_" + v)
        for i, s in enumerate(dt.NAMES):
            for j, d in enumerate(dt.NAMES):
                fn = C.cast(getattr(lib.dll, "solid_gpu_%s_%s_%s" % (v, s, d)), C.c_void_p).value
                assert table[i][j] == fn, (v, s, d)


def test_type_size_tables():
    lib = _lib.get()
    sizes = (C.c_int * 15).in_dll(lib.dll, "solid_gpu_type_size")
    work = (C.c_int * 15).in_dll(lib.dll, "solid_gpu_worktype_size")
    assert list(sizes) == [dt.SIZE[n] for n in dt.NAMES]
    assert list(work) == [dt.WORKSIZE[n] for n in dt.NAMES]


def test_argument_errors_return_minus_one_with_a_message():
    """Checks that run before any CUDA call: too many dimensions, bad type indices, unknown names."""
    lib = _lib.get()
    nine = [2] * 9
    with pytest.raises(_lib.SolidError, match="dimensions"):
        lib.unary("sqrt", "float", nine, [4] * 9, 256, [4] * 9, 512)
    with pytest.raises(_lib.SolidError, match="dimensions"):
        lib.binary("add", "int32", nine, [4] * 9, 256, [4] * 9, 256, [4] * 9, 512)
    with pytest.raises(_lib.SolidError, match="type index"):
        lib.fn("solid_gpu_copy_ex")(C.c_int(99), C.c_int(0), C.c_int(0), C.c_int(0), None, None, None,
                                     C.c_int(0), None, None, None, None) and None
        lib._check(-1, "copy_ex")
    with pytest.raises(_lib.SolidError, match="Unknown reduction"):
        lib.reduce_all_device("median", "float", [4], [4], 256, 512, 1024)
    with pytest.raises(_lib.SolidError, match="scratch buffer"):
        lib.reduce_all("sum", "float", [4], [4], 256, 0)


def test_layout_and_ops_host_logic():
    """Type promotion and view arithmetic of the host layer (no device needed)."""
    from solid_b200 import ops
    assert ops.common_type("double", "int32") == "double"
    assert ops.common_type("int8", "uint8") == "int16"
    assert ops.common_type("uint32", "int32") == "int64"
    assert ops.common_type("float", "cdouble") == "cdouble"
    assert ops.common_type("bool", "half") == "half"
    assert ops.common_type("chalf", "float") == "cfloat"
    assert ops.scalar_bytes(1.5, "half") == bytes([0x00, 0x3E])
    assert ops.scalar_bytes(2.0 ** 17, "half") == bytes([0x00, 0x7C])             # exponent >= 144 -> inf
    assert ops.scalar_bytes(2.0 ** -16, "half") == bytes([0x00, 0x00])           # below 2^-15 -> +0
    assert ops.scalar_bytes(-3, "int16") == (-3).to_bytes(2, "little", signed=True)
    assert ol.reduce_result_type("sum", "int8") == "int64"
    assert ol.reduce_result_type("axis_maximum_abs", "int16") == "uint16"
    assert ol.reduce_result_type("norm2", "cfloat") == "float"
    assert ol.reduce_result_type("sum_abs", "cdouble") == "double"
