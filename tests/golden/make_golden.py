#!/usr/bin/env python3
"""Generate tests/golden/solid_cpu_golden.npz from the reference's Solid CPU library.

Run where oracle/_ref/libsolid_core_cpu.so exists (built by oracle/build_ref.py from the
reference checkout):

    python tests/golden/make_golden.py

Every entry is "<family>/<op>/<dtype>[/...]/<role>" with small seeded inputs and the outputs the
reference produced, so that the numpy restatement (and the CUDA path) can be checked where the
reference library is absent.  Inputs avoid C undefined behaviour (no out-of-range float->int
casts, no signed overflow, shift counts below the type width).
"""
import sys
import zlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path[:0] = [str(ROOT), str(ROOT / "ocean-tensor-package_b200"), str(ROOT / "tests")]

import util                                                    # noqa: E402
from oracle import ref                                         # noqa: E402
from solid_b200 import dtypes as dt, oplist as ol              # noqa: E402

N = 96
GOLDEN_UNARY = ["negative", "conj", "reciprocal", "bitwise_not", "logical_not", "sqrt", "square", "fabs", "sign",
                "ceil", "floor", "trunc", "round", "isinf", "isnan", "isfinite", "absolute", "exp", "log", "sin"]
GOLDEN_BINARY = [op for op in ol.BINARY_OPS if op != "power"] + ["power"]
GOLDEN_REDUCE = ["any", "all", "nnz", "sum", "prod", "sum_abs", "maximum", "minimum", "maximum_abs", "minimum_abs", "norm2"]


def seed(*parts):
    return zlib.crc32(" ".join(parts).encode())


def main():
    cpu = ref.get()
    cpu.set_threads(1)                                         # sequential accumulation order
    out = {}
    for op in GOLDEN_UNARY:
        for dtype in dt.GROUPS[ol.UNARY_OPS[op]]:
            kind = "positive" if op in ("sqrt", "log") else ("special" if op in ("isinf", "isnan", "isfinite", "sign", "fabs") else "general")
            if op == "exp" and dtype in dt.GROUPS["integer"]:
                kind = "unit"                                   # keeps exp(x) inside every integer type
            x = util.random_values(dtype, N, np.random.default_rng(seed("u", op, dtype)), kind)
            od = "bool" if op.startswith("is") else (dt.elem_type(dtype) if op == "absolute" else dtype)
            y = np.zeros(N, dtype=dt.NUMPY[od])
            cpu.unary(op, dtype, [N], [dt.SIZE[dtype]], x.ctypes.data, [dt.SIZE[od]], y.ctypes.data)
            out["unary/%s/%s/in" % (op, dtype)] = x
            out["unary/%s/%s/out" % (op, dtype)] = y
    for op in GOLDEN_BINARY:
        for dtype in dt.GROUPS[ol.BINARY_OPS[op]]:
            rng = np.random.default_rng(seed("b", op, dtype))
            kind = "small" if (dtype in dt.GROUPS["integer"] and op in ("multiply", "power")) else \
                   ("positive" if op == "power" else "general")
            x = util.random_values(dtype, N, rng, kind)
            if op in ("bitshift_left", "bitshift_right"):
                t2, y = "int8", rng.integers(-3, min(8, 8 * dt.SIZE[dtype]), N).astype(np.int8)
            elif op == "power" and dtype in dt.GROUPS["integer_bool"]:
                t2, y = "int16", rng.integers(-2, 5, N).astype(np.int16)
            else:
                t2, y = dtype, util.random_values(dtype, N, rng, kind)
            od = "bool" if op in ol.COMPARE_OPS else dtype
            z = np.zeros(N, dtype=dt.NUMPY[od])
            cpu.binary(op, dtype, [N], [dt.SIZE[dtype]], x.ctypes.data, [dt.SIZE[t2]], y.ctypes.data, [dt.SIZE[od]], z.ctypes.data)
            out["binary/%s/%s/in1" % (op, dtype)] = x
            out["binary/%s/%s/in2" % (op, dtype)] = y
            out["binary/%s/%s/out" % (op, dtype)] = z
    for src in dt.NAMES:
        for dst in dt.NAMES:
            kind = "positive" if (dst in dt.UINT or dst == "bool") else "general"
            x = util.random_values(src, N, np.random.default_rng(seed("c", src, dst)), kind)
            y = np.zeros(N, dtype=dt.NUMPY[dst]); ys = np.zeros(N, dtype=dt.NUMPY[dst])
            cpu.copy(src, dst, [N], [dt.SIZE[src]], x.ctypes.data, [N], [dt.SIZE[dst]], y.ctypes.data)
            xs = x.copy()                                       # the same values stored with reversed bytes
            cpu.byteswap(src, [N], [dt.SIZE[src]], xs.ctypes.data)
            cpu.copy(src, dst, [N], [dt.SIZE[src]], xs.ctypes.data, [N], [dt.SIZE[dst]], ys.ctypes.data, variant="byteswap_copy")
            out["copy/%s/%s/in" % (src, dst)] = x
            out["copy/%s/%s/out" % (src, dst)] = y
            out["copy/%s/%s/in_swapped" % (src, dst)] = xs
            out["copy/%s/%s/out_swapped_source" % (src, dst)] = ys
    for op in GOLDEN_REDUCE:
        for dtype in dt.NAMES:
            rng = np.random.default_rng(seed("r", op, dtype))
            x = util.random_values(dtype, N, rng, "unit" if op == "prod" and dtype not in dt.GROUPS["integer_bool"] else
                                   ("small" if op == "prod" else "general"))
            if op == "prod" and dtype in dt.GROUPS["integer_bool"]:
                x = (x % 3 + (0 if dtype == "bool" else 1)).astype(dt.NUMPY[dtype])[:20]
            rtype = ol.reduce_result_type(op, dtype)
            n = len(x)
            raw = cpu.reduce_all(op, dtype, [n], [dt.SIZE[dtype]], x.ctypes.data)
            out["reduce/%s/%s/in" % (op, dtype)] = x
            out["reduce/%s/%s/out" % (op, dtype)] = np.frombuffer(raw[: dt.SIZE[rtype]], dtype=dt.NUMPY[rtype]).copy()
    # ranges: offset + i * step in int64 / double (/ complex double) for every element type
    for dtype in dt.NAMES:
        es = dt.SIZE[dtype]
        kinds = [("int64", 7, 3), ("int64", -5, 2), ("double", 0.25, 0.5)]
        if dtype not in dt.UINT and dtype != "bool":
            kinds.append(("double", 100.0, -0.375))             # negative double -> unsigned is undefined in C
        if dtype in dt.COMPLEX:
            kinds.append(("cdouble", 1 - 2j, 0.5 + 0.25j))
        for j, (kind, off, step) in enumerate(kinds):
            buf = np.zeros(N * es, dtype=np.uint8)
            cpu.steps(kind, dtype, [N], [es], buf.ctypes.data, off, step)
            out["steps/%s/%s/%d/param" % (kind, dtype, j)] = np.array([complex(off), complex(step)])
            out["steps/%s/%s/%d/out" % (kind, dtype, j)] = buf
    # integer and boolean matrix products (column-major, padded leading dimensions)
    for dtype in dt.GROUPS["integer_bool"]:
        rng = np.random.default_rng(seed("g", dtype))
        npdt = dt.NUMPY[dtype]
        m, n, k = 7, 5, 9
        for ta in "NT":
            for tb in "NT":
                ra, ca = (m, k) if ta == "N" else (k, m)
                rb, cb = (k, n) if tb == "N" else (n, k)
                lda, ldb, ldc = ra + 2, rb + 1, m + 3
                draw = (lambda cnt: (rng.random(cnt) < 0.4).astype(np.uint8)) if dtype == "bool" else \
                       (lambda cnt: rng.integers(0 if dtype in dt.UINT else -9, 10, cnt).astype(npdt))
                A, B, C0 = draw(lda * ca), draw(ldb * cb), draw(ldc * n)
                alpha, beta = (1, 1) if dtype == "bool" else (3, 2)
                al, be = np.array([alpha]).astype(npdt), np.array([beta]).astype(npdt)
                Cw = C0.copy()
                cpu.gemm(dtype, ta, tb, m, n, k, al.ctypes.data, A.ctypes.data, lda, B.ctypes.data, ldb, be.ctypes.data, Cw.ctypes.data, ldc)
                key = "gemm/%s%s/%s" % (ta, tb, dtype)
                out[key + "/A"], out[key + "/B"], out[key + "/C"], out[key + "/out"] = A, B, C0, Cw
                out[key + "/param"] = np.array([m, n, k, lda, ldb, ldc, alpha, beta], dtype=np.int64)
    path = Path(__file__).resolve().parent / "solid_cpu_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote %s: %d arrays, %.1f KiB" % (path, len(out), path.stat().st_size / 1024))


if __name__ == "__main__":
    main()
