#!/usr/bin/env python3
"""Build libsolid_core_gpu.so for sm_100a with nvcc (no GPU needed to compile).

Every per-type unit of csrc/ is compiled once per element type with
-DSDX=<type> -DSDX_KIND=<kind>; objects land in build/ and are rebuilt only when
a source, a header or the command line changed.  The library is written to
lib/libsolid_core_gpu.so next to this file.

    python ocean-tensor-package_b200/build.py [-j N] [--force] [--types float,double]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
BUILD = HERE / "build"
LIBDIR = HERE / "lib"
LIB = LIBDIR / "libsolid_core_gpu.so"
OCEAN_LIB = LIBDIR / "libocean_gpu_b200.so"        # Ocean-level dispatch on top of the Solid tables

# name -> kind (0 bool, 1 unsigned, 2 signed, 3 real floating point, 4 complex)
TYPES = {"bool": 0, "uint8": 1, "uint16": 1, "uint32": 1, "uint64": 1,
         "int8": 2, "int16": 2, "int32": 2, "int64": 2,
         "half": 3, "float": 3, "double": 3, "chalf": 4, "cfloat": 4, "cdouble": 4}
PER_TYPE_UNITS = ["reduce", "copy", "unary", "binary", "fill", "steps"]     # slowest first
SINGLE_UNITS = ["base", "luts", "reduce_plan", "fused", "noalloc", "index", "gemm", "peer"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--fmad=false",            # one rounding per operation, as the CPU oracle computes
              "-Xfatbin", "-compress-all",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",   # exports are narrowed at link time
              "-I%s" % INCLUDE, "-I%s" % CSRC]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stamp() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _jobs(types):
    jobs = []
    for unit in PER_TYPE_UNITS:
        for t in types:
            jobs.append((CSRC / (unit + ".cu"), BUILD / ("%s_%s.o" % (unit, t)),
                         ["-DSDX=%s" % t, "-DSDX_KIND=%d" % TYPES[t]]))
    for unit in SINGLE_UNITS:
        jobs.append((CSRC / (unit + ".cu"), BUILD / (unit + ".o"), []))
    return jobs


def _compile(job, stamp, force):
    src, obj, defs = job
    key = hashlib.sha256((stamp + src.read_text() + " ".join(defs)).encode()).hexdigest()
    keyfile = obj.with_suffix(".key")
    if not force and obj.exists() and keyfile.exists() and keyfile.read_text() == key:
        return obj, 0.0, False
    t0 = time.time()
    cmd = [nvcc(), *NVCC_FLAGS, *defs, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s %s:\n%s" % (src.name, " ".join(defs), res.stdout))
    keyfile.write_text(key)
    return obj, time.time() - t0, True


def build(jobs_n: int | None = None, force: bool = False, types=None, verbose: bool = True) -> Path:
    types = list(types or TYPES)
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    stamp = _stamp()
    jobs = _jobs(types)
    objects, rebuilt = [], False
    with cf.ThreadPoolExecutor(max_workers=jobs_n or os.cpu_count() or 4) as pool:
        futs = [pool.submit(_compile, j, stamp, force) for j in jobs]
        for f in futs:
            obj, secs, did = f.result()
            objects.append(obj)
            rebuilt |= did
            if did and verbose:
                print("[build] %-28s %6.1fs" % (obj.name, secs), flush=True)
    if rebuilt or not LIB.exists() or set(types) != set(TYPES):
        # only the C-ABI is exported (csrc/solid_exports.map); template instantiations stay local
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objects), "-lcudart",
               "-Xlinker", "--version-script=%s" % (CSRC / "solid_exports.map")]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout)
        if verbose:
            print("[build] linked", LIB, flush=True)
    # the dispatch layer is host code only; it links against the Solid library beside it
    obj, secs, did = _compile((CSRC / "ocean_gpu.cu", BUILD / "ocean_gpu.o", []), stamp, force)
    if did or rebuilt or not OCEAN_LIB.exists():
        cmd = [nvcc(), "-shared", "-o", str(OCEAN_LIB), str(obj), "-L%s" % LIBDIR, "-lsolid_core_gpu",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lcudart",
               "-Xlinker", "--version-script=%s" % (CSRC / "ocean_exports.map")]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout)
        if verbose:
            print("[build] linked", OCEAN_LIB, flush=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--types", default=None, help="comma separated subset (the library then lacks the others)")
    a = ap.parse_args()
    build(a.j, a.force, a.types.split(",") if a.types else None)
