#!/usr/bin/env python3
"""Build the reference's own Solid CPU library as the parity checker.

TEST INFRASTRUCTURE ONLY.  The product (the CUDA library) never links,
imports or calls anything produced here.

The Ocean reference keeps its CPU kernels in ``solid/src/core/cpu`` and its
shared helpers in ``solid/src/base``.  This script compiles those sources
*where they lie* in the reference checkout (nothing is copied into this
repository) with the flags of ``solid/src/core/cpu/CMakeLists.txt:47-61``
(``-O3 -std=c99 -fopenmp -fno-strict-aliasing``; no ``-march=native`` and no
fast-math, so there is no FMA contraction in the checker) and writes
``oracle/_ref/libsolid_core_cpu.so``.  The reference's CMake build is not run:
the two files CMake would generate are produced here instead:

* ``solid_core_cpu.h`` / ``solid_core_cpu.lut.c`` by running the reference's
  ``solid/bin/generate.py`` on ``solid/src/core/cpu/solid_core_cpu.src``;
* ``solid/base/cpu/solid_omp_config.h`` (``#define SOLID_ENABLE_OMP 1``), which
  ``solid/src/base/CMakeLists.txt:65-70`` normally writes.

Usage:  python oracle/build_ref.py [--force] [-j N]
The reference checkout is found through ``$OCEAN_REFERENCE_DIR``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libsolid_core_cpu.so"


def reference_root() -> Path | None:
    """The reference checkout: $OCEAN_REFERENCE_DIR, else a directory named `reference` beside this repository."""
    for cand in (os.environ.get("OCEAN_REFERENCE_DIR"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "solid" / "src" / "core" / "cpu").is_dir():
            return Path(cand)
    return None


def _run(cmd, **kw):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(map(str, cmd)), res.stdout))
    return res.stdout


def build(force: bool = False, jobs: int | None = None, verbose: bool = True) -> Path | None:
    """Return the path of the built library, or None when no reference is present."""
    root = reference_root()
    if root is None:
        return LIB if LIB.exists() else None
    if LIB.exists() and not force:
        return LIB
    solid = root / "solid"
    inc = OUT / "inc"
    obj = OUT / "obj"
    (inc / "solid" / "base" / "cpu").mkdir(parents=True, exist_ok=True)
    obj.mkdir(parents=True, exist_ok=True)
    gen = solid / "bin" / "generate.py"
    src = solid / "src" / "core" / "cpu" / "solid_core_cpu.src"
    _run([sys.executable, str(gen), "-h", str(src), str(inc)])
    _run([sys.executable, str(gen), "-c", str(src), str(obj)])
    (inc / "solid" / "base" / "cpu" / "solid_omp_config.h").write_text(
        "#ifndef __SOLID_OMP_CONFIG_H__\n#define __SOLID_OMP_CONFIG_H__\n"
        "#define SOLID_ENABLE_OMP 1\n#endif\n")
    cflags = ["-O3", "-Wno-variadic-macros", "-fno-strict-aliasing", "-std=c99", "-fopenmp",
              "-fPIC", "-w", "-I%s" % inc, "-I%s" % (solid / "include"), "-I%s" % (solid / "src")]
    sources = sorted((solid / "src" / "base" / "generic").glob("*.c"))
    sources += sorted((solid / "src" / "base" / "cpu").glob("*.c"))
    sources += sorted((solid / "src" / "core" / "cpu").glob("template_*.c"))
    sources += [obj / "solid_core_cpu.lut.c"]
    objects = []

    def compile_one(path: Path) -> Path:
        o = obj / (path.stem + ".o")
        _run(["gcc", *cflags, "-c", str(path), "-o", str(o)])
        return o

    jobs = jobs or os.cpu_count() or 4
    with cf.ThreadPoolExecutor(max_workers=jobs) as pool:
        for o in pool.map(compile_one, sources):
            objects.append(o)
            if verbose:
                print("[oracle/_ref] compiled", o.name, flush=True)
    _run(["gcc", "-shared", "-fopenmp", "-o", str(LIB), *map(str, objects), "-lm"])
    if verbose:
        print("[oracle/_ref] built", LIB, flush=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-j", type=int, default=None)
    a = ap.parse_args()
    lib = build(force=a.force, jobs=a.j)
    if lib is None:
        print("no reference checkout and no prebuilt library")
        sys.exit(1)
