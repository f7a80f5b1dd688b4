#!/usr/bin/env python3
"""Build the reference's UNCHANGED Ocean tensor library, its GPU module and its Python
binding on top of this repository's libsolid_core_gpu.so.

TEST INFRASTRUCTURE.  Nothing here is part of the product: the outputs show that the C-ABI
library is a drop-in for the reference's own callers, and let the reference's golden
scripts (examples/python/gpu/{tensors,index}/*.py with their .ref files) run on it.

Sources are compiled where they lie in the reference checkout ($OCEAN_REFERENCE_DIR, or a directory
`reference` beside this repository); only
outputs are written, all below oracle/_ref/ocean/ (git-ignored):

    lib/libocean_base.so   src/base/*.c
    lib/libocean_solid.so  src/external/ocean-solid/ocean_solid.c
    lib/libocean_blas.so   src/external/ocean-blas/ocean_custom_blas.c
    lib/libocean.so        src/core/{interface,generic,cpu,cpu/op}/*.c     (links oracle/_ref/libsolid_core_cpu.so)
    lib/libocean_gpu.so    src/core/gpu/*.c src/core/gpu/op/*.c            (links THIS repo's libsolid_core_gpu.so,
                                                                            compiled against THIS repo's include/solid_core_gpu.h)
    lib_b200/libocean_gpu.so  the same module with the six dispatch files of the hot path
                              (src/core/gpu/op/tensor_{unary,binary,copy,fill,reduce_all,reduce_axis}_gpu.c) replaced by
                              this repository's ocean-tensor-package_b200/csrc/ocean_module.c, which binds
                              libocean_gpu_b200.so into the OcModuleCore table; put lib_b200 first on LD_LIBRARY_PATH to
                              run the Python binding on it
    python/pyOcean_cpu_v<X>_<Y>.so, python/pyOcean_gpu_v<X>_<Y>.so         interfaces/python/pyOcean/{cpu,gpu}/*.c
    python/pyOceanNumpy_v<X>_<Y>.so                                       interfaces/python/pyOceanNumpy/pyOceanNumpy.c
    python/ocean.py, pyOcean_cpu.py, pyOcean_gpu.py                        loaders (the reference's own use the `imp`
                                                                            module, which Python 3.12 no longer has)
    examples/gpu/{tensors,index}/*.py, *.ref                               the golden scripts, staged so that they
                                                                            travel to a GPU machine without the checkout

The reference's CMake build is not run (its find_package(CUDA) and generated-config steps do not work here); the
compile flags are those of src/core/CMakeLists.txt:65-66.

    python oracle/build_ocean.py [--force] [-j N]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "_ref" / "ocean"
SOLID_CPU_DIR = HERE / "_ref"
GPU_LIBDIR = ROOT / "ocean-tensor-package_b200" / "lib"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

CFLAGS = ["-O2", "-std=gnu99", "-fPIC", "-fopenmp", "-fno-strict-aliasing", "-w",
          "-Wno-implicit-function-declaration"]


def reference_dir() -> Path | None:
    """The reference checkout: $OCEAN_REFERENCE_DIR, else a directory named `reference` beside this repository."""
    for cand in (os.environ.get("OCEAN_REFERENCE_DIR"), ROOT.parent / "reference"):
        if cand and (Path(cand) / "src" / "core" / "gpu").is_dir():
            return Path(cand)
    return None


def _run(cmd):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("%s\n%s" % (" ".join(map(str, cmd)), res.stdout[-4000:]))


def _compile_all(sources, objdir: Path, flags, jobs):
    objdir.mkdir(parents=True, exist_ok=True)
    objs = []

    def one(src):
        obj = objdir / (hashlib.md5(str(src).encode()).hexdigest()[:8] + "_" + src.stem + ".o")
        key = obj.with_suffix(".key")
        stamp = hashlib.sha256((src.read_text(errors="replace") + " ".join(flags)).encode()).hexdigest()
        if not (obj.exists() and key.exists() and key.read_text() == stamp):
            _run(["gcc", *flags, "-c", str(src), "-o", str(obj)])
            key.write_text(stamp)
        return obj

    with cf.ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(one, sources))
    return objs


def _link(objs, lib: Path, extra):
    lib.parent.mkdir(parents=True, exist_ok=True)
    _run(["gcc", "-shared", "-fopenmp", "-o", str(lib), *map(str, objs), *extra, "-lm"])


LOADER_OCEAN = '''"""Loader of the Ocean Python binding built by oracle/build_ocean.py (stands in for the reference's
interfaces/python/lib/ocean.py, which relies on the removed `imp` module)."""
from pyOcean_cpu import *          # noqa: F401,F403
try:
    from pyOcean_gpu import *      # noqa: F401,F403
except ImportError:
    gpu = []
'''

LOADER_CPU = '''import sys as _sys
_m = __import__("pyOcean_cpu_v%d_%d" % _sys.version_info[:2], fromlist="*")
globals().update({k: v for k, v in _m.__dict__.items()})
_m.setDefaultDevice(_m.cpu)
_m.setDefaultDType(_m.float)
del _m, _sys
'''

LOADER_GPU = '''import sys as _sys
_m = __import__("pyOcean_gpu_v%d_%d" % _sys.version_info[:2], fromlist="*")
globals().update({k: v for k, v in _m.__dict__.items()})
del _m, _sys
'''


def build(force: bool = False, jobs: int | None = None, verbose: bool = True):
    ref = reference_dir()
    if ref is None:
        if verbose:
            print("[build_ocean] no reference checkout ($OCEAN_REFERENCE_DIR): keeping what is in", OUT)
        return None
    if not (SOLID_CPU_DIR / "libsolid_core_cpu.so").exists():
        raise RuntimeError("run oracle/build_ref.py first (the Ocean CPU module links the Solid CPU library)")
    if not (GPU_LIBDIR / "libsolid_core_gpu.so").exists():
        raise RuntimeError("build ocean-tensor-package_b200/lib/libsolid_core_gpu.so first")
    jobs = jobs or os.cpu_count() or 4
    if force and OUT.exists():
        shutil.rmtree(OUT)
    lib, obj, py = OUT / "lib", OUT / "obj", OUT / "python"
    for d in (lib, obj, py):
        d.mkdir(parents=True, exist_ok=True)
    cfg = obj / "config"
    cfg.mkdir(exist_ok=True)
    (cfg / "ocean_blas_config.h").write_text(
        "#ifndef __OCEAN_EXTERNAL_OCBLAS_CONFIG_H__\n#define __OCEAN_EXTERNAL_OCBLAS_CONFIG_H__\n#endif\n")

    inc_ocean = ["-I%s" % (ref / "include")]
    inc_solid = ["-I%s" % (ref / "solid" / "include"), "-I%s" % (SOLID_CPU_DIR / "inc")]   # inc: generated CPU header, omp config
    rpath = ["-Wl,-rpath,$ORIGIN", "-L%s" % lib]

    def say(msg):
        if verbose:
            print("[build_ocean]", msg, flush=True)

    # ---- base, glue, blas --------------------------------------------------------------------------------------
    o = _compile_all(sorted((ref / "src" / "base").glob("*.c")), obj / "base", CFLAGS + inc_ocean, jobs)
    _link(o, lib / "libocean_base.so", ["-lpthread"]); say("libocean_base.so")
    o = _compile_all([ref / "src/external/ocean-solid/ocean_solid.c"], obj / "solid", CFLAGS + inc_ocean + inc_solid, jobs)
    _link(o, lib / "libocean_solid.so", rpath + ["-locean_base"]); say("libocean_solid.so")
    o = _compile_all([ref / "src/external/ocean-blas/ocean_custom_blas.c"], obj / "blas",
                     CFLAGS + inc_ocean + ["-I%s" % cfg], jobs)
    _link(o, lib / "libocean_blas.so", rpath); say("libocean_blas.so")

    # ---- the interface layer and the CPU module ------------------------------------------------------------------
    shutil.copy2(SOLID_CPU_DIR / "libsolid_core_cpu.so", lib / "libsolid_core_cpu.so")
    srcs = []
    for sub in ("interface", "generic", "cpu", "cpu/op"):
        srcs += sorted((ref / "src" / "core" / sub).glob("*.c"))
    o = _compile_all(srcs, obj / "core", CFLAGS + inc_ocean + inc_solid, jobs)
    _link(o, lib / "libocean.so", rpath + ["-locean_base", "-locean_solid", "-locean_blas", "-lsolid_core_cpu"])
    say("libocean.so")

    # ---- the reference's GPU module, against THIS repository's header and library -----------------------------------
    gpu_inc = ["-I%s" % (ROOT / "include")] + inc_ocean + inc_solid + ["-I%s" % (CUDA / "include")]
    srcs = sorted((ref / "src/core/gpu").glob("*.c")) + sorted((ref / "src/core/gpu/op").glob("*.c"))
    gflags = [f for f in CFLAGS if f != "-std=gnu99"] + ["-std=gnu11"]
    o = _compile_all(srcs, obj / "gpu", gflags + gpu_inc, jobs)
    gpu_link = rpath + ["-locean", "-locean_base", "-locean_solid", "-lsolid_core_cpu",
                        "-L%s" % GPU_LIBDIR, "-Wl,-rpath,$ORIGIN/../../../../ocean-tensor-package_b200/lib",
                        "-lsolid_core_gpu", "-L%s" % (CUDA / "lib64"), "-lcublas", "-lcudart"]
    _link(o, lib / "libocean_gpu.so", gpu_link); say("libocean_gpu.so (reference dispatch over this repository's Solid GPU library)")

    # ---- the same module with this repository's dispatch in place of the six hot-path files ---------------------------
    replaced = {"tensor_%s_gpu.c" % n for n in ("unary", "binary", "copy", "fill", "reduce_all", "reduce_axis")}
    kept = [f for f in srcs if f.name not in replaced]
    module_c = ROOT / "ocean-tensor-package_b200" / "csrc" / "ocean_module.c"
    o = _compile_all(kept + [module_c], obj / "gpu_b200", gflags + gpu_inc, jobs)
    lib_b200 = OUT / "lib_b200"
    _link(o, lib_b200 / "libocean_gpu.so",
          ["-Wl,-rpath,$ORIGIN/../lib"] + [f for f in gpu_link if f != "-Wl,-rpath,$ORIGIN"] + ["-locean_gpu_b200"])
    say("lib_b200/libocean_gpu.so (this repository's dispatch registered in OcModuleCore)")

    # ---- Python binding ---------------------------------------------------------------------------------------------
    ver = "v%d_%d" % sys.version_info[:2]
    pyinc = ["-I%s" % sysconfig.get_paths()["include"], "-I%s" % (ref / "interfaces/python"),
             "-I%s" % (ref / "interfaces/python/pyOcean/cpu")]
    o = _compile_all(sorted((ref / "interfaces/python/pyOcean/cpu").glob("*.c")), obj / "pycpu",
                     CFLAGS + inc_ocean + pyinc, jobs)
    cpu_so = py / ("pyOcean_cpu_%s.so" % ver)
    _link(o, cpu_so, ["-Wl,-rpath,$ORIGIN/../lib", "-L%s" % lib, "-locean", "-locean_base"]); say(cpu_so.name)
    o = _compile_all(sorted((ref / "interfaces/python/pyOcean/gpu").glob("*.c")), obj / "pygpu",
                     CFLAGS + inc_ocean + pyinc + ["-I%s" % (CUDA / "include")], jobs)
    gpu_so = py / ("pyOcean_gpu_%s.so" % ver)
    _link(o, gpu_so, ["-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN", "-L%s" % lib, "-L%s" % py,
                      "-locean_gpu", "-locean", "-locean_base", "-l:%s" % cpu_so.name]); say(gpu_so.name)
    # numpy interoperability (ocean_numpy), used by golden scripts that cross-check against numpy
    try:
        import numpy
        o = _compile_all([ref / "interfaces/python/pyOceanNumpy/pyOceanNumpy.c"], obj / "pynumpy",
                         CFLAGS + inc_ocean + pyinc + ["-I%s" % numpy.get_include()], jobs)
        np_so = py / ("pyOceanNumpy_%s.so" % ver)
        _link(o, np_so, ["-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN", "-L%s" % lib, "-L%s" % py,
                         "-locean", "-locean_base", "-l:%s" % cpu_so.name]); say(np_so.name)
        (py / "pyOceanNumpy.py").write_text(LOADER_GPU.replace("pyOcean_gpu", "pyOceanNumpy"))
        (py / "ocean_numpy.py").write_text("from pyOceanNumpy import *          # noqa: F401,F403\n")
    except Exception as exc:                                   # the binding works without it
        say("pyOceanNumpy not built: %s" % exc)
    (py / "ocean.py").write_text(LOADER_OCEAN)
    (py / "pyOcean_cpu.py").write_text(LOADER_CPU)
    (py / "pyOcean_gpu.py").write_text(LOADER_GPU)

    # ---- golden scripts, staged for machines without the checkout ----------------------------------------------------
    for sub in ("gpu/tensors", "gpu/index", "cpu/tensors"):
        dst = OUT / "examples" / sub
        dst.mkdir(parents=True, exist_ok=True)
        for f in sorted((ref / "examples/python" / sub).glob("*")):
            if f.suffix in (".py", ".ref"):
                shutil.copy2(f, dst / f.name)
    say("golden scripts staged under %s" % (OUT / "examples"))
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-j", type=int, default=None)
    a = ap.parse_args()
    if reference_dir() is None:
        sys.exit("no reference checkout: set OCEAN_REFERENCE_DIR")
    build(a.force, a.j)
