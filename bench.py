#!/usr/bin/env python3
"""Benchmark of the Solid GPU hot path on B200: achieved HBM GB/s per operation.

Headline workload (BASELINE.json configs[4], the sharded one): float32 x, y of 2^32 elements
(16 GiB each), U(-1,1) from a counter hash of the global index, leading-axis split over the
ranks; one step = fused z = a*x + y (a = 0.5) with sum(z) and sum(z*z) in the same pass, the
per-GPU pairs added by an NCCL all-reduce, norm2 = sqrt(sum(z*z)).  `value` is the whole-job
algorithmic throughput 12 bytes * 2^32 / step time (x and y read once, z written once), inputs
resident in HBM.  `e2e` is the same step through the host-facing API with the inputs streamed
from pinned host memory and the two scalars read back.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--log2n L]

N > 1 is launched by torch.distributed.run (one rank per GPU).  At N = 1 the line also carries
`ops`: one row per operation of configurations 1-4 (GB/s against the measured copy bandwidth,
with the reference's Solid CPU figure beside it) and `cpu_baseline` for the headline step.

`--impl reference` times the reference's own Solid CPU library (oracle/_ref) on the host cores
for the same step, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "ocean-tensor-package_b200"))

import numpy as np                                             # noqa: E402

NOMINAL_HBM_GBS = 8000.0            # the 8 TB/s the metric is defined against
FALLBACK_HBM_GBS = 6650.0           # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
BYTES_PER_ELEMENT = 12              # x read + y read + z written, float32
METRIC = "achieved HBM GB/s (fraction of 8 TB/s/GPU) per op at 1/2/4/8 B200 vs Solid CPU"
WORKLOAD = "C5 fused z=0.5*x+y, sum(z), norm2(z); float32, leading-axis shards, NCCL all-reduce of {sum, sumsq}"


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------
# synthetic data: counter hash of the global index -> U(-1, 1), identical on
# every rank count and on the host
# ---------------------------------------------------------------------------
def hash_uniform_torch(start: int, count: int, seed: int, out):
    """out[i] = u(start + i) on the device, in chunks so temporaries stay small."""
    import torch
    chunk = 1 << 26
    for off in range(0, count, chunk):
        m = min(chunk, count - off)
        idx = torch.arange(start + off, start + off + m, dtype=torch.int64, device=out.device)
        h = (idx * 2654435761 + seed * 40503) & 0xFFFFFFFF
        h = (h ^ (h >> 15)) * 2246822519 & 0xFFFFFFFF
        h = (h ^ (h >> 13)) & 0xFFFFFF                      # 24 bits: exact in float32
        out[off: off + m] = h.to(torch.float32) * (2.0 / 16777216.0) - 1.0
        del idx, h


def hash_uniform_numpy(start: int, count: int, seed: int) -> np.ndarray:
    idx = np.arange(start, start + count, dtype=np.int64)
    h = (idx * 2654435761 + seed * 40503) & 0xFFFFFFFF
    h = ((h ^ (h >> 15)) * 2246822519) & 0xFFFFFFFF
    h = (h ^ (h >> 13)) & 0xFFFFFF
    return (h.astype(np.float32) * np.float32(2.0 / 16777216.0) - np.float32(1.0)).astype(np.float32)


# ---------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, smax, reasons = [], 0, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax = max(smax, float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples taken under load are the upper half of the observed clocks
        loaded = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": smax or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# reference (Solid CPU) arm of the headline step
# ---------------------------------------------------------------------------
def cpu_step_setup(n: int):
    from oracle import ref
    cpu = ref.get()
    threads = os.cpu_count() or 1
    cpu.set_threads(threads)
    x, y = hash_uniform_numpy(0, n, 1), hash_uniform_numpy(0, n, 2)
    a = np.array([0.5], dtype=np.float32)
    t, z = np.empty_like(x), np.empty_like(x)

    def step():
        # what Ocean runs for a*x + y, sum and norm (src/core/interface/tensor_itf.c:4221-4251,5299-5351,5405-5447):
        # scale by a 0-d tensor (stride 0), add, then the two global reductions
        cpu.binary("multiply", "float", [n], [4], x.ctypes.data, [0], a.ctypes.data, [4], t.ctypes.data)
        cpu.binary("add", "float", [n], [4], t.ctypes.data, [4], y.ctypes.data, [4], z.ctypes.data)
        s = cpu.reduce_all("sum", "float", [n], [4], z.ctypes.data)
        q = cpu.reduce_all("norm2", "float", [n], [4], z.ctypes.data)
        return s, q
    return step, threads


def time_cpu(step, repeats: int, warmup: int):
    for _ in range(warmup):
        step()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter(); step(); times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    """`--impl reference`: the reference's Solid CPU code for the headline step on the host cores.  One step is the
    reference's four passes (multiply, add, sum, norm2) over a 2^28-element sample of the workload; `ms_per_step` is
    the MEASURED time of that sample step, `value` the throughput it gives (the same for any sample size of a
    streaming workload), and `config.ms_per_step_full_size` what the full 2^32 elements would take at that rate."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref
    n_full = 1 << args.log2n
    n = min(n_full, 1 << 28)                                   # bounded sample: 1 GiB per tensor
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libsolid_core_cpu.so was not built"}))
        return
    step, threads = cpu_step_setup(n)
    times = time_cpu(step, args.steps, args.warmup)
    t = sum(times) / len(times)
    gbs = BYTES_PER_ELEMENT * n / t / 1e9
    line = {
        "impl": "reference", "metric": METRIC,
        "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "elements": n_full, "sample_elements": n,
                   "ms_per_step_full_size": t * 1e3 * (n_full / n),
                   "note": "Solid CPU (OpenMP) runs multiply, add, sum, norm2 as four passes over the sample; "
                           "no GPU, no shards, no collective on this arm"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "reference",
                         "sample": "%d of %d elements per step" % (n, n_full)},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# per-operation table (configurations 1-4), N = 1 only
# ---------------------------------------------------------------------------
def time_gpu(fn, iters: int, warmup: int = 3, queued: bool = True):
    """Device seconds per call of `fn`.

    With `queued` the calls are issued behind a kernel that idles for a few milliseconds, so that all of them sit
    in the stream before the first one starts: the figure is then the device time of the operation, not the time the
    Python caller needs to issue it (which is larger than the kernel for the 30-60 us operations of this table).
    Calls that wait for the device themselves (global reductions that return a host value) must pass queued=False.
    """
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if queued:
        torch.cuda._sleep(int(2.0e6 * (2 + 0.25 * iters)))          # about 1 ms per 2e6 cycles
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1e-3


def time_call(fn, iters: int):
    """Wall seconds per call of `fn` as the Python caller sees it (issue cost; the device may lag behind)."""
    import torch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    return (t1 - t0) / iters


def ops_table(peak: float, with_cpu: bool, only=None, iters_scale: float = 1.0, checks_on: bool = True):
    """One row per named operation of configurations 1-4: GB/s on algorithmic bytes.  Each row's result is compared
    once with the reference's Solid CPU library (or, where noted, a numpy / float64 evaluation of the same data)
    outside the timed region; `checked` records the outcome."""
    import torch
    from solid_b200 import Tensor, ops, _lib, dtypes as dt
    lib = _lib.get()
    rows = []
    rng = np.random.default_rng(1234)
    cpu = None
    if with_cpu:
        from oracle import ref
        if ref.available():
            cpu = ref.get(); cpu.set_threads(os.cpu_count() or 1)

    def add_row(config, name, nbytes, fn, cpu_fn=None, iters=20, queued=True, check=None):
        """`check` runs once, outside the timed region, after the timed calls: it compares what the operation left
        behind (or returns) with the oracle or a float64 evaluation and returns True / False; None = not compared."""
        iters = max(1, int(iters * iters_scale))
        t = time_gpu(fn, iters, warmup=3 if iters_scale >= 1 else 1, queued=queued)
        row = {"config": config, "op": name, "bytes": nbytes, "us": t * 1e6, "gbs": nbytes / t / 1e9,
               "frac_measured": nbytes / t / 1e9 / peak, "frac_8tbs": nbytes / t / 1e9 / NOMINAL_HBM_GBS,
               "issue_us": time_call(fn, iters) * 1e6}
        if cpu is not None and cpu_fn is not None:
            tc = min(time_cpu(cpu_fn, 3, 1))
            row["cpu_gbs"] = nbytes / tc / 1e9
        row["checked"] = None
        if check is not None and checks_on:
            try:
                torch.cuda.synchronize()
                row["checked"] = bool(check())
            except Exception as exc:                          # a failed comparison is reported, never hidden
                row["checked"] = False
                row["check_error"] = str(exc)[:200]
        rows.append(row)

    def same_bits(a, b):
        a = np.ascontiguousarray(a).view(np.uint8).reshape(-1); b = np.ascontiguousarray(b).view(np.uint8).reshape(-1)
        return a.shape == b.shape and bool(np.array_equal(a, b))

    def tree_bound(n, scale, u=2.0 ** -24):
        return (4 * math.log2(max(n, 2)) + 4) * u * scale

    def max_ulp(got, want):
        ia = got.view(np.int32).astype(np.int64); ib = want.view(np.int32).astype(np.int64)
        ia = np.where(ia < 0, -(2 ** 31) - ia, ia); ib = np.where(ib < 0, -(2 ** 31) - ib, ib)
        return int(np.abs(ia - ib).max())

    def dev(arr, dtype=None):
        return Tensor.from_numpy(arr, dtype)

    rbuf = torch.empty(lib.reduce_all_buffer_size(1 << 26, 0), dtype=torch.uint8, device="cuda")
    rres = torch.empty(16, dtype=torch.uint8, device="cuda")
    cur = torch.cuda.current_stream().cuda_stream

    # ---- C1: float32 1-D, n = 2^24; three distinct buffer sets so 67-200 MB working sets are not L2 hits
    if only in (None, "C1"):
        n = 1 << 24
        hx = [rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3)]
        hy = [rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3)]
        xs, ys = [dev(a) for a in hx], [dev(a) for a in hy]
        zs = [Tensor.empty([n], "float") for _ in range(3)]
        state = {"i": 0}

        def rot():
            state["i"] = (state["i"] + 1) % 3
            return state["i"]
        hz = np.empty(n, dtype=np.float32)

        def check_binary(name):
            ops.binary(name, xs[0], ys[0], zs[0])
            return same_bits(zs[0].numpy(), hx[0] + hy[0] if name == "add" else hx[0] * hy[0])
        for name in ("add", "multiply"):
            add_row("C1", name + " f32 2^24", 12 * n,
                    lambda name=name: (lambda i: ops.binary(name, xs[i], ys[i], zs[i]))(rot()),
                    (lambda name=name: cpu.binary(name, "float", [n], [4], hx[0].ctypes.data, [4], hy[0].ctypes.data, [4], hz.ctypes.data)) if cpu else None,
                    check=lambda name=name: check_binary(name))
        # the scalar operand by value (Ocean's multiplyScalar without its 0-d device tensor) and a range
        add_row("C1", "multiply by a scalar (by value) f32 2^24", 8 * n,
                lambda: (lambda i: ops.scalar_op("multiply", xs[i], 0.5, zs[i]))(rot()),
                (lambda: cpu.binary("multiply", "float", [n], [4], hx[0].ctypes.data, [0], hy[0].ctypes.data, [4], hz.ctypes.data)) if cpu else None,
                check=lambda: (ops.scalar_op("multiply", xs[0], 0.5, zs[0]), same_bits(zs[0].numpy(), hx[0] * np.float32(0.5)))[1])
        add_row("C1", "range offset + i*step (steps_double) f32 2^24", 4 * n,
                lambda: (lambda i: lib.steps("double", "float", [n], [4], zs[i].ptr, -1.0, 1e-3, cur))(rot()),
                (lambda: cpu.steps("double", "float", [n], [4], hz.ctypes.data, -1.0, 1e-3)) if cpu else None,
                check=lambda: (lib.steps("double", "float", [n], [4], zs[0].ptr, -1.0, 1e-3, cur),
                               same_bits(zs[0].numpy(), (-1.0 + np.arange(n, dtype=np.float64) * 1e-3).astype(np.float32)))[1])

        def check_reduce(name, device_form):
            x64 = hx[0].astype(np.float64)
            if device_form:
                lib.reduce_all_device(name, "float", [n], [4], xs[0].ptr, rres.data_ptr(), rbuf.data_ptr(), cur)
                torch.cuda.synchronize()
                got = float(rres.cpu().numpy()[:4].view(np.float32)[0])
            else:
                got = float(ops.reduce_all(name, xs[0]))
            if name == "maximum":
                return got == float(hx[0].max())
            if name == "sum":
                return abs(got - x64.sum()) <= tree_bound(n, np.abs(x64).sum())
            nrm = math.sqrt((x64 * x64).sum())
            return abs(got - nrm) <= tree_bound(n, nrm)
        for name in ("sum", "norm2", "maximum"):
            add_row("C1", name + " f32 2^24 (incl. host read-back)", 4 * n,
                    lambda name=name: ops.reduce_all(name, xs[rot()]),
                    (lambda name=name: cpu.reduce_all(name, "float", [n], [4], hx[0].ctypes.data)) if cpu else None, queued=False,
                    check=lambda name=name: check_reduce(name, False))
        for name in ("sum", "norm2", "maximum"):
            add_row("C1", name + " f32 2^24 (result stays on the device)", 4 * n,
                    lambda name=name: (lambda i: lib.reduce_all_device(name, "float", [n], [4], xs[i].ptr, rres.data_ptr(),
                                                                       rbuf.data_ptr(), cur))(rot()),
                    check=lambda name=name: check_reduce(name, True))
        # the launch-to-result cost that every global reduction pays, whatever its size: the same call on 4096 elements
        small = Tensor(xs[0].storage, "float", [4096])
        add_row("C1", "sum f32 4096 elements (fixed cost of a device-resident reduction)", 4 * 4096,
                lambda: lib.reduce_all_device("sum", "float", [4096], [4], small.ptr, rres.data_ptr(), rbuf.data_ptr(), cur))
        add_row("C1", "sum f32 4096 elements (fixed cost incl. host read-back)", 4 * 4096,
                lambda: ops.reduce_all("sum", small), queued=False)

    # ---- C2: C(f32) = A(f64, transposed) * B(i32, byteswapped) + r(f32 row broadcast), 4096^2; unaligned byteswapped f64 -> f16
    if only in (None, "C2"):
        m = 4096
        A = rng.uniform(-1, 1, (m, m))                                   # row-major buffer viewed transposed
        B = rng.integers(-1000, 1001, (m, m)).astype(np.int32)
        r = rng.uniform(-1, 1, m).astype(np.float32)
        tA = Tensor(torch.from_numpy(A.view(np.uint8).reshape(-1)).cuda(), "double", [m, m], [8 * m, 8])
        tB = Tensor(torch.from_numpy(B.astype(">i4").view(np.uint8).reshape(-1)).cuda(), "int32", [m, m], [4, 4 * m], byteswapped=True)
        tr = Tensor(torch.from_numpy(r.view(np.uint8)).cuda(), "float", [m, m], [0, 4])
        tC = Tensor.empty([m, m], "float")
        want_c2 = (A.reshape(-1, order="F") * B.reshape(-1).astype(np.float64) + np.repeat(r.astype(np.float64), m)).astype(np.float32)
        add_row("C2", "fused C=f32(A_f64^T * bswap(B_i32) + r_f32) 4096^2", 16 * m * m,
                lambda: ops.multiply_add(tA, tB, tr, tC),
                check=lambda: same_bits(tC.numpy().reshape(-1, order="F"), want_c2))
        # the same expression as the reference runs it: three converting copies into dense doubles, multiply, add,
        # converting copy of the result (64 bytes per element instead of 16)
        # (src/core/generic/tensor_op.c:170-186: B and r are cast to the common type double through Tensor_copy, A is
        # already double and is read through its transposed view, r stays a broadcast row)
        tA64, tB64 = Tensor.empty([m, m], "double"), Tensor.empty([m, m], "double")
        tr64 = Tensor.empty([m], "double")
        tr64b = Tensor(tr64.storage, "double", [m, m], [0, 8])
        trv = Tensor(tr.storage, "float", [m], [4])
        tP, tS, tC2 = Tensor.empty([m, m], "double"), Tensor.empty([m, m], "double"), Tensor.empty([m, m], "float")

        def unfused():
            ops.copy(tB, tB64); ops.copy(trv, tr64)
            ops.binary("multiply", tA, tB64, tP); ops.binary("add", tP, tr64b, tS); ops.copy(tS, tC2)
        add_row("C2", "unfused sequence for the same C (convert B, multiply by A^T, add r, convert) 4096^2, 5 launches", 64 * m * m,
                unfused, iters=10, check=lambda: same_bits(tC2.numpy().reshape(-1, order="F"), want_c2))
        add_row("C2", "copy f64 4096^2 A^T -> dense (transposing copy)", 16 * m * m, lambda: ops.copy(tA, tA64),
                check=lambda: same_bits(tA64.numpy().reshape(-1, order="F"), A.reshape(-1, order="F")))
        F1 = rng.uniform(-1, 1, (m, m)).astype(np.float32); F2 = rng.uniform(-1, 1, (m, m)).astype(np.float32)
        tF1 = Tensor(torch.from_numpy(F1.view(np.uint8).reshape(-1)).cuda(), "float", [m, m], [4 * m, 4])   # transposed view
        tF2 = Tensor(torch.from_numpy(F2.view(np.uint8).reshape(-1)).cuda(), "float", [m, m], [4, 4 * m])
        tF3 = Tensor.empty([m, m], "float")
        add_row("C2", "add f32 A^T + B 4096^2 (one operand transposed)", 12 * m * m, lambda: ops.binary("add", tF1, tF2, tF3),
                check=lambda: same_bits(tF3.numpy().reshape(-1, order="F"), F1.reshape(-1, order="F") + F2.reshape(-1)))
        # strided views that are dense along dimension 0: padded rows (a 4096 x 4096 block of arrays with a pitch of
        # 4160 elements) and an operand broadcast along dimension 0
        pitch = m + 64
        G1 = rng.uniform(-1, 1, (m, pitch)).astype(np.float32); G2 = rng.uniform(-1, 1, (m, pitch)).astype(np.float32)
        tG1 = Tensor(torch.from_numpy(G1.view(np.uint8).reshape(-1)).cuda(), "float", [m, m], [4, 4 * pitch])
        tG2 = Tensor(torch.from_numpy(G2.view(np.uint8).reshape(-1)).cuda(), "float", [m, m], [4, 4 * pitch])
        tG3 = Tensor(torch.zeros(4 * m * pitch, dtype=torch.uint8, device="cuda"), "float", [m, m], [4, 4 * pitch])
        add_row("C2", "add f32 on 4096^2 blocks of arrays with padded rows (pitch 4160)", 12 * m * m,
                lambda: ops.binary("add", tG1, tG2, tG3),
                check=lambda: same_bits(np.ascontiguousarray(tG3.storage.cpu().numpy().view(np.float32).reshape(m, pitch)[:, :m]).reshape(-1),
                                        (G1[:, :m] + G2[:, :m]).reshape(-1)))
        add_row("C2", "add f64 P + r 4096^2 (r broadcast along dimension 0)", 16 * m * m,
                lambda: ops.binary("add", tP, tr64b, tS),
                check=lambda: same_bits(tS.numpy().reshape(-1, order="F"), tP.numpy().reshape(-1, order="F") + np.repeat(tr64.numpy().reshape(-1), m)))
        del tA64, tB64, tr64, tr64b, trv, tP, tS, tC2, tF1, tF2, tF3, tG1, tG2, tG3
        raw = np.zeros(8 * m * m + 64, dtype=np.uint8)
        raw[3: 3 + 8 * m * m] = A.astype(">f8").view(np.uint8).reshape(-1)
        tU = Tensor(torch.from_numpy(raw).cuda(), "double", [m * m], [8], offset=3, byteswapped=True)
        tH = Tensor.empty([m * m], "half")
        hH = np.empty(m * m, dtype=np.uint16)
        def check_unaligned():
            if cpu is None:
                return None
            cpu.copy("double", "half", [m * m], [8], raw.ctypes.data + 3, [m * m], [2], hH.ctypes.data, variant="byteswap_copy")
            ops.copy(tU, tH)
            return same_bits(tH.numpy(), hH)
        add_row("C2", "copy f64 (offset 3 B, byteswapped) -> f16 4096^2", 10 * m * m, lambda: ops.copy(tU, tH),
                (lambda: cpu.copy("double", "half", [m * m], [8], raw.ctypes.data + 3, [m * m], [2], hH.ctypes.data, variant="byteswap_copy")) if cpu else None,
                check=check_unaligned if cpu else None)
        # gather through offset tables (get_index): rows (the dense dimension) or columns of a column-major matrix
        gm, gn = 8192, 4096
        G = rng.normal(size=(gm, gn)).astype(np.float32)
        hG = np.asfortranarray(G)
        tG, tS = dev(hG), Tensor.empty([gm, gn], "float")
        hS = np.empty((gm, gn), dtype=np.float32, order="F")
        row_tab = (rng.permutation(gm).astype(np.int64) * 4); col_tab = (rng.permutation(gn).astype(np.int64) * 4 * gm)
        d_rows = torch.from_numpy(row_tab).cuda(); d_cols = torch.from_numpy(col_tab).cuda()
        add_row("C2", "get_index rows A[perm, :] f32 8192x4096 (4-byte gathers)", 8 * gm * gn,
                lambda: lib.index2("get_index", "float", [gm, gn], [d_rows.data_ptr(), None], [0, 4 * gm], tG.ptr,
                                   [4, 4 * gm], tS.ptr, cur), iters=10,
                cpu_fn=(lambda: cpu.index2("get_index", "float", [gm, gn], [row_tab.ctypes.data, None], [0, 4 * gm], hG.ctypes.data,
                                           [4, 4 * gm], hS.ctypes.data)) if cpu else None,
                check=lambda: same_bits(tS.numpy(), G[row_tab // 4, :]))
        add_row("C2", "get_index columns A[:, perm] f32 8192x4096 (32 KB runs)", 8 * gm * gn,
                lambda: lib.index2("get_index", "float", [gm, gn], [None, d_cols.data_ptr()], [4, 0], tG.ptr,
                                   [4, 4 * gm], tS.ptr, cur), iters=10,
                cpu_fn=(lambda: cpu.index2("get_index", "float", [gm, gn], [None, col_tab.ctypes.data], [4, 0], hG.ctypes.data,
                                           [4, 4 * gm], hS.ctypes.data)) if cpu else None,
                check=lambda: same_bits(tS.numpy(), G[:, col_tab // (4 * gm)]))
        del tA, tB, tC, tU, tH, tG, tS

    # ---- C3: axis reductions on 8192^2 (column-major: axis 0 is the dense one), global any/all/nnz on bool
    if only in (None, "C3"):
        k = 8192
        for dtype, npdt, gen in (("float", np.float32, lambda: rng.normal(size=(k, k)).astype(np.float32)),
                                 ("int64", np.int64, lambda: rng.integers(-2 ** 20, 2 ** 20, (k, k), dtype=np.int64))):
            h = np.asfortranarray(gen())
            t = dev(h)
            es = dt.SIZE[dtype]
            for name in ("sum", "minimum", "maximum", "norm2"):
                for axis in (0, 1):
                    rtype = {"sum": dtype, "minimum": dtype, "maximum": dtype, "norm2": "float" if dtype == "float" else "double"}[name]
                    out = Tensor.empty([k], rtype)
                    hout = np.empty(k, dtype=dt.NUMPY[rtype])
                    keep = 1 - axis

                    def check_axis(name=name, axis=axis, out=out, rtype=rtype):
                        got = out.numpy()
                        if dtype == "int64" and name != "norm2":
                            want = {"sum": h.sum(axis=axis), "minimum": h.min(axis=axis), "maximum": h.max(axis=axis)}[name]
                            return bool(np.array_equal(got, want))
                        if name in ("minimum", "maximum"):
                            return bool(np.array_equal(got, h.min(axis=axis) if name == "minimum" else h.max(axis=axis)))
                        h64 = h.astype(np.float64)
                        u = 2.0 ** -53 if rtype == "double" else 2.0 ** -24
                        if name == "sum":
                            return bool(np.all(np.abs(got - h64.sum(axis=axis)) <= tree_bound(k, np.abs(h64).sum(axis=axis), u)))
                        nrm = np.sqrt((h64 * h64).sum(axis=axis))
                        return bool(np.all(np.abs(got - nrm) <= tree_bound(k, nrm, u)))
                    add_row("C3", "axis_%s %s 8192^2 axis %d" % (name, dtype, axis), es * k * k,
                            lambda name=name, axis=axis, out=out: ops.reduce_axis(name, t, axis, out), iters=10,
                            cpu_fn=(lambda name=name, axis=axis, keep=keep, hout=hout: cpu.reduce_axis(
                                "axis_" + name, dtype, [k], [h.strides[keep]], h.ctypes.data, [hout.itemsize], hout.ctypes.data,
                                [k], [h.strides[axis]])) if cpu else None, check=check_axis)
            del t, h
        hb = (rng.random((k, k)) < 0.1).astype(np.uint8)
        tb = dev(hb, "bool")
        bool_want = {"any": int(hb.any()), "all": int(hb.all()), "nnz": int(hb.sum())}

        def check_bool(name, device_form):
            if not device_form:
                return int(ops.reduce_all(name, tb)) == bool_want[name]
            lib.reduce_all_device(name, "bool", [k * k], [1], tb.ptr, rres.data_ptr(), rbuf.data_ptr(), cur)
            torch.cuda.synchronize()
            raw8 = rres.cpu().numpy()
            return int(raw8[:8].view(np.uint64)[0] if name == "nnz" else raw8[0]) == bool_want[name]
        for name in ("any", "all", "nnz"):
            add_row("C3", "%s bool 8192^2 (incl. host read-back)" % name, k * k, lambda name=name: ops.reduce_all(name, tb),
                    (lambda name=name: cpu.reduce_all(name, "bool", [k * k], [1], hb.ctypes.data)) if cpu else None, queued=False,
                    check=lambda name=name: check_bool(name, False))
            add_row("C3", "%s bool 8192^2 (result stays on the device)" % name, k * k,
                    lambda name=name: lib.reduce_all_device(name, "bool", [k * k], [1], tb.ptr, rres.data_ptr(), rbuf.data_ptr(), cur),
                    check=lambda name=name: check_bool(name, True))
        del tb

    # ---- C4: unary chain on 2^26 elements
    if only in (None, "C4"):
        n4 = 1 << 26
        hf = rng.uniform(0.01, 10, n4).astype(np.float32)
        tf, to = dev(hf), Tensor.empty([n4], "float")
        ho = np.empty(n4, dtype=np.float32)
        def check_unary(name):
            if cpu is None:
                return None
            cpu.unary(name, "float", [n4], [4], hf.ctypes.data, [4], ho.ctypes.data)
            got = to.numpy()
            return same_bits(got, ho) if name in ("sqrt", "fabs") else max_ulp(got, ho) <= 2
        for name in ("sqrt", "exp", "log", "sin", "fabs"):
            add_row("C4", "%s f32 2^26" % name, 8 * n4, lambda name=name: ops.unary(name, tf, to), iters=10,
                    cpu_fn=(lambda name=name: cpu.unary(name, "float", [n4], [4], hf.ctypes.data, [4], ho.ctypes.data)) if cpu else None,
                    check=(lambda name=name: check_unary(name)) if cpu else None)
        del tf, to
        hc = (rng.normal(size=n4) + 1j * rng.normal(size=n4)).astype(np.complex128)
        hd = (rng.normal(size=n4) + 1j * rng.normal(size=n4)).astype(np.complex128)
        tc, td, tz = dev(hc), dev(hd), Tensor.empty([n4], "cdouble")
        ta = Tensor.empty([n4], "double")
        hz2 = np.empty(n4, dtype=np.complex128)
        def check_abs():
            cpu.unary("absolute", "cdouble", [n4], [16], hc.ctypes.data, [8], hz2.ctypes.data)
            got = ta.numpy().view(np.int64); want = hz2.view(np.float64)[:n4].view(np.int64)
            return int(np.abs(got - want).max()) <= 2                      # positive doubles: bit distance = ulp distance

        def check_cmul():
            cpu.binary("multiply", "cdouble", [n4], [16], hc.ctypes.data, [16], hd.ctypes.data, [16], hz2.ctypes.data)
            return same_bits(tz.numpy(), hz2)
        add_row("C4", "conj c128 2^26", 32 * n4, lambda: ops.unary("conj", tc, tz), iters=5,
                cpu_fn=(lambda: cpu.unary("conj", "cdouble", [n4], [16], hc.ctypes.data, [16], hz2.ctypes.data)) if cpu else None,
                check=lambda: same_bits(tz.numpy(), np.conj(hc)))
        add_row("C4", "absolute c128 2^26", 24 * n4, lambda: ops.unary("absolute", tc, ta), iters=5,
                cpu_fn=(lambda: cpu.unary("absolute", "cdouble", [n4], [16], hc.ctypes.data, [8], hz2.ctypes.data)) if cpu else None,
                check=check_abs if cpu else None)
        add_row("C4", "multiply c128 2^26", 48 * n4, lambda: ops.binary("multiply", tc, td, tz), iters=5,
                cpu_fn=(lambda: cpu.binary("multiply", "cdouble", [n4], [16], hc.ctypes.data, [16], hd.ctypes.data, [16], hz2.ctypes.data)) if cpu else None,
                check=check_cmul if cpu else None)
        del tc, td, tz, ta, hc, hd, hz2
        from oracle import solid_numpy as sn
        hh = sn.float_to_half(rng.uniform(-4, 4, n4).astype(np.float32))
        hg = sn.float_to_half(rng.uniform(-4, 4, n4).astype(np.float32))
        th, tg, tq = dev(hh, "half"), dev(hg, "half"), Tensor.empty([n4], "half")
        def check_haxpy():
            ah = sn.float_to_half(np.array([0.5], dtype=np.float32))
            t16, w16 = np.empty(n4, dtype=np.uint16), np.empty(n4, dtype=np.uint16)
            cpu.binary("multiply", "half", [n4], [2], hh.ctypes.data, [0], ah.ctypes.data, [2], t16.ctypes.data)
            cpu.binary("add", "half", [n4], [2], t16.ctypes.data, [2], hg.ctypes.data, [2], w16.ctypes.data)
            return same_bits(tq.numpy(), w16)
        add_row("C4", "fused a*x+y f16 2^26", 6 * n4, lambda: ops.axpy(0.5, th, tg, tq), iters=10,
                check=check_haxpy if cpu else None)
    torch.cuda.synchronize()
    return rows


# ---------------------------------------------------------------------------
# headline: C5 on N GPUs
# ---------------------------------------------------------------------------
def result_checked(log2n: int, final):
    """The step's two scalars against the float64 sums of the same hashed data, where tests/golden/c5_constants.json
    holds them for this size (made by tests/golden/make_c5_constants.py); None for other sizes."""
    f = ROOT / "tests" / "golden" / "c5_constants.json"
    try:
        c = json.loads(f.read_text())[str(log2n)]
    except Exception:
        return None
    n = float(1 << log2n)
    stat = 16 * 2.0 ** -24 * math.sqrt(n * math.log2(n)) * math.sqrt(c["sumsq"] / n)     # see tests/test_gpu_configs.py
    return bool(abs(final[0] - c["sum"]) <= stat and abs(final[1] - c["norm2"]) <= 4 * 2.0 ** -24 * c["norm2"])


def run_ours(args):
    import torch
    import torch.distributed as dist
    from solid_b200 import Tensor, ops, shard, _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GPU module has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a collective that cannot complete should end the run after minutes, not after the default ten
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
    lib = _lib.get()
    lib.initialize()
    peak, peak_kind = measured_peak()

    n_total = 1 << args.log2n
    per = (n_total + world - 1) // world                      # leading-axis split "as evenly as possible"
    lo, hi = shard.shard_range(n_total, rank, world)
    n = hi - lo
    x = torch.empty(n, dtype=torch.float32, device=device)
    y = torch.empty(n, dtype=torch.float32, device=device)
    z = torch.empty(n, dtype=torch.float32, device=device)
    hash_uniform_torch(lo, n, 1, x)
    hash_uniform_torch(lo, n, 2, y)
    tx = Tensor(x.view(torch.uint8), "float", [n]); ty = Tensor(y.view(torch.uint8), "float", [n])
    tz = Tensor(z.view(torch.uint8), "float", [n])
    sums = torch.zeros(2, dtype=torch.float32, device=device)
    t_sumsq = Tensor(sums.view(torch.uint8), "float", [1], offset=4)      # the second scalar: sum of squares, then norm2

    kstart = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    kstop = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]

    # The exchange of the per-GPU pairs: one kernel of the library over peer memory (NVLink) where symmetric memory can
    # be set up, else the NCCL all-reduce followed by the square root (SOLID_B200_EXCHANGE=nccl forces the latter).
    peer = shard.PeerSum.create(device) if world > 1 else None

    def step(i=None):
        if i is not None:
            kstart[i].record()
        ops.axpy_sums(0.5, tx, ty, tz, sums)                 # streaming kernel + one launch that folds its partial sums
        if i is not None:
            kstop[i].record()
        if peer is not None:
            peer.sum_pair(sums, sqrt_second=True)            # pairs exchanged through peer memory, added in rank order, norm2
        else:
            shard.combine(sums, "sum")                       # per-GPU {sum z, sum z^2} added over NVLink (NCCL all-reduce)
            ops.unary("sqrt", t_sumsq, t_sumsq)              # norm2 in place, one small launch of the library

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:                      # sampled from the warm-up on: the timed region is short
        time.sleep(0.25)
        for _ in range(args.warmup):
            step()
        barrier()
        start.record()
        for i in range(args.steps):
            step(i)
        stop.record()
        final_dev = sums.clone()                              # {sum, norm2} of the last timed step
        barrier()
        if peer is not None:
            peer.check()                                      # no exchange gave up waiting for a peer
        # keep the GPU under the same load until a few more samples exist.  The loop is bounded by the clock, so its
        # trip count differs between ranks: it must not contain a collective (the kernel alone is the load).
        t_end = time.time() + 0.6
        while time.time() < t_end:
            ops.axpy_sums(0.5, tx, ty, tz, sums)
            torch.cuda.synchronize()
        barrier()
    ms_total = start.elapsed_time(stop)
    kernel_ms = sum(a.elapsed_time(b) for a, b in zip(kstart, kstop)) / args.steps
    final = final_dev.cpu().numpy().tolist()

    # ---- end to end: inputs streamed from pinned host memory, result scalars read back
    win = min(n, 1 << 26)                                     # 256 MiB windows, double buffered
    hx = torch.empty(win, dtype=torch.float32).pin_memory()
    hy = torch.empty(win, dtype=torch.float32).pin_memory()
    hx.copy_(x[:win].cpu()); hy.copy_(y[:win].cpu())
    dx = [torch.empty(win, dtype=torch.float32, device=device) for _ in range(2)]
    dy = [torch.empty(win, dtype=torch.float32, device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device)
    acc = torch.zeros(2, dtype=torch.float32, device=device)
    part = torch.zeros(2, dtype=torch.float32, device=device)
    host_out = torch.zeros(2, dtype=torch.float32).pin_memory()

    def e2e_step():
        acc.zero_()
        main = torch.cuda.current_stream(device)
        ready = [None, None]
        done = [None, None]
        nwin = (n + win - 1) // win
        for w in range(nwin):
            b = w % 2
            m = min(win, n - w * win)
            with torch.cuda.stream(copy_stream):
                if done[b] is not None:
                    copy_stream.wait_event(done[b])
                dx[b][:m].copy_(hx[:m], non_blocking=True)
                dy[b][:m].copy_(hy[:m], non_blocking=True)
                ready[b] = copy_stream.record_event()
            main.wait_event(ready[b])
            tw = Tensor(dx[b].view(torch.uint8), "float", [m]); tv = Tensor(dy[b].view(torch.uint8), "float", [m])
            tzw = Tensor(z.view(torch.uint8), "float", [m], offset=4 * w * win)
            ops.axpy_sums(0.5, tw, tv, tzw, part)
            acc.add_(part)
            done[b] = main.record_event()
        shard.combine(acc, "sum")
        acc[1] = torch.sqrt(acc[1])
        host_out.copy_(acc, non_blocking=True)
        main.synchronize()

    # what the streamed step must give: every window is the first `win` elements of the shard, sent nwin times
    nwin_full, tail = divmod(n, win)
    zw = (np.float32(0.5) * hx.numpy() + hy.numpy()).astype(np.float32).astype(np.float64)
    e2e_sum = nwin_full * zw.sum() + (zw[:tail].sum() if tail else 0.0)
    e2e_sumsq = nwin_full * (zw * zw).sum() + ((zw[:tail] ** 2).sum() if tail else 0.0)
    e2e_sum_abs = nwin_full * np.abs(zw).sum() + (np.abs(zw[:tail]).sum() if tail else 0.0)
    del zw

    # bare host-to-device rate of this rank with every rank copying at the same time: the ceiling of the streamed step
    barrier()
    hs, he = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    hs.record()
    for _ in range(4):
        dx[0].copy_(hx, non_blocking=True); dy[0].copy_(hy, non_blocking=True)
    he.record()
    barrier()
    h2d_gbs = 4 * 8 * win / (hs.elapsed_time(he) * 1e-3) / 1e9

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    es.record()
    for _ in range(e2e_steps):
        e2e_step()
    ee.record()
    barrier()
    e2e_ms = es.elapsed_time(ee) / e2e_steps
    got = host_out.numpy().astype(np.float64)
    tot = torch.tensor([e2e_sum, e2e_sumsq, e2e_sum_abs], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tot)
    e2e_sum, e2e_sumsq, e2e_sum_abs = tot.cpu().tolist()
    bound = (4 * math.log2(n_total) + 4) * 2.0 ** -24
    e2e_checked = bool(abs(got[0] - e2e_sum) <= bound * e2e_sum_abs and abs(got[1] - math.sqrt(e2e_sumsq)) <= bound * math.sqrt(e2e_sumsq))

    # ---- max over ranks
    t = torch.tensor([ms_total, kernel_ms, e2e_ms, -h2d_gbs], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, kernel_ms, e2e_ms, h2d_neg = t.cpu().tolist()
    h2d_gbs = -h2d_neg                                        # the slowest rank's bare copy rate
    cl = clocks.summary()

    if rank == 0:
        ms_step = ms_total / args.steps
        value = BYTES_PER_ELEMENT * n_total / (ms_step * 1e-3) / 1e9
        achieved = BYTES_PER_ELEMENT * per / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC,
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "elements": n_total, "elements_per_gpu": per, "l2": "inputs (%.1f GiB per GPU) far larger than the 126 MB L2" % (8 * per / 2 ** 30),
                       "hash_seed": [1, 2],
                       "exchange": ("none (one GPU)" if world == 1 else
                                    "one kernel over peer memory: pairs stored into every peer's buffer, added in rank order, square root"
                                    if peer is not None else "NCCL all-reduce of the pair, then the square root")},
            "frac_of_8tbs_per_gpu": value / (world * NOMINAL_HBM_GBS),
            "frac_of_measured_copy_per_gpu": value / (world * peak),
            "elements_per_s": n_total / (ms_step * 1e-3),
            "result": {"sum": final[0], "norm2": final[1], "checked": result_checked(args.log2n, final)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": "of " + peak_kind, "kernel": "axpy_sums_kernel<float>",
                         "kernel_ms": kernel_ms,
                         # dram__bytes_read + dram__bytes_write of one launch: 3.184 GB measured by ncu at 2^28
                         # elements, proportional to the element count (one pass, nothing is read twice)
                         "traffic": 3.184e9 * per / float(1 << 28), "traffic_unit": "bytes per launch"},
            "e2e": {"value": BYTES_PER_ELEMENT * n_total / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": 8 * per, "d2h_bytes_per_step": 8, "ms_per_step": e2e_ms,
                    "h2d_gbs_per_rank_bare": h2d_gbs, "h2d_gbs_per_rank_in_step": 8 * per / (e2e_ms * 1e-3) / 1e9,
                    "checked": e2e_checked,
                    "note": "a host-to-device streaming probe through the library's public call (ops.axpy_sums), not a "
                            "full plugin round trip: every rank re-sends ONE pinned 256 MiB window of x and of y (the "
                            "first elements of its shard) until its whole shard length has crossed PCIe, double "
                            "buffered against the kernel; z (4 bytes per element) stays on the device; the two "
                            "scalars are read back and compared with a float64 evaluation of what was streamed "
                            "(`checked`).  h2d_gbs_per_rank_bare is the same two buffers copied with nothing else "
                            "running on the rank, all ranks at once: the ceiling this number can reach."},
            # per step: the streaming kernel, the fold of its partial sums, and the exchange kernel (sum over the GPUs
            # and square root) or, with one GPU or on the NCCL route, the square root kernel
            "gpu_launches": 3 * args.steps * world,
            "clocks": cl,
        }
        if world == 1 and not args.no_cpu:
            try:
                from oracle import ref
                if ref.available():
                    ns = min(n_total, 1 << 27)
                    cstep, threads = cpu_step_setup(ns)
                    tc = min(time_cpu(cstep, 3, 1))
                    line["cpu_baseline"] = {"value": BYTES_PER_ELEMENT * ns / tc / 1e9, "unit": "GB/s", "cores": threads,
                                            "kind": "reference", "sample": "%d of %d elements, four passes (multiply, add, sum, norm2)" % (ns, n_total)}
            except Exception as exc:                           # the baseline is a reported extra, never a blocker
                line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "reference", "sample": "failed: %s" % exc}
        if world == 1 and not args.no_ops:
            del x, y, z, tx, ty, tz, dx, dy
            torch.cuda.empty_cache()
            line["ops"] = ops_table(peak, with_cpu=not args.no_cpu)
            # the same rows in short form inside `roofline`, so that a record which keeps only the head of the line
            # still carries every per-operation fraction: [config, op, us, GB/s, fraction of measured copy, checked]
            line["roofline"]["per_op"] = [[r["config"], r["op"], round(r["us"], 2), round(r["gbs"], 1),
                                           round(r["frac_measured"], 3), r["checked"]] for r in line["ops"]]
            line["roofline"]["per_op_columns"] = ["config", "op", "us", "gbs", "frac_of_measured_copy", "checked"]
            line["ops_checked"] = {"true": sum(1 for r in line["ops"] if r["checked"] is True),
                                   "false": sum(1 for r in line["ops"] if r["checked"] is False),
                                   "not_compared": sum(1 for r in line["ops"] if r["checked"] is None)}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_peer_copy(args):
    """`--peer-copy`: the cross-device copy of the dispatch library (one process, GPUs 0 and 1) against the plain
    peer copy of the same bytes.  Cases: a dense float64 matrix (what cudaMemcpyPeerAsync can move too), and a
    converting, transposing copy (int32 4096^2 viewed transposed on GPU 1 -> float64 dense on GPU 0) that the
    reference stages through dense temporaries on both sides.  Time is measured with events on the destination's
    stream; the source is read with plain loads over NVLink by a kernel running on the destination GPU."""
    import torch
    from solid_b200 import Tensor, ops
    if torch.cuda.device_count() < 2:
        print(json.dumps({"peer_copy": None, "unavailable": "needs two GPUs"}))
        return
    m = 4096
    rng = np.random.default_rng(7)
    rows = []

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(0); torch.cuda.synchronize(1)
        with torch.cuda.device(0):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize(0); torch.cuda.synchronize(1)
            return a.elapsed_time(b) / iters * 1e-3

    D = rng.uniform(-1, 1, (m, m))
    src64 = Tensor.from_numpy(np.asfortranarray(D), device="cuda:1")
    dst64 = Tensor.empty([m, m], "double", device="cuda:0")
    raw_src = src64.storage; raw_dst = dst64.storage
    t_plain = timed(lambda: raw_dst[: 8 * m * m].copy_(raw_src[: 8 * m * m], non_blocking=True))
    rows.append({"op": "cudaMemcpyPeerAsync f64 4096^2 (128 MiB), GPU 1 -> GPU 0", "us": t_plain * 1e6, "gbs": 8 * m * m / t_plain / 1e9})
    t = timed(lambda: ops.copy(src64, dst64))
    ok = bool(np.array_equal(dst64.numpy(), D))
    rows.append({"op": "OcTensorGPU_copy f64 dense -> f64 dense, GPU 1 -> GPU 0 (peer loads)", "us": t * 1e6, "gbs": 8 * m * m / t / 1e9,
                 "of_plain_peer_copy": t_plain / t, "checked": ok})
    I = rng.integers(-1000, 1001, (m, m)).astype(np.int32)
    src32 = Tensor(torch.from_numpy(I.view(np.uint8).reshape(-1)).to("cuda:1"), "int32", [m, m], [4 * m, 4])     # transposed view
    t = timed(lambda: ops.copy(src32, dst64))
    ok = bool(np.array_equal(dst64.numpy(), I.astype(np.float64)))
    plain32 = timed(lambda: raw_dst[: 4 * m * m].copy_(src32.storage[: 4 * m * m], non_blocking=True))
    rows.append({"op": "OcTensorGPU_copy i32 4096^2 transposed on GPU 1 -> f64 dense on GPU 0 (4 bytes over the link, 8 written)",
                 "us": t * 1e6, "link_gbs": 4 * m * m / t / 1e9, "plain_peer_copy_of_the_source_gbs": 4 * m * m / plain32 / 1e9,
                 "of_plain_peer_copy": plain32 / t, "checked": ok})
    print(json.dumps({"peer_copy": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2n", type=int, default=32, help="log2 of the total element count (32 = the named workload)")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-operation table of configurations 1-4")
    ap.add_argument("--no-cpu", action="store_true", help="skip the Solid CPU baselines")
    ap.add_argument("--ops-only", default=None, choices=["C1", "C2", "C3", "C4"],
                    help="run only the per-operation rows of one configuration, a few calls each, and print them "
                         "(a small case for profilers; no headline measurement)")
    ap.add_argument("--peer-copy", action="store_true", help="time the cross-device copy between GPUs 0 and 1 (one process)")
    args = ap.parse_args()
    if args.peer_copy:
        run_peer_copy(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.ops_only:
        import torch
        torch.cuda.set_device(0)
        peak, _ = measured_peak()
        print(json.dumps({"ops": ops_table(peak, with_cpu=False, only=args.ops_only, iters_scale=0.1, checks_on=False)}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
