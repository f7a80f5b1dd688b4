#!/usr/bin/env python3
"""Float64 sums of the headline workload, for the full-size parity test.

x, y = U(-1, 1) from the counter hash of bench.py (seeds 1 and 2) over 2^32 global indices,
z = float32(float32(0.5 * x) + y) as the reference's multiply-then-add sequence rounds it;
writes sum(z), sum(z*z) and norm2 = sqrt(sum(z*z)) accumulated in float64 (per 2^24-element
block with numpy's pairwise sum, blocks added in index order) to c5_constants.json beside this file.
Pure numpy, a few minutes on eight cores:

    python tests/golden/make_c5_constants.py [--log2n 32] [--workers 8]
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
BLOCK = 1 << 24


def block_sums(start: int):
    from bench import hash_uniform_numpy
    x = hash_uniform_numpy(start, BLOCK, 1)
    y = hash_uniform_numpy(start, BLOCK, 2)
    z = (np.float32(0.5) * x + y).astype(np.float32)          # two float32 roundings: the product is exact here
    z64 = z.astype(np.float64)
    return start, float(z64.sum()), float((z64 * z64).sum()), float(np.abs(z64).sum())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2n", type=int, default=32)
    ap.add_argument("--workers", type=int, default=8)
    a = ap.parse_args()
    n = 1 << a.log2n
    starts = list(range(0, n, BLOCK)) if n >= BLOCK else [0]
    assert n >= BLOCK, "sizes below 2^24 are covered by the ordinary parity tests"
    with ProcessPoolExecutor(a.workers) as pool:
        parts = sorted(pool.map(block_sums, starts, chunksize=4))
    s = math.fsum(p[1] for p in parts)
    q = math.fsum(p[2] for p in parts)
    m = math.fsum(p[3] for p in parts)
    out = {"log2n": a.log2n, "seeds": [1, 2], "a": 0.5, "sum": s, "sumsq": q, "norm2": math.sqrt(q), "sum_abs": m}
    path = HERE / "c5_constants.json"
    known = json.loads(path.read_text()) if path.exists() else {}
    known[str(a.log2n)] = out
    path.write_text(json.dumps(known, indent=1, sort_keys=True) + "\n")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
