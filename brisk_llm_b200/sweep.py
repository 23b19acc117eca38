"""Kernel sweep: the quantised multiply on its own, every format x the sweep shapes x 1, 4, 9 and 512 tokens.

    python -m brisk_llm_b200.sweep [--formats Q4_0,Q8_0,...] [--quick]

Method of the reference's kernel_bench (brisk-llm bench/kernel_bench.cpp:61-90) carried to the GPU: weights f32
~N(0, 0.02) (ternary: uniform thirds) quantised to the format, activations random f32; the timed loop rotates over
enough repacked copies of the matrix that the working set exceeds the 126 MB L2, so every multiply streams its weights
from HBM. Reports microseconds per multiply, weight GB/s (n <= 8: HBM-bound) and GMAC/s (prompt batches).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import engine, formats as F

SHAPES = [(1024, 3072), (2048, 8192), (4096, 14336), (14336, 4096)]  # rows x cols
TOKENS = [1, 4, 9, 512]


def peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    return float(json.load(open(path))["hbm_gbs"]) if os.path.exists(path) else 6650.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--formats", default="Q4_0,Q8_0,Q4_K,Q6_K,TQ2_0")
    ap.add_argument("--quick", action="store_true", help="first and last shape only")
    ap.add_argument("--shapes", default="", help="rows x cols pairs instead of the grid's, e.g. 4096x14336,14336x4096")
    ap.add_argument("--tokens", default="", help="token counts instead of 1,4,9,512")
    ap.add_argument("--iterations", type=int, default=0, help="timed multiplies per case (default 200 up to 8 tokens, 20 beyond)")
    args = ap.parse_args()
    peak = peak_gbs()
    shapes = [SHAPES[0], SHAPES[-1]] if args.quick else SHAPES
    if args.shapes:
        shapes = [tuple(int(v) for v in pair.split("x")) for pair in args.shapes.split(",")]
    tokens = [int(v) for v in args.tokens.split(",")] if args.tokens else TOKENS
    rng = np.random.default_rng(0)
    print(f"{'format':6s} {'rows':>6s} {'cols':>6s} {'n':>4s} {'us':>9s} {'GB/s':>8s} {'of peak':>8s} {'GMAC/s':>9s}")
    for name in args.formats.split(","):
        fmt = F.BY_NAME[name]
        for rows, cols in shapes:
            if fmt == F.TQ2_0:
                w = rng.integers(-1, 2, size=(rows, cols)).astype(np.float32) * np.float32(0.02)
            else:
                w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
            wb = F.quantize(fmt, w)
            nbytes = wb.nbytes
            copies = max(2, int(300e6 // nbytes) + 1)
            for n in tokens:
                iters = args.iterations or (200 if n <= 8 else 20)
                sec = engine.matmul_seconds(fmt, wb, rows, cols, n, copies, iters)
                gbs = nbytes / sec / 1e9
                gmacs = rows * cols * n / sec / 1e9
                print(f"{name:6s} {rows:6d} {cols:6d} {n:4d} {sec * 1e6:9.2f} {gbs:8.1f} {gbs / peak:8.3f} {gmacs:9.1f}", flush=True)


if __name__ == "__main__":
    main()
