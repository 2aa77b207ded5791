"""Throughput of the HBM-bound operators (unary, binary, reductions,
contiguous() of a transposed view) against the measured copy bandwidth.

    python ops_bench.py [--rows R --cols C] [--reps N] [--only NAME]

Prints one JSON line per case: algorithmic bytes (every input element read
once, every output element written once), CUDA-event time per launch and the
fraction of the HBM copy rate in MEASURED_PEAKS.json at the repository root
(6650 GB/s when that file is absent).  Inputs are larger than L2."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from oxmera_b200 import B200Backend, DType, Tensor  # noqa: E402


def _peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"])
    except Exception:
        return 6650.0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16000)
    ap.add_argument("--cols", type=int, default=16400)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--only", default=None, help="run only the cases whose name contains this")
    args = ap.parse_args()
    be = B200Backend(0)
    peak = _peak_gbs()
    R, C = args.rows, args.cols
    n = R * C

    def timed(fn):
        fn()
        be.synchronize()
        tm = be.timer()
        tm.start()
        for _ in range(args.reps):
            fn()
        tm.stop()
        return tm.elapsed_ms() / args.reps

    for dtype in (DType.F32, DType.BF16):
        esz = dtype.size_in_bytes()
        a = be.synthetic((R, C), dtype, 1, 0)
        b = be.synthetic((R, C), dtype, 1, 1)
        bt = be.synthetic((C, R), dtype, 1, 2).permute([1, 0])  # a transposed view of shape [R, C]
        row = be.synthetic((C,), dtype, 1, 3)
        cases = [
            ("exp", lambda: be.exp(a), 2 * n),
            ("add contiguous", lambda: be.add(a, b), 3 * n),
            ("add row broadcast", lambda: be.add(a, row), 2 * n),
            ("add transposed view", lambda: be.add(a, bt), 3 * n),
            ("neg transposed view", lambda: be.neg(bt), 2 * n),
            ("contiguous of transposed view", lambda: bt.contiguous(), 2 * n),
            ("sum rows", lambda: be.sum(a, [1]), n),
            ("sum columns", lambda: be.sum(a, [0]), n),
            ("sum all", lambda: be.sum(a, []), n),
            ("max rows", lambda: be.max(a, [1]), n),
        ]
        for name, fn, elems in cases:
            if args.only and args.only not in name:
                continue
            ms = timed(fn)
            gbs = elems * esz / ms / 1e6
            print(json.dumps({"op": name, "dtype": dtype.name.lower(), "shape": [R, C], "bytes": elems * esz,
                              "ms": round(ms, 4), "gb_per_s": round(gbs, 1), "frac_of_hbm_copy": round(gbs / peak, 3),
                              "kernel": be.last_kernel()}), flush=True)
        del a, b, bt, row


if __name__ == "__main__":
    main()
