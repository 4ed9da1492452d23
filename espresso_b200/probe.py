"""Kernel-level probes of the library: times one stand-alone kernel on a matrix of a chosen shape.

    python -m espresso_b200.probe gemm --rows 32768 --cols 4096 --batch 64 --type f16
    python -m espresso_b200.probe gemv --rows 32768 --cols 4096 --type q8_0

Prints one JSON line (mean kernel milliseconds, GB/s over the algorithmic bytes, TFLOP/s for the GEMM).  The same
command is what the profiler captures for the kernel summaries: it launches nothing but the probed kernel (plus, for a
K-sliced GEMM, the clearing of its output).
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import gguf_quant, runtime

BYTES_PER_WEIGHT = {"f16": 2.0, "bf16": 2.0, "q8_0": 34 / 32, "q4_0": 18 / 32}


def stored_matrix(kind: str, w: np.ndarray) -> np.ndarray:
    if kind == "f16":
        return w.astype(np.float16)
    if kind == "bf16":
        return (w.view(np.uint32) >> 16).astype(np.uint16)
    return gguf_quant.quantize(kind, w)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("kernel", choices=["gemm", "gemv"])
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=64, help="gemm: activation rows (1..256)")
    ap.add_argument("--type", default="f16", choices=sorted(BYTES_PER_WEIGHT))
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iterations", type=int, default=40)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args()

    rng = np.random.default_rng(3)
    w = rng.standard_normal((args.rows, args.cols)).astype(np.float32) * np.float32(0.02)
    stored = stored_matrix(args.type, w)
    wbytes = args.rows * args.cols * BYTES_PER_WEIGHT[args.type]
    if args.kernel == "gemm":
        x = rng.standard_normal((args.batch, args.cols)).astype(np.float32)
        _, ms = runtime.gemm_tc_bench(args.type, stored, args.rows, args.cols, x, args.warmup, args.iterations, args.device)
        nbytes = wbytes + args.batch * args.cols * 2 + args.batch * args.rows * 4
        flops = 2.0 * args.rows * args.cols * args.batch
    else:
        x = rng.standard_normal(args.cols).astype(np.float32)
        copies = max(2, int(400e6 // wbytes) + 1)  # rotate copies so that reads miss L2
        _, ms = runtime.gemv_bench(args.type, stored, args.rows, args.cols, x, args.warmup, args.iterations, copies, args.device)
        nbytes = wbytes + args.cols * 4 + args.rows * 4
        flops = 2.0 * args.rows * args.cols
    print(json.dumps({"kernel": args.kernel, "type": args.type, "rows": args.rows, "cols": args.cols,
                      "batch": args.batch if args.kernel == "gemm" else 1, "ms": ms, "algorithmic_bytes": nbytes,
                      "GBps": nbytes / (ms / 1e3) / 1e9, "TFLOPs": flops / (ms / 1e3) / 1e12}))


if __name__ == "__main__":
    main()
