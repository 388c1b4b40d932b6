"""Single-GPU GEMM benchmark: the tiled tcgen05 kernel or the decode (skinny) kernel against
``torch.matmul`` (cuBLAS), timed with CUDA events and an L2 flush between calls.

Role in the reference: ``python/triton_dist/benchmark/bench_allgather_gemm.py`` (shape sweep with a torch baseline).

Example: ``python -m triton_distributed_b200.benchmark.bench_gemm --kind tiled --m 4096 --n 4096 --k 4096``
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..utils import perf_func_cold


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--kind", choices=["tiled", "skinny", "swiglu"], default="tiled")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--dtype", choices=["bf16", "f16"], default="bf16")
    args = ap.parse_args()
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    torch.manual_seed(0)
    a = torch.randn(args.m, args.k, device="cuda", dtype=dt)
    rows = 2 * args.n if args.kind == "swiglu" else args.n
    b = torch.randn(rows, args.k, device="cuda", dtype=dt) * 0.05
    c = torch.empty(args.m, args.n, device="cuda", dtype=dt)
    if args.kind == "tiled":
        fn = lambda: ops.gemm(a, b, c)
    elif args.kind == "skinny":
        fn = lambda: ops.gemm_skinny(a, b, c)
    else:
        fn = lambda: ops.gemm_skinny(a, b, c, swiglu=True)
    _, ms, ts = perf_func_cold(fn, args.iters, args.warmup)
    flops = 2.0 * args.m * rows * args.k
    wbytes = 2.0 * rows * args.k
    out = {"kind": args.kind, "m": args.m, "n": args.n, "k": args.k, "ms_min": min(ts), "ms_mean": ms,
           "tflops": flops / min(ts) / 1e9, "weight_gbs": wbytes / min(ts) / 1e6}
    if not args.no_baseline:
        full = torch.empty(args.m, rows, device="cuda", dtype=dt)
        _, bms, bts = perf_func_cold(lambda: torch.matmul(a, b.t(), out=full), args.iters, args.warmup)
        out["torch_ms_min"] = min(bts)
        out["speedup_vs_torch"] = min(bts) / min(ts)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
