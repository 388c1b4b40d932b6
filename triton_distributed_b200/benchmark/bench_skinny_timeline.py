"""Per-CTA timeline of the decode GEMM inside a chain of dependent launches.

Every CTA of ``gemm_skinny_kernel`` stamps ``%globaltimer`` at eight checkpoints when a trace buffer is installed
(``b200_gemm_skinny_set_trace``). This script captures six back-to-back GEMMs of one shape in a CUDA graph (programmatic
dependent launch between them, different weights each so nothing is cached) and prints, for two of the later calls,
when each checkpoint was reached by the slowest CTA, in microseconds after the previous kernel's last CTA finished.
What it shows is the fixed cost of a decode GEMM beyond its weight stream: dependency hand-over, first activation
load, MMA drain, and the stream-K fix-up through L2.

    python -m triton_distributed_b200.benchmark.bench_skinny_timeline [--tokens 8]
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from .. import _lib, ops

CHECKPOINTS = ["cta start", "setup done", "dependency seen", "last MMA issued", "accumulator complete",
               "partials added + fenced", "ticket drawn", "cta done"]
SHAPES = [  # name, N, K, swiglu: Qwen3-32B projections of one rank at TP8 and the qkv projection at TP1
    ("tp8 qkv", 1280, 5120, False), ("tp8 o_proj", 5120, 1024, False), ("tp8 gate_up", 3200, 5120, True),
    ("tp8 down", 5120, 3200, False), ("tp1 qkv", 10240, 5120, False)]


def timeline(M: int, N: int, K: int, swiglu: bool, calls: int = 6) -> list[dict]:
    dev = "cuda"
    lib = _lib.load()
    rows = 2 * N if swiglu else N
    ws = [torch.randn(rows, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(calls)]
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    bufs = [torch.zeros(160, 8, dtype=torch.int64, device=dev) for _ in range(calls)]
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

    def chain():
        for i in range(calls):
            lib.b200_gemm_skinny_set_trace(ctypes.c_void_p(bufs[i].data_ptr()))
            ops.gemm_skinny(x, ws[i], out=out, swiglu=swiglu)
        lib.b200_gemm_skinny_set_trace(None)

    chain()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    t = torch.stack(bufs).cpu()  # [calls, cta, checkpoint] in ns
    res = []
    for i in (3, 4):
        cur, prev = t[i][t[i][:, 0] > 0], t[i - 1][t[i - 1][:, 0] > 0]
        t0 = int(prev[:, 7].max())
        row = {"call": i, "ctas": int(cur.shape[0]), "first_cta_start_us": (int(cur[:, 0].min()) - t0) / 1e3}
        for c, name in enumerate(CHECKPOINTS):
            v = cur[:, c][cur[:, c] > 0]
            row[name] = (int(v.max()) - t0) / 1e3 if len(v) else float("nan")
        res.append(row)
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8)
    args = ap.parse_args()
    for name, N, K, swiglu in SHAPES:
        for row in timeline(args.tokens, N, K, swiglu):
            marks = "  ".join(f"{k} {row[k]:+.2f}" for k in CHECKPOINTS)
            print(f"{name:12s} {args.tokens}x{N}x{K} call {row['call']}: {row['ctas']} CTAs, first start "
                  f"{row['first_cta_start_us']:+.2f} | slowest CTA (us after the previous kernel's last CTA): {marks}")


if __name__ == "__main__":
    main()
