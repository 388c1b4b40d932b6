"""AG-GEMM and GEMM-RS against the NCCL + cuBLAS composition, Llama-3-70B MLP shapes, TP = world size.

  AG-GEMM   A [M / r, 8192] gathered, times W_gate_up shard [57344 / r, 8192]
  GEMM-RS   A [M, 28672 / r] times W_down shard [8192, 28672 / r], reduce-scattered to [M / r, 8192]

Every number is device-timed with CUDA events, L2 flushed before each call, and reported as the
maximum over ranks of the per-rank minimum over iterations. The roofline of a fused kernel is the
slower of its FLOPs at the measured cuBLAS peak and its NVLink bytes at the measured peer bandwidth.

Run: ``python -m torch.distributed.run --nproc-per-node N -m triton_distributed_b200.benchmark.bench_comm_gemm``
Role in the reference: ``python/triton_dist/benchmark/bench_allgather_gemm.py``, ``test/nvidia/test_gemm_rs.py`` perf mode.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import utils
from ..kernels.nvidia import ag_gemm, create_ag_gemm_context, create_gemm_rs_context, gemm_rs

PEAK_TFLOPS = 1605.6   # measured cuBLAS bf16 burst on this pool
LINK_GBS = 770.0       # measured peer copy per direction


def _time(fn, iters, warmup, group):
    _, _, ts = utils.perf_func_cold(fn, iters, warmup)
    return utils.max_over_ranks(min(ts), group)


def bench_pair(group, ms, iters: int, warmup: int, rows: list, hidden: int = 8192, inter: int = 28672,
               both_gathers: bool = True) -> None:
    """Append one AG-GEMM and one GEMM-RS row per M in `ms` (an int or a list) to `rows`."""
    rank, world = dist.get_rank(), dist.get_world_size()
    ms = [ms] if isinstance(ms, int) else list(ms)
    H, I = hidden, inter
    n_ag = 2 * I // world   # gate_up shard rows
    k_rs = I // world
    dt = torch.bfloat16
    maxM = max(ms)
    w1 = torch.randn(n_ag, H, device="cuda", dtype=dt) * 0.02
    w2 = torch.randn(H, k_rs, device="cuda", dtype=dt) * 0.02
    ag_ctx = create_ag_gemm_context(torch.empty(maxM // world, H, device="cuda", dtype=dt), w1, rank, world, maxM)
    rs_ctx = create_gemm_rs_context(maxM, H, rank, world, world, dt)
    for M in ms:
        a = torch.randn(M // world, H, device="cuda", dtype=dt)
        full = torch.empty(M, H, device="cuda", dtype=dt)
        c = torch.empty(M, n_ag, device="cuda", dtype=dt)

        def base_ag():
            if world > 1:
                dist.all_gather_into_tensor(full, a, group=group)
                torch.matmul(full, w1.t(), out=c)
            else:
                torch.matmul(a, w1.t(), out=c)

        t_ours = _time(lambda: ag_gemm(a, w1, ag_ctx, out=c), iters, warmup, group)
        chosen = ag_ctx.method_for(M // world)
        by_method = {}
        if world > 1 and both_gathers:  # both gathers, so that the automatic choice can be checked against the data
            for m in ("sm_push_fused", "sm_pull_fused"):
                ag_ctx.all_gather_method = m
                by_method[m] = _time(lambda: ag_gemm(a, w1, ag_ctx, out=c), iters, warmup, group) * 1e3
            ag_ctx.all_gather_method = "auto"
        t_base = _time(base_ag, iters, warmup, group)
        flops = 2.0 * M * n_ag * H
        nv_bytes = (world - 1) * (M // world) * H * 2
        roof = max(flops / (PEAK_TFLOPS * 1e9), nv_bytes / (LINK_GBS * 1e6))
        rows.append({"op": "ag_gemm", "world": world, "M": M, "N": n_ag, "K": H, "ours_us": t_ours * 1e3,
                     "nccl_cublas_us": t_base * 1e3, "speedup": t_base / t_ours, "roofline_us": roof * 1e3,
                     "frac_of_roofline": roof / t_ours, "tflops": flops / t_ours / 1e9, "gather": chosen,
                     "push_us": by_method.get("sm_push_fused"), "pull_us": by_method.get("sm_pull_fused")})
        x = torch.randn(M, k_rs, device="cuda", dtype=dt) * 0.1
        part = torch.empty(M, H, device="cuda", dtype=dt)
        out = torch.empty(M // world, H, device="cuda", dtype=dt)

        def base_rs():
            torch.matmul(x, w2.t(), out=part)
            if world > 1:
                dist.reduce_scatter_tensor(out, part, group=group)

        # both reduction modes of the fused kernel: per-source slots summed by the owner, and the in-switch reduction
        modes = {}
        default_nvls = rs_ctx.nvls
        for name, nvls in (("slots", False), ("nvls", True)):
            if nvls and not (rs_ctx.heap.has_multicast and world > 1):
                continue
            rs_ctx.nvls = nvls
            modes[name] = _time(lambda: gemm_rs(x, w2, rs_ctx, out=out), iters, warmup, group)
        rs_ctx.nvls = default_nvls
        auto_nvls = rs_ctx.use_nvls(M)
        t_ours = modes["nvls" if auto_nvls and "nvls" in modes else "slots"]
        t_base = _time(base_rs, iters, warmup, group)
        flops = 2.0 * M * H * k_rs
        nv_bytes = (world - 1) * (M // world) * H * 2
        roof = max(flops / (PEAK_TFLOPS * 1e9), nv_bytes / (LINK_GBS * 1e6))
        rows.append({"op": "gemm_rs", "world": world, "M": M, "N": H, "K": k_rs, "ours_us": t_ours * 1e3,
                     "nccl_cublas_us": t_base * 1e3, "speedup": t_base / t_ours, "roofline_us": roof * 1e3,
                     "frac_of_roofline": roof / t_ours, "tflops": flops / t_ours / 1e9,
                     "reduce_mode": "nvls" if auto_nvls else "slots",
                     "modes_us": {k: v * 1e3 for k, v in modes.items()}})
    utils.get_heap().check_status("bench_comm_gemm")
    ag_ctx.finalize()
    rs_ctx.finalize()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ms", type=int, nargs="+", default=[1024, 2048, 4096, 8192])
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    group = utils.initialize_distributed(seed=0, heap_bytes=4 << 30)
    rank = dist.get_rank()
    rows: list[dict] = []
    bench_pair(group, args.ms, args.iters, args.warmup, rows, args.hidden, args.inter)
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(rows, f, indent=1)
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
