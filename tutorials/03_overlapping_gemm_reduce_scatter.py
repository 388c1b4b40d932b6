"""Tutorial 03 - a GEMM overlapped with its reduce-scatter (row-parallel linear, output sharded by rows).

Every rank multiplies the full batch by its K-shard of the weight; the partial sums of rows that belong to rank r must
be added up on rank r. ``gemm_rs`` is ONE kernel: the epilogue of every finished tile stores it straight into the
owner's slot over NVLink, a signalling warp bumps the owner's arrival counter, and owners reduce the slots of a row
block as soon as every source has delivered it.

    bash launch.sh --nproc 8 tutorials/03_overlapping_gemm_reduce_scatter.py --m 8192

Reference counterpart: ``tutorials/08-overlapping-gemm-reduce-scatter.py``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import utils
from triton_distributed_b200.kernels.nvidia import create_gemm_rs_context, gemm_rs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=28672, help="total reduction dim (all ranks)")
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29573")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=2 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    a = torch.randn(args.m, args.k // world, device="cuda", dtype=torch.bfloat16) * 0.1
    b = torch.randn(args.n, args.k // world, device="cuda", dtype=torch.bfloat16) * 0.02      # [N, K / world]
    ctx = create_gemm_rs_context(args.m, args.n, rank, world, world, torch.bfloat16)
    out = gemm_rs(a, b, ctx)                                                                  # [M / world, N]
    part = (a @ b.t()).float()
    want = torch.empty(args.m // world, args.n, device="cuda", dtype=torch.float32)
    if world > 1:
        dist.reduce_scatter_tensor(want, part, group=group)
    else:
        want.copy_(part)
    utils.assert_allclose(out.float(), want, rtol=3e-2, atol=3e-2 * world)
    utils.get_heap().check_status("gemm_rs")
    full = torch.empty(args.m, args.n, device="cuda", dtype=torch.bfloat16)
    shard = torch.empty(args.m // world, args.n, device="cuda", dtype=torch.bfloat16)

    def baseline():
        torch.matmul(a, b.t(), out=full)
        if world > 1:
            dist.reduce_scatter_tensor(shard, full, group=group)
        return shard

    _, _, t_fused = utils.perf_func_cold(lambda: gemm_rs(a, b, ctx), 10, 3)
    _, _, t_base = utils.perf_func_cold(baseline, 10, 3)
    fused, base = utils.max_over_ranks(min(t_fused), group), utils.max_over_ranks(min(t_base), group)
    utils.dist_print(f"tutorial 03: M={args.m} N={args.n} K/r={args.k // world} on {world} rank(s): fused {fused * 1e3:.1f} us, "
                     f"matmul + reduce-scatter {base * 1e3:.1f} us ({base / fused:.2f}x)", allowed_ranks=[0])
    ctx.finalize()
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
