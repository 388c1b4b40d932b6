"""Tutorial 02 - all-gather overlapped with a GEMM (column-parallel linear on sequence-sharded activations).

Every rank holds M / world rows of A and its own shard of the weight. ``ag_gemm`` is ONE kernel: communication warps
move the peers' rows over NVLink into a symmetric buffer and raise per-row-block flags, while the tcgen05 mainloop
multiplies the row blocks that have already landed (its own rows first). The script checks the result against
``all_gather_into_tensor`` + ``matmul`` and times both.

    bash launch.sh --nproc 8 tutorials/02_overlapping_allgather_gemm.py --m 8192

Reference counterpart: ``tutorials/07-overlapping-allgather-gemm.py``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import utils
from triton_distributed_b200.kernels.nvidia import ag_gemm, create_ag_gemm_context


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096, help="total rows (all ranks)")
    ap.add_argument("--n", type=int, default=28672, help="total output features (all ranks)")
    ap.add_argument("--k", type=int, default=8192)
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29572")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=2 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    a = torch.randn(args.m // world, args.k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(args.n // world, args.k, device="cuda", dtype=torch.bfloat16) * 0.02      # [N / world, K]
    # 1. a context owns the symmetric gather buffer and the flags; it is reused by every call of this shape or smaller
    ctx = create_ag_gemm_context(a, b, rank, world, max_M=args.m)
    # 2. the fused op
    c = ag_gemm(a, b, ctx)
    # 3. golden: NCCL all-gather, then cuBLAS
    full = torch.empty(args.m, args.k, device="cuda", dtype=torch.bfloat16)
    if world > 1:
        dist.all_gather_into_tensor(full, a, group=group)
    else:
        full.copy_(a)
    want = full @ b.t()
    utils.assert_allclose(c, want, rtol=2e-2, atol=2e-2)
    utils.get_heap().check_status("ag_gemm")

    def baseline():
        if world > 1:
            dist.all_gather_into_tensor(full, a, group=group)
        return torch.matmul(full, b.t())

    _, _, t_fused = utils.perf_func_cold(lambda: ag_gemm(a, b, ctx), 10, 3)
    _, _, t_base = utils.perf_func_cold(baseline, 10, 3)
    fused, base = utils.max_over_ranks(min(t_fused), group), utils.max_over_ranks(min(t_base), group)
    utils.dist_print(f"tutorial 02: M={args.m} N/r={args.n // world} K={args.k} on {world} rank(s): fused {fused * 1e3:.1f} us, "
                     f"all-gather + matmul {base * 1e3:.1f} us ({base / fused:.2f}x), gather = {ctx.method_for(args.m // world)}",
                     allowed_ranks=[0])
    ctx.finalize()
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
