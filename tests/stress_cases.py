"""Stress loop for the fused kernels: many back-to-back calls with random shapes, no host barrier between them, and a
straggler that rotates over the ranks, each result checked against the NCCL composition.

    bash launch.sh --nproc 8 tests/stress_cases.py --iters 40

Role in the reference: ``python/triton_dist/test/stress/stress_test_ag_gemm.py`` and the ``--stress`` mode of
``test/nvidia/test_allreduce.py:95-136``.
"""
import argparse
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import utils
from triton_distributed_b200.kernels.nvidia import (ag_gemm, all_reduce, all_reduce_rmsnorm, create_ag_gemm_context,
                                                    create_allreduce_ctx, create_gemm_rs_context, gemm_rs)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--straggler-ms", type=float, default=2.0)
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29575")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=3 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    heap = utils.get_heap()
    rng = random.Random(args.seed)  # same shape sequence on every rank
    K, N, maxM = 2048, 1536, 2048 * world
    w1 = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.02
    ag = create_ag_gemm_context(torch.empty(maxM // world, K, device="cuda", dtype=torch.bfloat16), w1, rank, world, maxM)
    rs = create_gemm_rs_context(maxM, K, rank, world, world, torch.bfloat16)
    ar = create_allreduce_ctx(8 << 20, rank, world, world)
    gamma = torch.randn(K, device="cuda", dtype=torch.bfloat16)
    spin = int(args.straggler_ms * 1.9e6)
    fails = torch.zeros(1, dtype=torch.int64, device="cuda")  # counted on the device: nothing synchronises the host in the loop
    checks = 0

    class pending:  # noqa: N801 - keeps the call sites below readable
        @staticmethod
        def append(item):
            nonlocal checks
            _, got, want, tol = item
            fails.add_((~torch.isclose(got, want, rtol=tol, atol=tol)).any().to(torch.int64))
            checks += 1
    for it in range(args.iters):
        mr = rng.choice([1, 3, 16, 100, 128, 257, 1000, 2048])          # rows per rank
        if it % world == rank:
            torch.cuda._sleep(spin)                                     # this rank arrives late at this iteration
        a = torch.randn(mr, K, device="cuda", dtype=torch.bfloat16)
        c = ag_gemm(a, w1, ag)                                          # [mr * world, N]
        full = torch.empty(mr * world, K, device="cuda", dtype=torch.bfloat16)
        if world > 1:
            dist.all_gather_into_tensor(full, a, group=group)
        else:
            full.copy_(a)
        pending.append((f"ag_gemm it{it} mr{mr}", c.float(), (full @ w1.t()).float(), 3e-2))
        act = (c * 0.1).contiguous()
        y = gemm_rs(act, w2, rs)                                        # [mr, K]
        part = (act @ w2.t()).float()
        want = torch.empty(mr, K, device="cuda", dtype=torch.float32)
        if world > 1:
            dist.reduce_scatter_tensor(want, part, group=group)
        else:
            want.copy_(part)
        pending.append((f"gemm_rs it{it} mr{mr}", y.float(), want, 3e-2 * world))
        rows = rng.choice([1, 8, 33, 256])
        x = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
        summed = x.float().clone()
        if world > 1:
            dist.all_reduce(summed, group=group)
        h = (summed + res.float()).to(torch.bfloat16).float()
        yn, hn = all_reduce_rmsnorm(x, res.clone(), gamma, 1e-6, ar)
        pending.append((f"ar_rmsnorm it{it} rows{rows}", hn.float(), h, 5e-2 * world))
        z = all_reduce(x, None, None, ar)
        pending.append((f"all_reduce it{it} rows{rows}", z.float(), summed, 5e-2 * world))
    torch.cuda.synchronize()
    heap.check_status("stress loop")
    t = fails.clone()
    if int(t.item()):
        print(f"[rank {rank}] {int(t.item())} of {checks} checks failed", flush=True)
    if world > 1:
        dist.all_reduce(t, group=group)
    if rank == 0:
        print(f"STRESS {'PASS' if int(t.item()) == 0 else 'FAIL'}: {args.iters} iterations, {checks} checks per rank, "
              f"{int(t.item())} mismatches on {world} rank(s)", flush=True)
    for c_ in (ag, rs, ar):
        c_.finalize()
    utils.finalize_distributed()
    return 0 if int(t.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
