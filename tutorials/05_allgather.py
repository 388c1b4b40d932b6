"""Tutorial 05 - all-gather with the device primitives: push + per-source signal, and ``fcollect`` + barrier.

The kernels are in ``05_allgather.cu``. Both write into a symmetric ``[world, n]`` buffer; the script checks them
against ``torch.distributed.all_gather_into_tensor``.

    python tutorials/05_allgather.py                       # one GPU
    bash launch.sh --nproc 8 tutorials/05_allgather.py     # eight ranks over NVSwitch

Reference counterpart: ``tutorials/02-intra-node-allgather.py``. The library's own all-gather kernels (pull, push,
low-latency packets, packets over multimem) are ``triton_distributed_b200.kernels.nvidia.fast_allgather``.
"""
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import _lib, utils
from triton_distributed_b200.build import compile_extension


def run(rounds: int = 3, n: int = 64 * 1024) -> None:
    ext = ctypes.CDLL(str(compile_extension(os.path.join(os.path.dirname(os.path.abspath(__file__)), "05_allgather.cu"))))
    heap = utils.get_heap()
    rank, world = heap.rank, heap.world
    out = heap.create_tensor((world, n), torch.int32)      # symmetric: slot r sits at the same offset on every rank
    sync = [heap.create_tensor((16,), torch.int32) for _ in range(2)]  # one counter / flag block per variant, never reset
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    for variant, name in ((0, "push + signal"), (1, "fcollect + barrier")):
        for r in range(rounds):
            src = torch.randint(0, 1 << 20, (n,), device="cuda", dtype=torch.int32) + rank
            want = torch.empty((world, n), dtype=torch.int32, device="cuda")
            if world > 1:
                dist.all_gather_into_tensor(want, src)
            else:
                want[0] = src
            heap.barrier_all()  # no rank overwrites a slot that a slower peer is still comparing
            rc = ext.tutorial_allgather(heap.ctx, variant, ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(out.data_ptr()), n,
                                        ctypes.c_void_p(sync[variant].data_ptr()), ctypes.c_uint(r),
                                        ctypes.c_void_p(ok.data_ptr()), _lib.stream_ptr())
            assert rc == 0, f"launch failed: {rc}"
            torch.cuda.synchronize()
            heap.check_status(f"tutorial 05 ({name})")
            assert int(ok.item()) == 1 and torch.equal(out, want), f"{name}: mismatch in round {r}"
    heap.barrier_all()
    torch.cuda.synchronize()
    for t in sync + [out]:
        heap.free(t)
    utils.dist_print(f"tutorial 05: all-gather of {n} words, two variants x {rounds} rounds passed on {world} rank(s)",
                     allowed_ranks=[0])


if __name__ == "__main__":
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29575")):
        os.environ.setdefault(k, v)
    utils.initialize_distributed(seed=0, heap_bytes=256 << 20)
    run()
    utils.finalize_distributed()
