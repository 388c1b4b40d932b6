"""Tutorial 06 - reduce-scatter with the device primitives: pull + sum, and the in-switch sum (``multimem.ld_reduce``).

The kernel is in ``06_reduce_scatter.cu``; the script checks both variants against
``torch.distributed.reduce_scatter_tensor``.

    python tutorials/06_reduce_scatter.py                       # one GPU
    bash launch.sh --nproc 8 tutorials/06_reduce_scatter.py     # eight ranks over NVSwitch

Reference counterpart: ``tutorials/05-intra-node-reduce-scatter.py``. The library's own kernels are
``triton_distributed_b200.kernels.nvidia.reduce_scatter`` and the fused ``gemm_rs``.
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
    ext = ctypes.CDLL(str(compile_extension(os.path.join(os.path.dirname(os.path.abspath(__file__)), "06_reduce_scatter.cu"))))
    heap = utils.get_heap()
    rank, world = heap.rank, heap.world
    partial = heap.create_tensor((world, n), torch.float32)   # symmetric: peers read row [r] at the same offset
    flags = heap.create_tensor((16,), torch.int32)            # barrier flags, epochs only grow
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    epoch = 0
    variants = [(0, "pull")] + ([(1, "multimem")] if heap.has_multicast else [])
    for use_mc, name in variants:
        for r in range(rounds):
            heap.barrier_all()  # the previous round's readers are done before the partials change
            partial.copy_(torch.randn(world, n, device="cuda") * (rank + 1))
            want = torch.empty(n, dtype=torch.float32, device="cuda")
            if world > 1:
                dist.reduce_scatter_tensor(want, partial.clone())
            else:
                want.copy_(partial[0])
            epoch += 1
            rc = ext.tutorial_reduce_scatter(heap.ctx, ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(out.data_ptr()), n,
                                             ctypes.c_void_p(flags.data_ptr()), ctypes.c_uint(epoch), use_mc,
                                             ctypes.c_void_p(ok.data_ptr()), _lib.stream_ptr())
            assert rc == 0, f"launch failed: {rc}"
            torch.cuda.synchronize()
            heap.check_status(f"tutorial 06 ({name})")
            assert int(ok.item()) == 1, f"{name}: barrier timed out"
            torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-4 * world, msg=lambda s: f"{name} round {r}: {s}")
    heap.barrier_all()
    torch.cuda.synchronize()
    heap.free(flags), heap.free(partial)
    utils.dist_print(f"tutorial 06: reduce-scatter of {n} floats, {len(variants)} variant(s) x {rounds} rounds passed on "
                     f"{world} rank(s)", allowed_ranks=[0])


if __name__ == "__main__":
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29576")):
        os.environ.setdefault(k, v)
    utils.initialize_distributed(seed=0, heap_bytes=256 << 20)
    run()
    utils.finalize_distributed()
