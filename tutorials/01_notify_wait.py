"""Tutorial 01 - notify / wait: a producer / consumer queue between neighbouring ranks.

The kernel is in ``01_notify_wait.cu`` (40 lines of device code against ``b200/primitives.cuh``). This script compiles
it for sm_100a, allocates the queue and its counter in the symmetric heap, runs it on every rank and checks the sum of
what the previous rank produced.

    python tutorials/01_notify_wait.py                                  # one GPU: the rank is its own neighbour
    bash launch.sh --nproc 2 tutorials/01_notify_wait.py                # two ranks over NVLink

Reference counterpart: ``tutorials/01-distributed-notify-wait.py``.
"""
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import _lib, utils
from triton_distributed_b200.build import compile_extension


def run(rounds: int = 3, chunks: int = 16, chunk_words: int = 4096) -> None:
    ext = ctypes.CDLL(str(compile_extension(os.path.join(os.path.dirname(os.path.abspath(__file__)), "01_notify_wait.cu"))))
    heap = utils.get_heap()
    rank, world = heap.rank, heap.world
    queue = heap.create_tensor((chunks * chunk_words,), torch.int32)   # symmetric: same offset on every rank
    counter = heap.create_tensor((1,), torch.int32)                    # chunks received so far, never reset
    total = torch.zeros(1, dtype=torch.int64, device="cuda")
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    for r in range(rounds):
        produced = torch.randint(0, 1000, (chunks * chunk_words,), device="cuda", dtype=torch.int32) + rank
        # what the previous rank produces this round (same generator state on every rank would be simpler; here the
        # sums are exchanged with the process group, which is only the golden)
        mine = produced.sum().to(torch.int64)
        sums = [torch.zeros_like(mine) for _ in range(world)]
        if world > 1:
            dist.all_gather(sums, mine)
        else:
            sums = [mine]
        heap.barrier_all()  # nobody overwrites the queue while a slower neighbour still reads the previous round
        rc = ext.tutorial_producer_consumer(heap.ctx, ctypes.c_void_p(produced.data_ptr()), ctypes.c_void_p(queue.data_ptr()),
                                            ctypes.c_void_p(counter.data_ptr()), ctypes.c_uint(r * chunks), chunks, chunk_words,
                                            ctypes.c_void_p(total.data_ptr()), ctypes.c_void_p(ok.data_ptr()),
                                            _lib.stream_ptr())
        assert rc == 0, f"launch failed: {rc}"
        torch.cuda.synchronize()
        heap.check_status("tutorial 01")   # a wait that ran out of its budget surfaces here, not as a hang
        want = int(sums[(rank - 1) % world])
        assert int(ok.item()) == 1 and int(total.item()) == want, (int(total.item()), want)
    heap.barrier_all()
    torch.cuda.synchronize()
    heap.free(counter), heap.free(queue)
    utils.dist_print(f"tutorial 01: {rounds} rounds x {chunks} chunks passed on {world} rank(s)", allowed_ranks=[0])


if __name__ == "__main__":
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29571")):
        os.environ.setdefault(k, v)
    utils.initialize_distributed(seed=0, heap_bytes=256 << 20)
    run()
    utils.finalize_distributed()
