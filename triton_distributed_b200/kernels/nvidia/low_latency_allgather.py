"""Small-message all-gather on a symmetric buffer.

API parity with ``python/triton_dist/kernels/nvidia/low_latency_allgather.py``
(``create_fast_allgather_context`` :805, ``fast_allgather`` :975). The buffer is symmetric,
``[world, bytes_per_rank]`` with slot ``rank`` pre-filled; after the call every slot is filled.
Behind an NVSwitch the reference's 2D / 3D / NUMA variants have no topology to exploit, so they map
onto the push and LL kernels (``csrc/kernels/comm_ops.cu``).
"""
from __future__ import annotations

import dataclasses

import torch

from ... import _lib, ops
from ..._lib import ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap

_MODES = {
    "pull": 0,
    "push2d": 1, "push3d": 1, "push_numa_2d": 1,
    "push2d_ll": 2, "push3d_ll": 2, "push_numa_2d_ll": 2, "push_numa_2d_ll_multinode": 2,
    "push2d_ll_multimem": 3,
}


@dataclasses.dataclass
class FastAllGatherContext:
    rank: int
    node: int
    num_ranks: int
    num_nodes: int
    max_buffer_size: int
    heap: SymmHeap
    ll_buffers: list[torch.Tensor]  # two parity packet areas, 2x the payload each
    flags: torch.Tensor
    sync: torch.Tensor
    max_ctas: int

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.ll_buffers + [self.flags]:
            self.heap.free(t)
        self.ll_buffers = []


def create_fast_allgather_context(rank: int, node: int, num_ranks: int, num_nodes: int,
                                  max_buffer_size: int = 2 * 32 * 1024 * 1024) -> FastAllGatherContext:
    """`max_buffer_size` bounds the gathered bytes (all ranks together) the LL modes can move."""
    if num_nodes != 1:
        raise NotImplementedError("single node only: the inter-node paths of the reference are out of scope")
    heap = get_heap()
    lib = _lib.load()
    max_ctas = lib.b200_allgather_max_ctas()
    ll = [heap.create_tensor((max(2 * max_buffer_size, 16),), torch.uint8, align=1024) for _ in range(2)]
    flags = heap.create_tensor((2 * max_ctas * 8,), torch.int32)
    ctx = FastAllGatherContext(rank, node, num_ranks, num_nodes, max_buffer_size, heap, ll, flags,
                               torch.zeros(4, dtype=torch.int32, device="cuda"), max_ctas)
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def fast_allgather(symm_buffer: torch.Tensor, ctx: FastAllGatherContext | None = None, rank: int | None = None,
                   node: int | None = None, num_ranks: int | None = None, num_nodes: int | None = None,
                   mode: str = "pull", num_ctas: int = 0) -> torch.Tensor:
    """In-place all-gather of a symmetric buffer viewed as ``[world, bytes_per_rank]``."""
    if ctx is None:
        raise ValueError("fast_allgather needs a context from create_fast_allgather_context")
    if mode not in _MODES:
        raise ValueError(f"unknown mode {mode!r}; choose from {sorted(_MODES)}")
    if not ctx.heap.is_symmetric(symm_buffer) or not symm_buffer.is_contiguous():
        raise ValueError("fast_allgather needs a contiguous tensor from the symmetric heap")
    nbytes = symm_buffer.numel() * symm_buffer.element_size()
    if nbytes % ctx.num_ranks != 0:
        raise ValueError("buffer bytes must be divisible by the number of ranks")
    per_rank = nbytes // ctx.num_ranks
    native = _MODES[mode]
    if native >= 2 and nbytes > ctx.max_buffer_size:
        raise ValueError("message larger than the context's LL packet area")
    if num_ctas <= 0:
        num_ctas = max(1, min(ctx.max_ctas, per_rank // (16 * 1024)))
    _lib.call("b200_allgather", ctx.heap.ctx, ptr(symm_buffer), _lib.c_u64(per_rank), ptr(ctx.ll_buffers[0]),
              ptr(ctx.ll_buffers[1]), ptr(ctx.flags), ptr(ctx.sync), native, num_ctas, stream_ptr())
    ops._count()
    return symm_buffer
