"""Stand-alone reduce-scatter over the symmetric heap.

API parity with ``python/triton_dist/kernels/nvidia/reduce_scatter.py`` (``create_reduce_scater_2d_ctx`` :147 [sic],
``reduce_scatter_2d_op`` :873, ``ring_reduce`` :830). The reference scatters with copy-engine memcpys gated on
flags and then runs a ring-reduce kernel; on one NVSwitch node a single push + slot-reduce kernel does both. The
ring-push variants for PCIe / non-full-mesh boxes (:284-513) have no use behind an NVSwitch and are not provided.
"""
from __future__ import annotations

import dataclasses

import torch

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap


@dataclasses.dataclass
class ReduceScatter2DContext:
    max_M: int
    N: int
    rank: int
    world_size: int
    local_world_size: int
    dtype: torch.dtype
    heap: SymmHeap
    workspaces: list[torch.Tensor]
    flags: torch.Tensor
    sync: torch.Tensor

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.workspaces + [self.flags]:
            self.heap.free(t)
        self.workspaces = []


def create_reduce_scater_2d_ctx(max_M: int, N: int, rank: int, world_size: int, local_world_size: int, dtype: torch.dtype,
                                overlap_with_gemm: bool = True, num_reduction_sms: int = 16) -> ReduceScatter2DContext:
    heap = get_heap()
    ws = [heap.create_tensor((max_M, N), dtype, align=1024) for _ in range(2)]
    flags = heap.create_tensor((2 * 64 * 8,), torch.int32)
    ctx = ReduceScatter2DContext(max_M, N, rank, world_size, local_world_size, dtype, heap, ws, flags,
                                 torch.zeros(4, dtype=torch.int32, device="cuda"))
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


create_reduce_scatter_2d_ctx = create_reduce_scater_2d_ctx


def reduce_scatter_2d_op(input: torch.Tensor, ctx: ReduceScatter2DContext, output: torch.Tensor | None = None) -> torch.Tensor:
    """input [M, N] (every rank's partial) -> this rank's rows [M / world, N] of the sum."""
    M, N = input.shape
    if M % ctx.world_size or M > ctx.max_M or N != ctx.N or not input.is_contiguous():
        raise ValueError("input does not fit the context")
    per = M // ctx.world_size
    if output is None:
        output = torch.empty((per, N), dtype=input.dtype, device=input.device)
    nbytes = per * N * input.element_size()
    _lib.call("b200_reduce_scatter", ctx.heap.ctx, ptr(input), ptr(output), _lib.c_u64(nbytes), dtype_code(input.dtype),
              ptr(ctx.workspaces[0]), ptr(ctx.workspaces[1]), ptr(ctx.flags), ptr(ctx.sync),
              max(1, min(64, nbytes // (64 * 1024))), stream_ptr())
    ops._count()
    return output


def ring_reduce(input: torch.Tensor, output: torch.Tensor, begin_idx: int, num_splits: int, num_sms: int = -1) -> torch.Tensor:
    """output = sum of the `num_splits` equal row blocks of `input`, added in ring order starting after `begin_idx`."""
    per = input.shape[0] // num_splits
    acc = torch.zeros_like(output, dtype=torch.float32)
    for i in range(num_splits):
        k = (begin_idx + 1 + i) % num_splits
        acc += input[k * per:(k + 1) * per].float()
    output.copy_(acc.to(output.dtype))
    return output
