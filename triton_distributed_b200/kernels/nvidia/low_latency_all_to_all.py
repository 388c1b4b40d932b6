"""Low-latency expert-parallel all-to-all on rows already sorted by expert.

API parity with ``python/triton_dist/kernels/nvidia/low_latency_all_to_all.py`` (``create_all_to_all_context`` :176,
``fast_all_to_all`` :198, ``all_to_all_post_process`` :260): the receive slot of source rank s starts at row
``s * max_m``; splits come back as ``[world, experts_per_rank]``; scales travel with their rows (one fp32 per row in
the reference, ``H / 128`` per row for block-quantised fp8 here as well).
"""
from __future__ import annotations

import dataclasses

import torch

from ... import _lib, ops
from ..._lib import ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap


@dataclasses.dataclass
class AllToAllContext:
    max_m: int
    hidden: int
    rank: int
    num_tot_experts: int
    WORLD_SIZE: int
    experts_per_rank: int
    dtype: torch.dtype
    scale_dtype: torch.dtype
    scale_per_row: int
    heap: SymmHeap
    recv_bufs: list[torch.Tensor]
    scale_recv_bufs: list[torch.Tensor]
    split_recv_bufs: list[torch.Tensor]
    flags: torch.Tensor
    sync: torch.Tensor
    calls: int = 0   # host mirror of the device-resident epoch (one per fast_all_to_all), so no call reads it back

    @property
    def call_count(self) -> int:
        return self.calls + 1

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.recv_bufs + self.scale_recv_bufs + self.split_recv_bufs + [self.flags]:
            self.heap.free(t)
        self.recv_bufs = []


def create_all_to_all_context(max_m: int, hidden: int, rank: int, num_tot_experts: int, WORLD_SIZE: int,
                              experts_per_rank: int, dtype=torch.bfloat16, scale_dtype=torch.float,
                              scale_per_row: int = 1) -> AllToAllContext:
    """max_m: most rows one rank may send to one peer in a call."""
    heap = get_heap()
    if WORLD_SIZE != heap.world:
        raise ValueError("the all-to-all spans the ranks of the symmetric heap (single node)")
    recv = [heap.create_tensor((WORLD_SIZE * max_m, hidden), dtype, align=1024) for _ in range(2)]
    srecv = [heap.create_tensor((WORLD_SIZE * max_m, scale_per_row), torch.float32) for _ in range(2)]
    splits = [heap.create_tensor((WORLD_SIZE, experts_per_rank), torch.int32) for _ in range(2)]
    flags = heap.create_tensor((16,), torch.int32)
    ctx = AllToAllContext(max_m, hidden, rank, num_tot_experts, WORLD_SIZE, experts_per_rank, dtype, scale_dtype,
                          scale_per_row, heap, recv, srecv, splits, flags, torch.zeros(4, dtype=torch.int32, device="cuda"))
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def fast_all_to_all(ctx: AllToAllContext, send_tensor: torch.Tensor, send_split_cumsum: torch.Tensor,
                    send_scale: torch.Tensor | None = None):
    """send_tensor [n, hidden] sorted by global expert; send_split_cumsum int32 [E + 1]; send_scale fp32 [n] or
    [n, scale_per_row]. Returns [recv_splits [world, E_local], recv_buf [world * max_m, hidden], recv_scale | None]
    (views of the buffer half used by this call; valid until the call after next). A rank may send at most
    ``ctx.max_m`` rows to one peer: rows beyond that are dropped by the kernel and reported through the heap's status
    word (``SymmHeap.check_status`` raises), never written past the peer's receive area."""
    if not send_tensor.is_contiguous() or send_tensor.dtype != ctx.dtype or send_tensor.shape[1] != ctx.hidden:
        raise ValueError("send_tensor must be contiguous [n, hidden] in the context dtype")
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("fast_all_to_all cannot be captured in a CUDA graph: the returned views name the buffer half "
                           "of this call, which the host selects from its call counter")
    cum = send_split_cumsum.to(torch.int32).contiguous()
    ctx.calls += 1
    par = ctx.calls & 1
    sc = None
    if send_scale is not None:
        sc = send_scale.reshape(send_tensor.shape[0], -1).float().contiguous()
        if sc.shape[1] != ctx.scale_per_row:
            raise ValueError("send_scale does not match the context's scales per row")
    _lib.call("b200_ep_row_a2a", ctx.heap.ctx, ptr(send_tensor), ctx.hidden * send_tensor.element_size(), ptr(cum),
              send_tensor.shape[0], ctx.num_tot_experts, ctx.experts_per_rank, ctx.max_m, ptr(sc), ctx.scale_per_row,
              ptr(ctx.recv_bufs[0]), ptr(ctx.recv_bufs[1]), ptr(ctx.scale_recv_bufs[0]), ptr(ctx.scale_recv_bufs[1]),
              ptr(ctx.split_recv_bufs[0]), ptr(ctx.split_recv_bufs[1]), ptr(ctx.flags), ptr(ctx.sync), stream_ptr())
    ops._count()
    scale_out = None
    if send_scale is not None:
        scale_out = ctx.scale_recv_bufs[par] if ctx.scale_per_row > 1 else ctx.scale_recv_bufs[par].view(-1)
    return [ctx.split_recv_bufs[par], ctx.recv_bufs[par], scale_out]


def all_to_all_post_process(ctx: AllToAllContext, input_splits: torch.Tensor, recv_buffer: torch.Tensor,
                            scale_buffer: torch.Tensor | None = None):
    """Compact the per-source segments into one tensor (source-major), as the reference does with torch slicing."""
    per_src = input_splits.reshape(ctx.WORLD_SIZE, -1).sum(dim=1).tolist()
    data = torch.cat([recv_buffer[s * ctx.max_m: s * ctx.max_m + n] for s, n in enumerate(per_src)])
    scale = None
    if scale_buffer is not None:
        scale = torch.cat([scale_buffer[s * ctx.max_m: s * ctx.max_m + n] for s, n in enumerate(per_src)])
    return data, scale
