"""Expert-parallel dispatch / combine layer.

API parity with ``python/triton_dist/layers/nvidia/ep_a2a_layer.py:40-248`` (``EPAll2AllLayer.dispatch`` /
``combine`` / ``finalize``). Differences by design: the permutation and (optionally) the fp8 quantisation are fused
into the send kernel, the receive layout is produced on the device without the reference's CPU polling of pinned
memory and buffer regrowth, and ``combine`` can apply the routing weights while it sums the k copies.
"""
from __future__ import annotations

import torch

from ... import _lib, ops
from ..._lib import ptr, stream_ptr
from ...kernels.nvidia.moe_utils import create_sort_plan, moe_sort
from ...runtime.heap import get_heap


class EPAll2AllLayer:

    def __init__(self, ep_group, max_tokens: int, hidden: int, topk: int, rank: int, num_tot_experts: int,
                 local_world_size: int, world_size: int, dtype=torch.bfloat16, num_sm: int = 20, fp8: bool = False):
        heap = get_heap()
        if world_size != heap.world:
            raise ValueError("the EP layer spans the ranks of the symmetric heap (single node)")
        if num_tot_experts % world_size:
            raise ValueError("experts must divide evenly over the ranks")
        self.heap, self.group, self.rank, self.world_size = heap, ep_group, rank, world_size
        self.max_tokens, self.hidden, self.topk, self.dtype, self.fp8 = max_tokens, hidden, topk, dtype, fp8
        self.num_tot_experts, self.experts_per_rank = num_tot_experts, num_tot_experts // world_size
        self.max_m = max_tokens * topk  # worst case: every pair of a rank goes to one peer
        rows = world_size * self.max_m
        self.recv = [heap.create_tensor((rows, hidden), torch.uint8 if fp8 else dtype, align=1024) for _ in range(2)]
        self.recv_scale = [heap.create_tensor((rows, max(1, hidden // 128)), torch.float32) for _ in range(2)]
        self.recv_splits = [heap.create_tensor((world_size, self.experts_per_rank), torch.int32) for _ in range(2)]
        self.comb = [heap.create_tensor((rows, hidden), dtype, align=1024) for _ in range(2)]
        self.dflags = heap.create_tensor((16,), torch.int32)
        self.cflags = heap.create_tensor((16,), torch.int32)
        z = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")  # noqa: E731
        self.dsync, self.csync = z(4), z(4)
        self.plans: dict[int, object] = {}
        # grouped-GEMM metadata of the received rows
        cap = (rows + self.experts_per_rank * 127 + 127) // 128 * 128
        self.recv_sorted_ids, self.recv_tile_expert = z(cap), z(cap // 128)
        self.recv_totals, self.recv_rows_per_expert = z(4), z(self.experts_per_rank)
        self.recv_cap = cap
        self._last = None
        self._dispatch_calls = 0
        heap.barrier_all()
        torch.cuda.synchronize()

    def _plan(self, T: int):
        if T not in self.plans:
            self.plans[T] = create_sort_plan(T * self.topk, self.topk, self.num_tot_experts, 1, 1, with_positions=True)
        return self.plans[T]

    @torch.no_grad()
    def dispatch(self, input: torch.Tensor, exp_indices: torch.Tensor):
        """input [T, hidden] bf16; exp_indices int32 [T, topk]. Returns the receive buffer view
        ``[world * max_m, hidden]`` (bf16, or e4m3 bytes + per-128 scales when the layer is fp8), laid out per source
        rank in that source's expert order. ``recv_plan()`` gives the row list grouped by local expert."""
        T = input.shape[0]
        if T > self.max_tokens or exp_indices.shape != (T, self.topk):
            raise ValueError("batch does not fit the layer")
        if torch.cuda.is_current_stream_capturing():
            # the receive half is chosen on the host from a call counter; a replayed graph would keep the captured
            # half while the device-side epoch moves on, and the consumers would read the stale one
            raise RuntimeError("EPAll2AllLayer.dispatch cannot be captured in a CUDA graph: its double-buffer half is "
                               "selected on the host per call")
        ids = exp_indices.to(torch.int32).contiguous()
        plan = self._plan(T)
        moe_sort(ids, plan)
        self._dispatch_calls += 1  # mirrors the device-resident epoch without reading it back
        par = self._dispatch_calls & 1
        # one launch: permute (+ quantise) + send, and CTA 0 lays out the grouped-GEMM plan of the received rows
        _lib.call("b200_ep_dispatch_planned", self.heap.ctx, ptr(input.contiguous()), T, self.hidden, self.topk, ptr(ids),
                  ptr(plan.pair_pos), ptr(plan.group_count), self.num_tot_experts, self.experts_per_rank, self.max_m,
                  1 if self.fp8 else 0, ptr(self.recv[0]), ptr(self.recv[1]), ptr(self.recv_scale[0]), ptr(self.recv_scale[1]),
                  ptr(self.recv_splits[0]), ptr(self.recv_splits[1]), ptr(self.dflags), ptr(self.dsync), 128,
                  ptr(self.recv_sorted_ids), ptr(self.recv_tile_expert), ptr(self.recv_totals), ptr(self.recv_rows_per_expert),
                  self.recv_cap, stream_ptr())
        ops._count()
        self._last = (T, ids, plan, par)
        buf = self.recv[par].view(torch.float8_e4m3fn) if self.fp8 else self.recv[par]
        return (buf, self.recv_scale[par]) if self.fp8 else buf

    def recv_splits_view(self) -> torch.Tensor:
        """int32 [world, experts_per_rank]: rows received from every source for every local expert."""
        return self.recv_splits[self._last[3]]

    def recv_plan(self):
        """(sorted_ids, tile_expert, totals, rows_per_expert): grouped-GEMM metadata over the receive buffer rows."""
        return self.recv_sorted_ids, self.recv_tile_expert, self.recv_totals, self.recv_rows_per_expert

    @torch.no_grad()
    def combine(self, expert_out: torch.Tensor, topk_weight: torch.Tensor | None = None) -> torch.Tensor:
        """expert_out bf16 [world * max_m, hidden] in the receive layout of the last dispatch -> [T, hidden]:
        the sum over the k experts of every token (weighted when `topk_weight` [T, topk] is given)."""
        if self._last is None:
            raise RuntimeError("combine() needs a preceding dispatch()")
        T, ids, plan, _ = self._last
        out = torch.empty((T, self.hidden), dtype=self.dtype, device=expert_out.device)
        w = topk_weight.float().contiguous() if topk_weight is not None else None
        _lib.call("b200_ep_combine", self.heap.ctx, ptr(expert_out), T, self.hidden, self.topk, ptr(ids), ptr(plan.pair_pos),
                  ptr(plan.group_count), ptr(w), self.num_tot_experts, self.experts_per_rank, self.max_m, ptr(self.dsync),
                  ptr(self.recv_splits[0]), ptr(self.recv_splits[1]), ptr(self.comb[0]), ptr(self.comb[1]), ptr(self.cflags),
                  ptr(self.csync), ptr(out), stream_ptr())
        ops._count()
        return out

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.recv + self.recv_scale + self.recv_splits + self.comb + [self.dflags, self.cflags]:
            self.heap.free(t)
        self.recv = []
