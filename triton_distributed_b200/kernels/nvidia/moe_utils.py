"""MoE routing metadata on the device.

API parity with ``python/triton_dist/kernels/nvidia/moe_utils.py`` (``calc_gather_scatter_index_triton`` :218,
``histogram_by_expert_*`` :32-38, ``reduce_topk_*`` :251-394) and with the CUDA op
``moe_ag_scatter_align_block_size`` (``csrc/lib/moe_utils.cu``). Four short launches of ``csrc/kernels/moe_align.cu``
(count, prefix, offsets, scatter) sort the (token, k) pairs by expert (optionally inside every source-rank block), pad
every run to the tile height and emit the per-tile metadata the grouped GEMMs read; nothing synchronises with the
host, nothing allocates, and no kernel waits on another CTA.
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from ... import _lib, ops
from ..._lib import ptr, stream_ptr


@dataclasses.dataclass
class MoeSortPlan:
    """Device buffers of one sort (sized for the worst case) and its scratch."""
    n_pairs: int
    topk: int
    num_experts: int
    block_m: int
    segments: int
    capacity: int
    sorted_ids: torch.Tensor      # int32 [capacity] pair index per sorted row, pad = n_pairs
    tile_expert: torch.Tensor     # int32 [capacity / block_m]
    tile_seg_start: torch.Tensor  # int32 [tiles]: first source rank (segments == 1) or segment of the tile
    tile_seg_end: torch.Tensor
    tile_order: torch.Tensor      # int32 [tiles]: issue order (filled by order_tiles)
    group_count: torch.Tensor     # int32 [segments * E]
    totals: torch.Tensor          # int32 [2 + segments]: m_pad, tiles, cumulative tiles per segment
    scratch: torch.Tensor         # int32: per-chunk expert counts / prefixes and group offsets
    status: torch.Tensor          # int32 [16], stays zero: the sort has no device-side waits that could expire
    pair_pos: torch.Tensor | None = None  # int32 [n_pairs]: sorted position of every pair (when requested)

    @property
    def max_tiles(self) -> int:
        return self.capacity // self.block_m


def create_sort_plan(n_pairs: int, topk: int, num_experts: int, block_m: int = 128, segments: int = 1,
                     device="cuda", with_positions: bool = False) -> MoeSortPlan:
    lib = _lib.load()
    lib.b200_moe_sorted_capacity.restype = ctypes.c_longlong
    cap = int(lib.b200_moe_sorted_capacity(n_pairs, num_experts, block_m, segments))
    tiles = cap // block_m
    lib.b200_moe_sort_scratch_ints.restype = ctypes.c_longlong
    scratch = int(lib.b200_moe_sort_scratch_ints(n_pairs, num_experts, segments))
    i32 = dict(dtype=torch.int32, device=device)
    return MoeSortPlan(n_pairs, topk, num_experts, block_m, segments, cap,
                       torch.empty(cap, **i32), torch.empty(tiles, **i32), torch.empty(tiles, **i32),
                       torch.empty(tiles, **i32), torch.empty(tiles, **i32), torch.zeros(segments * num_experts, **i32),
                       torch.zeros(2 + segments, **i32), torch.empty(scratch, **i32), torch.zeros(16, **i32),
                       torch.empty(n_pairs, **i32) if with_positions else None)


def moe_sort(topk_ids: torch.Tensor, plan: MoeSortPlan, tokens_per_rank: int | None = None) -> MoeSortPlan:
    """Fill `plan` from topk_ids int32 [T, topk]."""
    _lib.require_cuda()
    ids = topk_ids.reshape(-1)
    if ids.dtype != torch.int32 or not ids.is_contiguous() or ids.numel() != plan.n_pairs:
        raise ValueError("topk_ids must be contiguous int32 with the plan's number of pairs")
    if tokens_per_rank is None:
        tokens_per_rank = max(1, plan.n_pairs // plan.topk)
    _lib.call("b200_moe_sort", ptr(ids), plan.n_pairs, plan.topk, plan.num_experts, plan.block_m, plan.segments,
              tokens_per_rank, ptr(plan.sorted_ids), ptr(plan.tile_expert), ptr(plan.tile_seg_start), ptr(plan.tile_seg_end),
              ptr(plan.group_count), ptr(plan.totals), ptr(plan.scratch), ptr(plan.pair_pos), stream_ptr())
    ops._count(4)
    return plan


def order_tiles(plan: MoeSortPlan, rank: int, world: int, shift: int = 0) -> torch.Tensor:
    """Issue order of the tiles by arrival stage (stable): the ring step, starting at ``rank + shift``, after which every
    source shard seg_start..seg_end of the tile has arrived."""
    _lib.call("b200_moe_tile_order", ptr(plan.tile_seg_start), ptr(plan.tile_seg_end), ptr(plan.totals), rank, world, shift, ptr(plan.tile_order),
              stream_ptr())
    ops._count()
    return plan.tile_order


def calc_gather_scatter_index(chosen_experts: torch.Tensor, nexperts: int, alignment_by_expert: int = 1):
    """(ntokens_by_expert, scatter_index [T, topk], gather_index [M_pad cap], expert_index [tiles cap], M_pad [1])."""
    T, topk = chosen_experts.shape
    plan = create_sort_plan(T * topk, topk, nexperts, alignment_by_expert, 1, chosen_experts.device)
    moe_sort(chosen_experts.to(torch.int32).contiguous(), plan)
    scatter = torch.empty(T * topk, dtype=torch.int32, device=chosen_experts.device)
    valid = plan.sorted_ids < T * topk
    pos = torch.arange(plan.capacity, dtype=torch.int32, device=chosen_experts.device)
    m_pad = plan.totals[0:1]
    live = valid & (pos < m_pad)
    scatter[plan.sorted_ids[live].long()] = pos[live]
    return plan.group_count, scatter.view(T, topk), plan.sorted_ids, plan.tile_expert, m_pad


calc_gather_scatter_index_triton = calc_gather_scatter_index


def calc_scatter_index_torch(chosen_experts: torch.Tensor, nexperts: int) -> torch.Tensor:
    """scatter_index [T, topk]: position of every (token, k) pair in the stable expert-sorted order (no padding).
    Plain torch; the oracle of the device sort (``moe_utils.py:94-135`` of the reference)."""
    flat = chosen_experts.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    scatter = torch.empty_like(order)
    scatter[order] = torch.arange(order.numel(), device=order.device)
    return scatter.view_as(chosen_experts).to(torch.int32)


def calc_gather_index_from_scatter_index(scatter_index: torch.Tensor, n_rows: int | None = None) -> torch.Tensor:
    """Inverse permutation: gather_index[scatter_index[p]] = p (rows that nothing scatters to hold -1)."""
    flat = scatter_index.reshape(-1).long()
    n = int(n_rows) if n_rows is not None else flat.numel()
    gather = torch.full((n,), -1, dtype=torch.int32, device=flat.device)
    gather[flat] = torch.arange(flat.numel(), dtype=torch.int32, device=flat.device)
    return gather


def histogram_by_expert(chosen_experts: torch.Tensor, nexperts: int) -> torch.Tensor:
    return torch.bincount(chosen_experts.reshape(-1).long(), minlength=nexperts).to(torch.int32)


histogram_by_expert_triton = histogram_by_expert_torch = histogram_by_expert


def reduce_topk(x: torch.Tensor, topk: int, weights: torch.Tensor | None = None) -> torch.Tensor:
    """[T * topk, N] -> [T, N]: sum (optionally weighted) of the k copies of every token (fp32 accumulation)."""
    T = x.shape[0] // topk
    xf = x.view(T, topk, -1).float()
    if weights is not None:
        xf = xf * weights.view(T, topk, 1).float()
    return xf.sum(1).to(x.dtype)


reduce_topk_tma = reduce_topk_non_tma = reduce_topk
