"""Grouped GEMM + top-k reduce + reduce-scatter (tensor-parallel MoE down-projection) in one fused kernel.

API parity with ``python/triton_dist/kernels/nvidia/moe_reduce_rs.py``: ``select_experts`` :172,
``create_moe_rs_context`` :287, ``moe_reduce_rs_rowise`` :816, ``create_moe_rs_context_colwise`` :983,
``moe_reduce_rs_colwise`` :1357. The reference splits the work into a producer grouped GEMM, a consumer
topk-reduce/scatter kernel and a ring reduce on three streams (row-wise), or chunks N (col-wise); here one
kernel does the grouped GEMM (routing weight applied in the epilogue), a grid barrier, the sum over the k
copies of every token, the push into the owner rank's slot and the owner-side reduction. The col-wise entry
point maps onto the same kernel: on one NVSwitch node there is no second topology level to pipeline against.
"""
from __future__ import annotations

import dataclasses
import os

import torch
import torch.distributed as dist

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap
from .moe_utils import MoeSortPlan, create_sort_plan, moe_sort


def select_experts(pg, num_ranks: int, topk: int, input_dtype, device, router_logits: torch.Tensor):
    """softmax -> top-k (native router kernel) on the local tokens, all-gathered over `pg`:
    (full_topk_ids int32 [T, topk], full_topk_weight [T, topk] in input_dtype)."""
    ids, w = ops.topk_softmax(router_logits.contiguous(), topk)
    w = w.to(input_dtype)
    if num_ranks > 1:
        full_ids = torch.empty((ids.shape[0] * num_ranks, topk), dtype=ids.dtype, device=ids.device)
        full_w = torch.empty((w.shape[0] * num_ranks, topk), dtype=w.dtype, device=w.device)
        dist.all_gather_into_tensor(full_ids, ids, group=pg)
        dist.all_gather_into_tensor(full_w, w, group=pg)
        return full_ids, full_w
    return ids, w


@dataclasses.dataclass
class MoEReduceRSContext:
    rank: int
    world_size: int
    max_token_num: int
    hidden_dim: int
    num_experts: int
    topk: int
    dtype: torch.dtype
    heap: SymmHeap
    slots: list[torch.Tensor]
    rs_cnt: torch.Tensor
    rs_base: torch.Tensor
    sync: torch.Tensor
    gemm_out: torch.Tensor
    plans: dict
    full_topk_ids: torch.Tensor | None = None
    full_topk_weight: torch.Tensor | None = None
    nvls: bool = False   # final sum over the ranks inside the switch (multimem.ld_reduce); needs the multicast mapping

    def plan_for(self, ntokens: int) -> MoeSortPlan:
        if ntokens not in self.plans:
            self.plans[ntokens] = create_sort_plan(ntokens * self.topk, self.topk, self.num_experts, 128, 1)
        return self.plans[ntokens]

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.slots + [self.rs_cnt]:
            self.heap.free(t)
        self.slots = []


def create_moe_rs_context(pg, local_world_size: int, max_token_num: int, hidden_dim: int, num_experts: int, topk: int,
                          input_dtype, output_dtype, device="cuda", moe_block_size: int = 128,
                          router_logits: torch.Tensor | None = None) -> MoEReduceRSContext:
    heap = get_heap()
    world = heap.world
    tr_cap = max_token_num // world
    slots = [heap.create_tensor((world, tr_cap, hidden_dim), output_dtype, align=1024) for _ in range(2)]
    rs_cnt = heap.create_tensor((16,), torch.int32)
    ctx = MoEReduceRSContext(heap.rank, world, max_token_num, hidden_dim, num_experts, topk, output_dtype, heap, slots, rs_cnt,
                             torch.zeros(16, dtype=torch.int32, device="cuda"), torch.zeros(4, dtype=torch.int32, device="cuda"),
                             torch.empty((max_token_num * topk, hidden_dim), dtype=output_dtype, device="cuda"), {})
    ctx.nvls = heap.has_multicast and world > 1 and os.environ.get("B200DIST_MOE_RS_NVLS", "0") == "1"
    if router_logits is not None:
        ctx.full_topk_ids, ctx.full_topk_weight = select_experts(pg, world, topk, input_dtype, device, router_logits)
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def moe_reduce_rs(x: torch.Tensor, w: torch.Tensor, topk_ids: torch.Tensor, topk_weight: torch.Tensor,
                  ctx: MoEReduceRSContext, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [T * topk, K / r] (row t * topk + k); w [E, N, K / r]; topk_ids / topk_weight [T, topk]. Returns [T / r, N]."""
    n_pairs, K = x.shape
    T = n_pairs // ctx.topk
    E, N, _ = w.shape
    if T > ctx.max_token_num or N != ctx.hidden_dim or T % ctx.world_size != 0:
        raise ValueError("problem does not fit the context")
    plan = ctx.plan_for(T)
    moe_sort(topk_ids.to(torch.int32).contiguous(), plan)
    Tr = T // ctx.world_size
    if out is None:
        out = torch.empty((Tr, N), dtype=x.dtype, device=x.device)
    scale = topk_weight.reshape(-1).float().contiguous()
    _lib.call("b200_grouped_gemm_rs", ctx.heap.ctx, ptr(x), x.stride(0), ptr(w), E, N, K, Tr, ctx.topk, ptr(plan.sorted_ids),
              ptr(plan.tile_expert), None, ptr(plan.totals), plan.max_tiles, ptr(scale), ptr(ctx.gemm_out), ptr(ctx.slots[0]),
              ptr(ctx.slots[1]), ctx.max_token_num // ctx.world_size, ptr(ctx.rs_cnt), ptr(ctx.rs_base), ptr(ctx.sync),
              ptr(out), dtype_code(x.dtype), 1 if ctx.nvls else 0, stream_ptr())
    ops._count()
    return out


def _weights_nk(b: torch.Tensor, K: int) -> torch.Tensor:
    """Accept the reference's [E, K / r, N] layout by transposing (callers should cache the result)."""
    if b.shape[2] == K and b.shape[1] != K:
        return b
    if b.shape[1] == K and b.shape[2] != K:
        return b.transpose(1, 2).contiguous()
    return b


def moe_reduce_rs_rowise(rank: int, world_size: int, local_world_size: int, a: torch.Tensor, b: torch.Tensor,
                         ctx: MoEReduceRSContext) -> torch.Tensor:
    """a [ntokens * topk, K / r]; b [E, N, K / r] (or [E, K / r, N]); routing taken from the context."""
    ntok = a.shape[0] // ctx.topk
    return moe_reduce_rs(a, _weights_nk(b, a.shape[1]), ctx.full_topk_ids[:ntok], ctx.full_topk_weight[:ntok], ctx)


def create_moe_rs_context_colwise(rank: int, world_size: int, local_world_size: int, max_token_num: int, hidden_dim: int,
                                  num_experts: int, topk: int, input_dtype) -> MoEReduceRSContext:
    return create_moe_rs_context(None, local_world_size, max_token_num, hidden_dim, num_experts, topk, input_dtype, input_dtype)


def moe_reduce_rs_colwise(x: torch.Tensor, weights: torch.Tensor, choosed_experts: torch.Tensor, expert_weight: torch.Tensor,
                          ctx: MoEReduceRSContext, n_chunks: int = 2, config=None) -> torch.Tensor:
    return moe_reduce_rs(x, _weights_nk(weights, x.shape[1]), choosed_experts, expert_weight, ctx)


def moe_reduce_rs_fp8(x8: torch.Tensor, x_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                      topk_ids: torch.Tensor, topk_weight: torch.Tensor, ctx: MoEReduceRSContext,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Block-scaled fp8 form of :func:`moe_reduce_rs`: x8 e4m3 [T * topk, K / r] with fp32 scales x_scale
    [T * topk, K / r / 128] (what ``ops.silu_mul_fp8`` writes), w8 e4m3 [E, N, K / r] with one fp32 scale per 128 x 128
    block, w_scale [E, ceil(N / 128), K / r / 128]. Same kernel phases after the GEMM (top-k sum, push, owner reduce);
    the output has the context's 16-bit dtype. Returns [T / r, N]."""
    n_pairs, K = x8.shape
    T = n_pairs // ctx.topk
    E, N, _ = w8.shape
    if T > ctx.max_token_num or N != ctx.hidden_dim or T % ctx.world_size != 0:
        raise ValueError("problem does not fit the context")
    if x8.element_size() != 1 or w8.element_size() != 1 or K % 128:
        raise ValueError("x8 / w8 must be 1-byte tensors with K a multiple of 128")
    if tuple(w_scale.shape) != (E, (N + 127) // 128, K // 128) or tuple(x_scale.shape) != (n_pairs, K // 128):
        raise ValueError("scale shapes do not match the operands")
    plan = ctx.plan_for(T)
    moe_sort(topk_ids.to(torch.int32).contiguous(), plan)
    Tr = T // ctx.world_size
    if out is None:
        out = torch.empty((Tr, N), dtype=ctx.dtype, device=x8.device)
    scale = topk_weight.reshape(-1).float().contiguous()
    _lib.call("b200_grouped_gemm_fp8_rs", ctx.heap.ctx, ptr(x8), x8.stride(0), ptr(x_scale.contiguous()), x_scale.stride(0),
              ptr(w8.contiguous()), ptr(w_scale.contiguous()), E, N, K, Tr, ctx.topk, ptr(plan.sorted_ids), ptr(plan.tile_expert),
              None, ptr(plan.totals), plan.max_tiles, ptr(scale), ptr(ctx.gemm_out), ptr(ctx.slots[0]), ptr(ctx.slots[1]),
              ctx.max_token_num // ctx.world_size, ptr(ctx.rs_cnt), ptr(ctx.rs_base), ptr(ctx.sync), ptr(out),
              dtype_code(out.dtype), 1 if ctx.nvls else 0, stream_ptr())
    ops._count()
    return out
