"""AG + grouped GEMM (tensor-parallel MoE up-projection) in one fused sm_100a kernel.

API parity with ``python/triton_dist/kernels/nvidia/allgather_group_gemm.py`` (``create_ag_group_gemm_context`` :334,
``ag_group_gemm`` :398): ``a`` is this rank's tokens ``[ntokens / r, K]``, ``b`` the experts' weight shards, and the
result row ``t * topk + k`` is token t times the weights of its k-th expert.

Weights are consumed K-major, ``[E, N_per_rank, K]`` (the Hugging Face layout of an expert's ``nn.Linear``). The
reference's ``[E, K, N_per_rank]`` layout is accepted and transposed once per weight tensor.
"""
from __future__ import annotations

import dataclasses

import torch

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap
from .moe_utils import MoeSortPlan, create_sort_plan, moe_sort, order_tiles


@dataclasses.dataclass
class MoEAllGatherGroupGEMMTensorParallelContext:
    rank: int
    num_ranks: int
    max_ntokens: int
    N_per_rank: int
    K: int
    num_experts: int
    topk: int
    dtype: torch.dtype
    heap: SymmHeap
    symm_workspaces: list[torch.Tensor]
    symm_ready: torch.Tensor
    rank_cnt: torch.Tensor
    rank_flag: torch.Tensor
    sync: torch.Tensor
    plans: dict
    _weights_nk: dict

    def plan_for(self, ntokens: int) -> MoeSortPlan:
        if ntokens not in self.plans:
            self.plans[ntokens] = create_sort_plan(ntokens * self.topk, self.topk, self.num_experts, 128, 1)
        return self.plans[ntokens]

    def weights_nk(self, b: torch.Tensor) -> torch.Tensor:
        """[E, N, K] view of the weights; a [E, K, N] tensor is transposed once and cached."""
        if b.shape[2] == self.K and b.shape[1] == self.N_per_rank:
            return b  # already [E, N, K]; a square weight is always read this way
        if b.shape[1] == self.K and b.shape[2] == self.N_per_rank:
            key = (b.data_ptr(), b._version)
            if key not in self._weights_nk:
                self._weights_nk = {key: b.transpose(1, 2).contiguous()}
            return self._weights_nk[key]
        raise ValueError(f"weights {tuple(b.shape)} match neither [E, {self.N_per_rank}, {self.K}] nor [E, {self.K}, {self.N_per_rank}]")

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.symm_workspaces + [self.symm_ready]:
            self.heap.free(t)
        self.symm_workspaces = []



def create_ag_group_gemm_context(max_ntokens: int, N_per_rank: int, K: int, num_experts: int, topk: int,
                                 dtype: torch.dtype, rank: int, num_ranks: int, num_local_ranks: int | None = None,
                                 ag_intranode_stream=None, ag_internode_stream=None, BLOCK_SIZE_M: int = 128,
                                 BLOCK_SIZE_N: int = 128, BLOCK_SIZE_K: int = 64, GROUP_SIZE_M: int = 8, stages: int = 6,
                                 num_warps: int = 12) -> MoEAllGatherGroupGEMMTensorParallelContext:
    heap = get_heap()
    if num_ranks != heap.world:
        raise ValueError("AG + grouped GEMM spans the ranks of the symmetric heap (single node)")
    ws = [heap.create_tensor((max_ntokens, K), dtype, align=1024) for _ in range(2)]
    ready = heap.create_tensor((16,), torch.int32)
    z = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")  # noqa: E731
    ctx = MoEAllGatherGroupGEMMTensorParallelContext(rank, num_ranks, max_ntokens, N_per_rank, K, num_experts, topk, dtype,
                                                     heap, ws, ready, z(16), z(16), z(4), {}, {})
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def _reorder_pays(ctx, T: int, E: int, N: int, K: int, es: int) -> bool:
    world = ctx.num_ranks
    if world == 1:
        return False
    tiles_per_expert = max(1, (T * ctx.topk) // (E * 128))
    restreams = min(world, tiles_per_expert) - 1                 # extra passes over the weights
    weight_time = restreams * E * N * K * es / 6.5e12            # at the measured HBM copy rate
    gather_time = (world - 1) / world * T * K * es / 6.0e11      # at what the pulling warps sustain per GPU
    return weight_time < 0.5 * gather_time


def ag_group_gemm(a: torch.Tensor, b: torch.Tensor, ctx: MoEAllGatherGroupGEMMTensorParallelContext,
                  full_topk_ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [ntokens / r, K]; b [E, N / r, K] (or [E, K, N / r]); full_topk_ids int32 [ntokens, topk] (all ranks' tokens).
    Returns [ntokens * topk, N / r]."""
    Tr, K = a.shape
    T = Tr * ctx.num_ranks
    if T > ctx.max_ntokens or K != ctx.K or full_topk_ids.shape != (T, ctx.topk):
        raise ValueError("problem does not fit the context")
    w = ctx.weights_nk(b)
    E, N, _ = w.shape
    plan = ctx.plan_for(T)
    moe_sort(full_topk_ids.to(torch.int32).contiguous(), plan, tokens_per_rank=Tr)
    # Issuing tiles in the order their source shards arrive lets the GEMM start under the gather, but it also splits
    # every expert's tiles over several arrival stages, and each stage streams the expert's weights again. Reorder only
    # when those extra weight bytes cost clearly less HBM time than the gather takes on the links; otherwise keep the
    # expert-major order (each tile still waits only for the shards its own rows come from).
    order = order_tiles(plan, ctx.rank, ctx.num_ranks, 0) if _reorder_pays(ctx, T, E, N, K, a.element_size()) else None
    if out is None:
        out = torch.empty((T * ctx.topk, N), dtype=a.dtype, device=a.device)
    _lib.call("b200_ag_grouped_gemm", ctx.heap.ctx, ptr(a.contiguous()), ptr(ctx.symm_workspaces[0]),
              ptr(ctx.symm_workspaces[1]), Tr, ctx.topk, ptr(w), E, N, K, ptr(plan.sorted_ids), ptr(plan.tile_expert),
              ptr(order), ptr(plan.totals), plan.max_tiles, ptr(out), out.stride(0), ptr(ctx.symm_ready), ptr(ctx.rank_cnt),
              ptr(ctx.rank_flag), ptr(ctx.sync), dtype_code(a.dtype), stream_ptr())
    ops._count()
    return out


@dataclasses.dataclass
class MoEAllGatherGroupGEMMFp8Context:
    """Buffers of :func:`ag_group_gemm_fp8`. A token row travels as ``K`` e4m3 bytes followed by its ``K / 128`` fp32
    scales (``pitch`` bytes, a multiple of 16), so that one gather moves both."""
    rank: int
    num_ranks: int
    max_ntokens: int
    N_per_rank: int
    K: int
    num_experts: int
    topk: int
    out_dtype: torch.dtype
    pitch: int
    heap: SymmHeap
    symm_workspaces: list[torch.Tensor]
    symm_ready: torch.Tensor
    rank_cnt: torch.Tensor
    rank_flag: torch.Tensor
    sync: torch.Tensor
    staging: torch.Tensor          # local [max_ntokens / r, pitch] bytes: this rank's packed rows
    plans: dict

    def plan_for(self, ntokens: int) -> MoeSortPlan:
        if ntokens not in self.plans:
            self.plans[ntokens] = create_sort_plan(ntokens * self.topk, self.topk, self.num_experts, 128, 1)
        return self.plans[ntokens]

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.symm_workspaces + [self.symm_ready]:
            self.heap.free(t)
        self.symm_workspaces = []


def create_ag_group_gemm_fp8_context(max_ntokens: int, N_per_rank: int, K: int, num_experts: int, topk: int,
                                     out_dtype: torch.dtype, rank: int, num_ranks: int) -> MoEAllGatherGroupGEMMFp8Context:
    heap = get_heap()
    if num_ranks != heap.world:
        raise ValueError("AG + grouped GEMM spans the ranks of the symmetric heap (single node)")
    if K % 128:
        raise ValueError("K must be a multiple of 128 (one activation scale per 128 channels)")
    pitch = (K + K // 32 + 15) // 16 * 16
    ws = [heap.create_tensor((max_ntokens, pitch), torch.uint8, align=1024) for _ in range(2)]
    ready = heap.create_tensor((16,), torch.int32)
    z = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")  # noqa: E731
    staging = torch.zeros((max_ntokens // num_ranks, pitch), dtype=torch.uint8, device="cuda")
    ctx = MoEAllGatherGroupGEMMFp8Context(rank, num_ranks, max_ntokens, N_per_rank, K, num_experts, topk, out_dtype, pitch,
                                          heap, ws, ready, z(16), z(16), z(4), staging, {})
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def ag_group_gemm_fp8(a8: torch.Tensor, a_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                      ctx: MoEAllGatherGroupGEMMFp8Context, full_topk_ids: torch.Tensor,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Block-scaled fp8 form of :func:`ag_group_gemm`: a8 e4m3 [ntokens / r, K] with fp32 scales a_scale
    [ntokens / r, K / 128] (this rank's tokens), w8 e4m3 [E, N / r, K] with w_scale [E, ceil(N / r / 128), K / 128];
    full_topk_ids int32 [ntokens, topk]. The gather moves one byte per channel plus the scales, half of what the bf16
    kernel moves. Returns [ntokens * topk, N / r] in the context's 16-bit dtype."""
    Tr, K = a8.shape
    T = Tr * ctx.num_ranks
    E, N, _ = w8.shape
    if T > ctx.max_ntokens or K != ctx.K or full_topk_ids.shape != (T, ctx.topk):
        raise ValueError("problem does not fit the context")
    if a8.element_size() != 1 or w8.element_size() != 1:
        raise ValueError("a8 / w8 must be 1-byte tensors")
    if tuple(a_scale.shape) != (Tr, K // 128) or tuple(w_scale.shape) != (E, (N + 127) // 128, K // 128):
        raise ValueError("scale shapes do not match the operands")
    plan = ctx.plan_for(T)
    moe_sort(full_topk_ids.to(torch.int32).contiguous(), plan, tokens_per_rank=Tr)
    order = order_tiles(plan, ctx.rank, ctx.num_ranks, 0) if _reorder_pays(ctx, T, E, N, K, 1) else None
    # pack [row bytes | row scales] once: the peers pull whole packed rows
    stage = ctx.staging[:Tr]
    stage[:, :K].copy_(a8.view(torch.uint8))
    stage[:, K:K + K // 32].copy_(a_scale.contiguous().view(torch.uint8).view(Tr, K // 32))
    if out is None:
        out = torch.empty((T * ctx.topk, N), dtype=ctx.out_dtype, device=a8.device)
    _lib.call("b200_ag_grouped_gemm_fp8", ctx.heap.ctx, ptr(stage), ctx.pitch, ptr(ctx.symm_workspaces[0]),
              ptr(ctx.symm_workspaces[1]), Tr, ctx.topk, ptr(w8.contiguous()), ptr(w_scale.contiguous()), E, N, K,
              ptr(plan.sorted_ids), ptr(plan.tile_expert), ptr(order), ptr(plan.totals), plan.max_tiles, ptr(out),
              out.stride(0), ptr(ctx.symm_ready), ptr(ctx.rank_cnt), ptr(ctx.rank_flag), ptr(ctx.sync), dtype_code(out.dtype),
              stream_ptr())
    ops._count()
    return out


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, topk_ids: torch.Tensor, a_per_pair: bool = False,
                 row_scale: torch.Tensor | None = None, plan: MoeSortPlan | None = None) -> torch.Tensor:
    """Local grouped GEMM: out[t * topk + k] = a[t (or pair)] @ w[topk_ids[t, k]].T (* row_scale). w [E, N, K]."""
    T, topk = topk_ids.shape
    E, N, K = w.shape
    if plan is None:
        plan = create_sort_plan(T * topk, topk, E, 128, 1, a.device)
    moe_sort(topk_ids.to(torch.int32).contiguous(), plan)
    out = torch.empty((T * topk, N), dtype=a.dtype, device=a.device)
    rs = row_scale.reshape(-1).float().contiguous() if row_scale is not None else None
    _lib.call("b200_grouped_gemm", ptr(a), a.stride(0), 1 if a_per_pair else topk, ptr(w), E, N, K, T * topk,
              ptr(plan.sorted_ids), ptr(plan.tile_expert), None, ptr(plan.totals), plan.max_tiles, ptr(out), out.stride(0),
              ptr(rs), dtype_code(a.dtype), stream_ptr())
    ops._count()
    return out
