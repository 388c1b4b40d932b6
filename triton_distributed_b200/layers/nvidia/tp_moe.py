"""Mixture-of-experts MLP blocks: tensor-parallel (every expert's intermediate dimension is sharded over ranks) and
expert-parallel (whole experts are partitioned over ranks).

The reference ships the kernels (AG + grouped GEMM, grouped GEMM + RS, EP all-to-all) and composes them only in
tests (``test/nvidia/test_ag_moe.py``, ``test_moe_reduce_rs.py``, ``test_ep_moe_inference.py:337-490``); these
layers are that composition as reusable modules, with a pure-torch forward as golden.

Weights are K-major per expert: ``w_gate_up [E, 2 * I_local, H]`` (gate rows then up rows) and ``w_down [E, H, I_local]``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...kernels.nvidia import (ag_group_gemm, all_reduce, create_ag_group_gemm_context, create_moe_rs_context, grouped_gemm,
                               moe_reduce_rs, reduce_topk)
from .ep_a2a_layer import EPAll2AllLayer


def _route_torch(x, gate_w, topk, renorm):
    probs = torch.softmax(F.linear(x.float(), gate_w.float()), dim=-1)
    w, ids = torch.topk(probs, topk, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w


def _experts_torch(x, ids, w, w_gate_up, w_down):
    """Golden: per-expert dense matmuls on the rows routed to it. Returns fp32 [T, H]."""
    T, topk = ids.shape
    inter = w_gate_up.shape[1] // 2
    out = torch.zeros((T, w_down.shape[1]), dtype=torch.float32, device=x.device)
    for e in range(w_gate_up.shape[0]):
        tok, k = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = F.linear(x[tok], w_gate_up[e])
        act = (F.silu(gu[:, :inter].float()) * gu[:, inter:].float()).to(x.dtype)
        out.index_add_(0, tok, F.linear(act, w_down[e]).float() * w[tok, k, None].float())
    return out


class TP_MoE:

    def __init__(self, rank: int = 0, world_size: int = 8, group=None, topk: int = 8, norm_topk_prob: bool = True,
                 fp8: bool = False):
        """fp8: the sequence-sharded forward runs both projections on the block-scaled fp8 fused kernels (tokens are
        quantised per 128 channels and gathered as bytes, the SwiGLU kernel quantises the activations); needs the hidden
        size and the local intermediate size to be multiples of 128."""
        self.rank, self.world_size, self.group = rank, world_size, group
        self.topk, self.norm_topk_prob = topk, norm_topk_prob
        self.fp8 = fp8
        self.ag_ctx = self.rs_ctx = self.ar_ctx = self.ag_ctx8 = None
        self.ar_method = None

    def _init_parameters(self, gate: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        """gate [E, H]; w_gate_up [E, 2 * I / world, H]; w_down [E, H, I / world] (already sharded)."""
        self.gate = gate.contiguous()
        self.w_gate_up = w_gate_up.contiguous()
        self.w_down = w_down.contiguous()
        self.num_experts, _, self.hidden = w_gate_up.shape
        self.inter_local = w_gate_up.shape[1] // 2
        self.dtype = w_gate_up.dtype
        if self.fp8:
            if self.hidden % 128 or self.inter_local % 128:
                raise ValueError("fp8 TP_MoE needs hidden and intermediate / world to be multiples of 128")
            from ...kernels.nvidia.grouped_gemm_fp8 import quantize_fp8_weight_blocks
            self.w_gate_up8, self.w_gate_up_scale = quantize_fp8_weight_blocks(self.w_gate_up)
            self.w_down8, self.w_down_scale = quantize_fp8_weight_blocks(self.w_down)

    def _init_ctx(self, max_tokens: int):
        self.ag_ctx = create_ag_group_gemm_context(max_tokens, 2 * self.inter_local, self.hidden, self.num_experts, self.topk,
                                                   self.dtype, self.rank, self.world_size)
        self.rs_ctx = create_moe_rs_context(self.group, self.world_size, max_tokens, self.hidden, self.num_experts, self.topk,
                                            self.dtype, self.dtype)
        if self.fp8:
            from ...kernels.nvidia.allgather_group_gemm import create_ag_group_gemm_fp8_context
            self.ag_ctx8 = create_ag_group_gemm_fp8_context(max_tokens, 2 * self.inter_local, self.hidden, self.num_experts,
                                                            self.topk, self.dtype, self.rank, self.world_size)

    def finalize(self):
        for c in (self.ag_ctx, self.rs_ctx, self.ag_ctx8):
            if c is not None:
                c.finalize()
        self.ag_ctx = self.rs_ctx = self.ag_ctx8 = None

    def route(self, x: torch.Tensor):
        """Router on the native kernels: (ids int32 [T, topk], weights fp32 [T, topk])."""
        logits = ops.linear(x, self.gate)
        return ops.topk_softmax(logits, self.topk, self.norm_topk_prob)

    @torch.no_grad()
    def torch_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, H] replicated -> [T, H]; cuBLAS per expert + NCCL all-reduce."""
        ids, w = _route_torch(x, self.gate, self.topk, self.norm_topk_prob)
        out = _experts_torch(x, ids, w, self.w_gate_up, self.w_down)
        if self.world_size > 1:
            dist.all_reduce(out, group=self.group)
        return out.to(x.dtype)

    @torch.no_grad()
    def partial_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Replicated activations: this rank's partial sum [T, H] (grouped tcgen05 GEMMs, no communication)."""
        ids, w = self.route(x)
        up = grouped_gemm(x, self.w_gate_up, ids)
        act = ops.silu_mul(up)
        down = grouped_gemm(act, self.w_down, ids, a_per_pair=True, row_scale=w)
        return reduce_topk(down, self.topk)

    @torch.no_grad()
    def dist_triton_AR_fwd(self, x: torch.Tensor) -> torch.Tensor:
        out = self.partial_fwd(x)
        if self.world_size > 1:
            out = all_reduce(out, None, self.ar_method, self.ar_ctx)
        return out

    @torch.no_grad()
    def dist_triton_fwd(self, x_local: torch.Tensor) -> torch.Tensor:
        """Sequence-sharded activations [T / world, H] -> [T / world, H]:
        route -> all-gather routing -> AG + grouped GEMM -> SwiGLU -> grouped GEMM + topk-reduce + RS."""
        ids, w = self.route(x_local)
        if self.world_size > 1:
            T = ids.shape[0] * self.world_size
            full_ids = torch.empty((T, self.topk), dtype=ids.dtype, device=ids.device)
            full_w = torch.empty((T, self.topk), dtype=w.dtype, device=w.device)
            dist.all_gather_into_tensor(full_ids, ids, group=self.group)
            dist.all_gather_into_tensor(full_w, w, group=self.group)
            ids, w = full_ids, full_w
        if self.fp8:
            from ...kernels.nvidia.allgather_group_gemm import ag_group_gemm_fp8
            from ...kernels.nvidia.grouped_gemm_fp8 import quantize_fp8_rows
            from ...kernels.nvidia.moe_reduce_rs import moe_reduce_rs_fp8
            x8, sx = quantize_fp8_rows(x_local)
            up = ag_group_gemm_fp8(x8, sx, self.w_gate_up8, self.w_gate_up_scale, self.ag_ctx8, ids)
            act8, act_scale = ops.silu_mul_fp8(up)
            return moe_reduce_rs_fp8(act8, act_scale, self.w_down8, self.w_down_scale, ids, w, self.rs_ctx)
        up = ag_group_gemm(x_local, self.w_gate_up, self.ag_ctx, ids)
        act = ops.silu_mul(up)
        return moe_reduce_rs(act, self.w_down, ids, w, self.rs_ctx)

    fwd = torch_fwd


class EP_MoE:
    """Experts partitioned over ranks; tokens travel by the fused dispatch / combine kernels."""

    def __init__(self, rank: int, world_size: int, group, num_experts: int, topk: int, hidden: int, max_tokens: int,
                 dtype=torch.bfloat16, norm_topk_prob: bool = True, fp8_dispatch: bool = False, fp8_experts: bool = False):
        """fp8_dispatch: tokens travel as e4m3 + one fp32 scale per 128 channels. fp8_experts (needs fp8_dispatch):
        both expert projections run on the block-scaled fp8 grouped GEMM: the up-projection directly on the dispatched
        bytes, the down-projection on the SwiGLU output that one kernel gates and quantises (intermediate % 128 == 0)."""
        if fp8_experts and not fp8_dispatch:
            raise ValueError("fp8_experts needs fp8_dispatch")
        self.fp8_experts = fp8_experts
        self.rank, self.world_size, self.group = rank, world_size, group
        self.num_experts, self.topk, self.hidden, self.dtype = num_experts, topk, hidden, dtype
        self.norm_topk_prob = norm_topk_prob
        self.experts_local = num_experts // world_size
        self.fp8_dispatch = fp8_dispatch
        self.a2a = EPAll2AllLayer(group, max_tokens, hidden, topk, rank, num_experts, world_size, world_size, dtype,
                                  fp8=fp8_dispatch)

    def _init_parameters(self, gate: torch.Tensor, w_gate_up_local: torch.Tensor, w_down_local: torch.Tensor):
        """gate [E, H]; w_gate_up_local [E / world, 2 * I, H]; w_down_local [E / world, H, I] (this rank's experts)."""
        self.gate, self.w_gate_up, self.w_down = gate.contiguous(), w_gate_up_local.contiguous(), w_down_local.contiguous()
        if self.fp8_experts:
            from ...kernels.nvidia.grouped_gemm_fp8 import quantize_fp8_weight_blocks
            self.w_gate_up8, self.w_gate_up_scale = quantize_fp8_weight_blocks(self.w_gate_up)
            self.fp8_down = self.w_down.shape[2] % 128 == 0
            if self.fp8_down:
                self.w_down8, self.w_down_scale = quantize_fp8_weight_blocks(self.w_down)

    def _grouped(self, a: torch.Tensor, w: torch.Tensor, n_rows: int) -> torch.Tensor:
        sorted_ids, tile_expert, totals, _ = self.a2a.recv_plan()
        E, N, K = w.shape
        out = torch.zeros((n_rows, N), dtype=a.dtype, device=a.device)
        _lib.call("b200_grouped_gemm", ptr(a), a.stride(0), 1, ptr(w), E, N, K, n_rows, ptr(sorted_ids), ptr(tile_expert), None,
                  ptr(totals), self.a2a.recv_cap // 128, ptr(out), out.stride(0), None, dtype_code(a.dtype), stream_ptr())
        ops._count()
        return out

    @torch.no_grad()
    def dist_triton_fwd(self, x_local: torch.Tensor) -> torch.Tensor:
        """x_local [T_local, H] (this rank's tokens) -> [T_local, H]."""
        ids, w = ops.topk_softmax(ops.linear(x_local, self.gate), self.topk, self.norm_topk_prob)
        res = self.a2a.dispatch(x_local, ids)
        if self.fp8_experts:
            from ...kernels.nvidia.grouped_gemm_fp8 import grouped_gemm_fp8_planned
            q, sc = res
            n_rows = q.shape[0]
            sorted_ids, tile_expert, totals, _ = self.a2a.recv_plan()
            up = torch.zeros((n_rows, self.w_gate_up8.shape[1]), dtype=self.dtype, device=q.device)
            grouped_gemm_fp8_planned(q, sc, self.w_gate_up8, self.w_gate_up_scale, sorted_ids, tile_expert, totals,
                                     self.a2a.recv_cap // 128, n_rows, 1, None, up)
        else:
            if self.fp8_dispatch:
                q, sc = res
                rows = (q.float().view(q.shape[0], -1, 128) * sc[:, :, None]).view(q.shape[0], -1).to(self.dtype)
            else:
                rows = res
            n_rows = rows.shape[0]
            up = self._grouped(rows, self.w_gate_up, n_rows)
        if self.fp8_experts and self.fp8_down:
            act8, act_scale = ops.silu_mul_fp8(up)
            down = torch.zeros((n_rows, self.w_down8.shape[1]), dtype=self.dtype, device=up.device)
            grouped_gemm_fp8_planned(act8, act_scale, self.w_down8, self.w_down_scale, sorted_ids, tile_expert, totals,
                                     self.a2a.recv_cap // 128, n_rows, 1, None, down)
        else:
            act = ops.silu_mul(up)
            down = self._grouped(act, self.w_down, n_rows)
        return self.a2a.combine(down, w)

    @torch.no_grad()
    def torch_fwd(self, x_local: torch.Tensor, w_gate_up_full: torch.Tensor, w_down_full: torch.Tensor) -> torch.Tensor:
        """Golden with ALL experts' weights present on this rank (tests only)."""
        ids, w = _route_torch(x_local, self.gate, self.topk, self.norm_topk_prob)
        return _experts_torch(x_local, ids, w, w_gate_up_full, w_down_full).to(x_local.dtype)

    def finalize(self):
        self.a2a.finalize()
