"""Block-scaled fp8 (e4m3) grouped GEMM for MoE experts.

``out[pair] = sum_kb sa[row, kb] * sw[e, n // 128, kb] * (A8[row, kb] . W8[e, n, kb])``: activations carry one fp32
scale per row and 128 channels (the layout the expert-parallel dispatch kernel writes), weights one per 128 x 128
block (the DeepSeek-V3 recipe). The kernel (``csrc/kernels/grouped_gemm_fp8_sm100.cu``) multiplies one scale block
per pipeline stage with ``tcgen05.mma kind::f8f6f4`` and promotes the partial sums into fp32 registers between
k-blocks.

Role in the reference: the fp8 expert GEMMs of ``python/triton_dist/test/nvidia/test_ep_moe_inference.py:169-327``
and the quantisation numerics of ``tutorials/04-deepseek-infer-all2all.py:189-193`` (scale = amax / 448, no epsilon).
"""
from __future__ import annotations

import torch

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from .moe_utils import MoeSortPlan, create_sort_plan, moe_sort

FP8_MAX = 448.0


def quantize_fp8_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x [T, K] (K % 128 == 0) -> (e4m3 [T, K], fp32 scales [T, K / 128]); scale = amax / 448 per 128 channels."""
    T, K = x.shape
    if K % 128:
        raise ValueError("K must be a multiple of 128")
    xb = x.float().view(T, K // 128, 128)
    scale = xb.abs().amax(-1) / FP8_MAX
    den = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (xb / den[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(T, K).contiguous(), scale.contiguous()


def quantize_fp8_weight_blocks(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [E, N, K] (K % 128 == 0) -> (e4m3 [E, N, K], fp32 scales [E, ceil(N / 128), K / 128]), one per 128 x 128 block."""
    E, N, K = w.shape
    if K % 128:
        raise ValueError("K must be a multiple of 128")
    nb = (N + 127) // 128
    wp = torch.zeros((E, nb * 128, K), dtype=torch.float32, device=w.device)
    wp[:, :N] = w.float()
    blocks = wp.view(E, nb, 128, K // 128, 128)
    scale = blocks.abs().amax(dim=(2, 4)) / FP8_MAX
    den = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (blocks / den[:, :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(E, nb * 128, K)[:, :N].contiguous(), scale.contiguous()


def grouped_gemm_fp8_planned(a8: torch.Tensor, a_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                             sorted_ids: torch.Tensor, tile_expert: torch.Tensor, totals: torch.Tensor, max_tiles: int,
                             n_pairs: int, a_div: int = 1, row_scale: torch.Tensor | None = None,
                             out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Grouped GEMM over an existing tile plan (``moe_sort`` or the EP layer's ``recv_plan``).

    a8 e4m3 (or uint8 bytes) [rows, K]; a_scale fp32 [rows, K / 128]; w8 [E, N, K]; w_scale fp32 [E, ceil(N / 128), K / 128].
    Row ``sorted_ids[i] // a_div`` of a8 feeds sorted row i; the result of pair p lands in ``out[p]`` ([n_pairs, N]).
    Rows of ``out`` that no tile covers are left untouched (pass a zeroed ``out`` if that matters)."""
    _lib.require_cuda()
    E, N, K = w8.shape
    if a8.shape[1] != K or a8.element_size() != 1 or w8.element_size() != 1:
        raise ValueError("a8 / w8 must be 1-byte tensors that agree on K")
    if not (a8.stride(1) == 1 and w8.is_contiguous() and a_scale.is_contiguous() and w_scale.is_contiguous()):
        raise ValueError("operands must be contiguous (a8 may have a row pitch)")
    if a_scale.dtype != torch.float32 or w_scale.dtype != torch.float32:
        raise ValueError("scales are fp32")
    if tuple(w_scale.shape) != (E, (N + 127) // 128, K // 128) or a_scale.shape[1] != K // 128:
        raise ValueError("scale shapes do not match the operands")
    if out is None:
        out = torch.empty((n_pairs, N), dtype=out_dtype, device=a8.device)
    rs = row_scale.reshape(-1).float().contiguous() if row_scale is not None else None
    status = torch.zeros(1, dtype=torch.int32, device=a8.device)
    _lib.call("b200_grouped_gemm_fp8", ptr(a8), a8.stride(0), ptr(a_scale), a_scale.stride(0), a_div, ptr(w8), ptr(w_scale),
              E, N, K, n_pairs, ptr(sorted_ids), ptr(tile_expert), ptr(totals), max_tiles, ptr(out), out.stride(0), ptr(rs),
              dtype_code(out.dtype), ptr(status), stream_ptr())
    ops._count()
    return out


def grouped_gemm_fp8(a8: torch.Tensor, a_scale: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                     topk_ids: torch.Tensor, a_per_pair: bool = False, row_scale: torch.Tensor | None = None,
                     plan: MoeSortPlan | None = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``out[t * topk + k] = dequant(a8[t (or pair)]) @ dequant(w8[topk_ids[t, k]]).T (* row_scale)`` -> [T * topk, N]."""
    T, topk = topk_ids.shape
    E = w8.shape[0]
    if plan is None:
        plan = create_sort_plan(T * topk, topk, E, 128, 1, a8.device)
    moe_sort(topk_ids.to(torch.int32).contiguous(), plan)
    return grouped_gemm_fp8_planned(a8, a_scale, w8, w_scale, plan.sorted_ids, plan.tile_expert, plan.totals, plan.max_tiles,
                                    T * topk, 1 if a_per_pair else topk, row_scale, None, out_dtype)
