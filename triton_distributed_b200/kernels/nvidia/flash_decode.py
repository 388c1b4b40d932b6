"""GQA flash-decode over a paged KV cache (split-KV + LSE combine).

API parity with ``python/triton_dist/kernels/nvidia/flash_decode.py``: ``gqa_fwd_batch_decode`` :763,
``gqa_fwd_batch_decode_intra_rank`` :847 (output ``[B, Hq, D + 1]`` with the natural-log LSE in the last
column), ``gqa_fwd_batch_decode_persistent`` :931, the ``*_aot`` names :1008-1161 (all kernels here are
compiled ahead of time, so they are aliases) and the inter-rank combine :482-532.
"""
from __future__ import annotations

import torch

from ... import ops


def _splits(q, k_cache, kv_lens_max: int, kv_split: int) -> int:
    if kv_split and kv_split > 0:
        return kv_split
    B, Hq, _ = q.shape
    Hkv = k_cache.shape[2]
    return ops.choose_kv_splits(B, Hkv, Hq // Hkv, kv_lens_max, torch.cuda.get_device_properties(q.device).multi_processor_count)


def gqa_fwd_batch_decode(q, k_cache, v_cache, workspace, q_lens, kv_lens, block_table, scale, soft_cap: float = 0.0,
                         output_split=None, output_combine=None, kv_split: int = -1, max_kv_len: int | None = None):
    """q [B,Hq,128]; caches [num_blocks, page, Hkv, 128]; kv_lens int32 [B]; block_table int32 [B, max_blocks].
    `max_kv_len` (an upper bound on kv_lens) avoids a device-to-host sync when choosing the split count."""
    if max_kv_len is None:
        max_kv_len = block_table.shape[1] * k_cache.shape[1]
    ws = workspace if isinstance(workspace, dict) else None
    return ops.decode_attention(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap,
                                _splits(q, k_cache, max_kv_len, kv_split), out=output_combine, workspace=ws)


def gqa_fwd_batch_decode_intra_rank(q, k_cache, v_cache, workspace, q_lens, kv_lens, block_table, scale,
                                    soft_cap: float = 0.0, output_split=None, output_combine=None, kv_split: int = -1,
                                    max_kv_len: int | None = None):
    """As above but returns fp32 ``[B, Hq, D + 1]``: the local attention output with its LSE appended, the
    partial that sequence-parallel decode exchanges between ranks."""
    if max_kv_len is None:
        max_kv_len = block_table.shape[1] * k_cache.shape[1]
    ws = workspace if isinstance(workspace, dict) else None
    out, lse = ops.decode_attention(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap,
                                    _splits(q, k_cache, max_kv_len, kv_split), return_lse=True, workspace=ws)
    res = output_combine if output_combine is not None else torch.empty(
        (*out.shape[:-1], out.shape[-1] + 1), dtype=torch.float32, device=q.device)
    res[..., :-1] = out
    res[..., -1] = lse
    return res


def gqa_fwd_batch_decode_persistent(q, k_cache, v_cache, workspace, q_lens, kv_lens, block_table, scale,
                                    soft_cap: float = 0.0, output_split=None, output_combine=None, kv_split: int = -1,
                                    max_kv_len: int | None = None):
    """Split + combine in ONE launch (reference: flash_decode.py:587-760, a cooperative launch of 132 CTAs with a grid
    barrier between the phases). Here no CTA waits for another: every CTA of a (batch, head group) draws a ticket
    once its partial is visible and the one that draws the last merges the partials, so the grid may be larger than
    the machine and needs no co-residency. ``gqa_fwd_batch_decode`` takes the same path."""
    return gqa_fwd_batch_decode(q, k_cache, v_cache, workspace, q_lens, kv_lens, block_table, scale, soft_cap,
                                output_split, output_combine, kv_split, max_kv_len)


def kernel_inter_rank_gqa_fwd_batch_decode_combine_kv(partials: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16):
    """Merge per-rank partials fp32 ``[R, B, Hq, D + 1]`` (LSE last; ``-inf`` marks a rank without KV) -> [B, Hq, D]."""
    R, B, Hq, D1 = partials.shape
    flat = partials.reshape(R, B * Hq, D1)
    return ops.combine_partials(flat[..., :-1], flat[..., -1], out_dtype).reshape(B, Hq, D1 - 1)


def get_triton_combine_kv_algo_info(*args, **kwargs) -> dict:
    """The reference returns AOT algo-info for its Triton kernel; the nvcc-built kernel has one configuration."""
    return {"BLOCK_DV": 128, "num_warps": 4}


gqa_fwd_batch_decode_aot = gqa_fwd_batch_decode
gqa_fwd_batch_decode_intra_rank_aot = gqa_fwd_batch_decode_intra_rank
gqa_fwd_batch_decode_persistent_aot = gqa_fwd_batch_decode_persistent
kernel_gqa_fwd_batch_decode_split_kv_persistent = gqa_fwd_batch_decode_persistent
