"""Sequence-parallel prefill attention by all-gathering the KV shards (context parallelism without a ring).

API parity with ``python/triton_dist/kernels/nvidia/sp_ag_attention_intra_node.py``
(``create_sp_ag_attention_context_intra_node`` :59, ``fused_sp_ag_attn_intra_node`` :432): Q stays sharded along the
sequence, every rank's K/V shard is gathered into a symmetric buffer, and each rank runs causal variable-length
attention of its Q rows over the gathered keys, with the zig-zag sharding that balances causal work.

As in the reference snapshot, the gather completes before attention starts (its kernel has no per-shard wait,
:159-183). The gather is this library's push all-gather kernel over NVLink; the attention math is the library SDPA
call, which is the role flash-attn plays for the reference's layers. The inter-node twin is out of scope.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.nn.functional as F

from ...runtime.heap import SymmHeap, get_heap
from .low_latency_allgather import FastAllGatherContext, create_fast_allgather_context, fast_allgather


@dataclasses.dataclass
class SPAllGatherAttentionContextIntraNode:
    rank: int
    world_size: int
    heap: SymmHeap
    ag_ctx: FastAllGatherContext
    k_buffer: torch.Tensor   # symmetric [world, max_kv_shard_tokens, kv_head, head_dim]
    v_buffer: torch.Tensor

    def finalize(self) -> None:
        torch.cuda.synchronize()
        self.heap.free(self.k_buffer)
        self.heap.free(self.v_buffer)
        self.ag_ctx.finalize()


def create_sp_ag_attention_context_intra_node(batch_size: int, q_head: int, kv_head: int, max_seqlen_k: int,
                                              max_q_shard_len: int, head_dim: int, input_dtype, output_dtype, rank: int,
                                              world_size: int, device="cuda") -> SPAllGatherAttentionContextIntraNode:
    heap = get_heap()
    shard = batch_size * ((max_seqlen_k + world_size - 1) // world_size)
    kb = heap.create_tensor((world_size, shard, kv_head, head_dim), input_dtype, align=1024)
    vb = heap.create_tensor((world_size, shard, kv_head, head_dim), input_dtype, align=1024)
    ag = create_fast_allgather_context(rank, 0, world_size, 1, max_buffer_size=16)
    return SPAllGatherAttentionContextIntraNode(rank, world_size, heap, ag, kb, vb)


def zigzag_positions(seq_len: int, rank: int, world: int, device) -> torch.Tensor:
    """Global positions of the tokens rank `rank` holds under zig-zag sharding: the sequence is cut into 2 * world
    chunks and rank r owns chunks r and 2 * world - 1 - r, so causal work is equal on every rank."""
    c = seq_len // (2 * world)
    a = torch.arange(rank * c, (rank + 1) * c, device=device)
    b = torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c, device=device)
    return torch.cat([a, b])


def fused_sp_ag_attn_intra_node(ctx: SPAllGatherAttentionContextIntraNode, q_shard: torch.Tensor, k_shard: torch.Tensor,
                                v_shard: torch.Tensor, output: torch.Tensor | None, cu_seqlens_q: torch.Tensor,
                                cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, rank: int,
                                world_size: int, is_causal: bool = True, enable_zig_zag: bool = True) -> torch.Tensor:
    """q_shard [sum_q_local, Hq, D]; k_shard / v_shard [sum_k_local, Hkv, D] (this rank's tokens of every sequence,
    concatenated); cu_seqlens_q int32 [B + 1] over the LOCAL q tokens; cu_seqlens_k int32 [B + 1] over the GLOBAL keys.
    Every sequence length must be divisible by ``2 * world`` (zig-zag) or ``world``. Returns [sum_q_local, Hq, D]."""
    n_local = k_shard.shape[0]
    ctx.k_buffer[rank, :n_local].copy_(k_shard)
    ctx.v_buffer[rank, :n_local].copy_(v_shard)
    ctx.heap.barrier_all()
    fast_allgather(ctx.k_buffer, ctx.ag_ctx, mode="push2d")
    fast_allgather(ctx.v_buffer, ctx.ag_ctx, mode="push2d")
    if output is None:
        output = torch.empty_like(q_shard)
    cu_q, cu_k = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    scale = q_shard.shape[-1] ** -0.5
    for b in range(len(cu_q) - 1):
        Lk = cu_k[b + 1] - cu_k[b]
        lk_local = Lk // world_size
        k_off = cu_k[b] // world_size
        # assemble the sequence's keys in global order from the per-rank shards
        k_full = torch.empty((Lk, *k_shard.shape[1:]), dtype=k_shard.dtype, device=k_shard.device)
        v_full = torch.empty_like(k_full)
        for r in range(world_size):
            pos = zigzag_positions(Lk, r, world_size, k_shard.device) if enable_zig_zag else torch.arange(
                r * lk_local, (r + 1) * lk_local, device=k_shard.device)
            k_full[pos] = ctx.k_buffer[r, k_off:k_off + lk_local]
            v_full[pos] = ctx.v_buffer[r, k_off:k_off + lk_local]
        q = q_shard[cu_q[b]:cu_q[b + 1]]
        lq = q.shape[0]
        qpos = zigzag_positions(Lk, rank, world_size, q.device) if enable_zig_zag else torch.arange(
            rank * lq, (rank + 1) * lq, device=q.device)
        mask = (torch.arange(Lk, device=q.device)[None, :] <= qpos[:, None]) if is_causal else None
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k_full.transpose(0, 1)[None], v_full.transpose(0, 1)[None],
                                           attn_mask=mask, scale=scale, enable_gqa=True)
        output[cu_q[b]:cu_q[b + 1]] = o[0].transpose(0, 1)
    ctx.heap.barrier_all()
    return output


def create_sp_ag_attention_context_inter_node(*args, **kwargs):
    """The reference's two-level (node x local rank) variant (``sp_ag_attention_inter_node.py:504-594``). Ranks of one
    NVSwitch domain are all one hop apart, so the single-level context serves; more than one node is not supported."""
    return create_sp_ag_attention_context_intra_node(*args, **kwargs)


def fused_sp_ag_attn_inter_node(*args, **kwargs):
    """See ``create_sp_ag_attention_context_inter_node``: same kernel path as the intra-node form."""
    return fused_sp_ag_attn_intra_node(*args, **kwargs)
