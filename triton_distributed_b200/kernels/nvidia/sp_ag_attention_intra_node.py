"""Sequence-parallel prefill attention by all-gathering the KV shards (context parallelism without a ring).

API parity with ``python/triton_dist/kernels/nvidia/sp_ag_attention_intra_node.py``
(``create_sp_ag_attention_context_intra_node`` :59, ``fused_sp_ag_attn_intra_node`` :432): Q stays sharded along the
sequence, every rank's K/V shard is gathered into a symmetric buffer, and each rank runs causal variable-length
attention of its Q rows over the gathered keys, with the zig-zag sharding that balances causal work.

Two native launches and no host synchronisation: ``sp_kv_scatter_kernel`` pushes every local K / V row over NVLink into
the row of its global position in every rank's buffer (the zig-zag permutation is folded into the gather), and the
tcgen05 prefill attention kernel then treats every (sequence, local chunk) as one causal problem whose keys are the
contiguous prefix that chunk may see: chunk r of a sequence cut into 2 * world chunks attends the first (r + 1)
chunks with the bottom-right aligned mask. As in the reference snapshot the gather completes before attention starts
(its kernel has no per-shard wait, :159-183). Head dim 128. The inter-node twin is out of scope.
"""
from __future__ import annotations

import dataclasses

import torch

from ... import _lib, ops
from ..._lib import ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap


@dataclasses.dataclass
class SPAllGatherAttentionContextIntraNode:
    rank: int
    world_size: int
    heap: SymmHeap
    k_buffer: torch.Tensor   # symmetric [max total keys, kv_head, head_dim], global token order
    v_buffer: torch.Tensor

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        self.heap.free(self.k_buffer)
        self.heap.free(self.v_buffer)


def create_sp_ag_attention_context_intra_node(batch_size: int, q_head: int, kv_head: int, max_seqlen_k: int,
                                              max_q_shard_len: int, head_dim: int, input_dtype, output_dtype, rank: int,
                                              world_size: int, device="cuda") -> SPAllGatherAttentionContextIntraNode:
    """Buffers for up to ``batch_size`` sequences of up to ``max_seqlen_k`` keys each (global lengths)."""
    if head_dim != 128:
        raise NotImplementedError("the native prefill attention is specialised for head_dim 128")
    heap = get_heap()
    rows = batch_size * ((max_seqlen_k + world_size - 1) // world_size) * world_size
    kb = heap.create_tensor((rows, kv_head, head_dim), input_dtype, align=1024)
    vb = heap.create_tensor((rows, kv_head, head_dim), input_dtype, align=1024)
    return SPAllGatherAttentionContextIntraNode(rank, world_size, heap, kb, vb)


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
    """q_shard [sum_q_local, Hq, 128]; k_shard / v_shard [sum_k_local, Hkv, 128] (this rank's tokens of every sequence,
    concatenated); cu_seqlens_q int32 [B + 1] over the LOCAL q tokens; cu_seqlens_k int32 [B + 1] over the GLOBAL keys.
    Every sequence length must be divisible by ``2 * world`` (zig-zag) or ``world``. Returns [sum_q_local, Hq, 128]."""
    dev = q_shard.device
    W = world_size
    k_shard, v_shard = k_shard.contiguous(), v_shard.contiguous()
    cu_q = cu_seqlens_q.to(device=dev, dtype=torch.int32)
    cu_k = cu_seqlens_k.to(device=dev, dtype=torch.int32).contiguous()
    B = cu_k.numel() - 1
    row_bytes = k_shard.shape[1] * k_shard.shape[2] * k_shard.element_size()
    if max_seqlen_k * B > ctx.k_buffer.shape[0]:
        raise ValueError("the batch does not fit the context's gather buffers")
    _lib.call("b200_sp_kv_scatter", ctx.heap.ctx, ptr(k_shard), ptr(v_shard), ptr(ctx.k_buffer), ptr(ctx.v_buffer), ptr(cu_k),
              B, k_shard.shape[0], row_bytes, 1 if enable_zig_zag else 0, stream_ptr())
    ops._count()
    ctx.heap.barrier_all()   # every rank's rows have landed everywhere
    # one causal problem per (sequence, local chunk): queries = the chunk, keys = the prefix the chunk may see
    lq = cu_q[1:] - cu_q[:-1]
    if not is_causal:
        cu_q2, cu_k2, k_lens, max_q = cu_q, cu_k, cu_k[1:] - cu_k[:-1], max_seqlen_q
    elif enable_zig_zag:
        c = lq // 2
        cu_q2 = torch.cat([torch.stack([cu_q[:-1], cu_q[:-1] + c], 1).reshape(-1), cu_q[-1:]])
        cu_k2 = torch.cat([cu_k[:-1].repeat_interleave(2), cu_k[-1:]])
        k_lens = torch.stack([(rank + 1) * c, (2 * W - rank) * c], 1).reshape(-1)
        max_q = (max_seqlen_q + 1) // 2
    else:
        cu_q2, cu_k2, k_lens, max_q = cu_q, cu_k, (rank + 1) * lq, max_seqlen_q
    out = ops.prefill_attention(q_shard.contiguous(), ctx.k_buffer, ctx.v_buffer, cu_q2, cu_k2, max_q, max_seqlen_k,
                                q_shard.shape[-1] ** -0.5, is_causal, out=output, seqlens_k=k_lens)
    ctx.heap.barrier_all()   # nobody overwrites the buffers of a rank that is still reading them
    return out


def create_sp_ag_attention_context_inter_node(*args, **kwargs):
    """The reference's two-level (node x local rank) variant (``sp_ag_attention_inter_node.py:504-594``). Ranks of one
    NVSwitch domain are all one hop apart, so the single-level context serves; more than one node is not supported."""
    return create_sp_ag_attention_context_intra_node(*args, **kwargs)


def fused_sp_ag_attn_inter_node(*args, **kwargs):
    """See ``create_sp_ag_attention_context_inter_node``: same kernel path as the intra-node form."""
    return fused_sp_ag_attn_intra_node(*args, **kwargs)
