"""Sequence-parallel GQA flash-decode: the KV cache is sharded along the sequence over the ranks.

API parity with ``python/triton_dist/layers/nvidia/sp_flash_decode_layer.py:44-185``
(``SpGQAFlashDecodeAttention(rank, node, num_ranks, num_nodes, num_q_heads, num_kv_heads, q_head_dim, v_head_dim,
page_size, scale, soft_cap, max_allowed_batch, thrink_buffer_threshold, stages)`` and
``forward(q, k_cache, v_cache, global_kv_lens, block_table)``).

Two launches per call: the paged split-KV kernel over this rank's shard, then one kernel that merges the splits,
exchanges the per-rank (O, LSE) partials and does the cross-rank LSE combine. Up to ``bulk_rows`` rows (batch x query
heads; default 1024, 256 at four ranks, ``B200DIST_SP_BULK_ROWS``) the exchange uses low-latency packets (NVLS multicast when available);
above it the rows travel as plain coalesced stores behind one flag per rank, because the packet rate, not the bytes,
bounds the packet form at large batches. The reference uses four kernels and a staged symmetric buffer that it resizes
at run time; here the exchange areas are sized once from ``max_allowed_batch``.
"""
from __future__ import annotations

import os

import torch

from ... import _lib, ops
from ..._lib import c_float, dtype_code, ptr, stream_ptr
from ...runtime.heap import get_heap


class SpGQAFlashDecodeAttention:

    def __init__(self, rank: int, node: int, num_ranks: int, num_nodes: int, num_q_heads: int, num_kv_heads: int,
                 q_head_dim: int, v_head_dim: int, page_size: int = 1, scale: float = 1.0, soft_cap: float = 0.0,
                 max_allowed_batch: int = 1, thrink_buffer_threshold: int = 500, stages: int = 20,
                 use_multicast: bool | None = None, bulk_rows: int | None = None):
        if num_nodes != 1:
            raise NotImplementedError("single node only")
        if q_head_dim != 128 or v_head_dim != 128:
            raise NotImplementedError("head_dim 128 only")
        self.heap = get_heap()
        self.rank, self.num_ranks = rank, num_ranks
        self.num_q_heads, self.num_kv_heads = num_q_heads, num_kv_heads
        self.page_size, self.scale, self.soft_cap = page_size, scale, soft_cap
        self.max_allowed_batch = max_allowed_batch
        self.use_multicast = self.heap.has_multicast if use_multicast is None else use_multicast
        self.bh_cap = max_allowed_batch * num_q_heads
        self.ll = [self.heap.create_tensor((num_ranks * self.bh_cap * 129,), torch.int64, align=1024) for _ in range(2)]
        self.sync = torch.zeros(4, dtype=torch.int32, device="cuda")
        # At four ranks the packet exchange of 512 rows measured ~100 us slower than at two or eight ranks (343 us against
        # 244 us for local decode + NCCL at batch 8, 128 K tokens), so the bulk exchange takes over earlier there.
        default_rows = "256" if num_ranks == 4 else "1024"
        self.bulk_rows = int(os.environ.get("B200DIST_SP_BULK_ROWS", default_rows)) if bulk_rows is None else bulk_rows
        self.bulk = []
        if self.bh_cap > self.bulk_rows:
            self.bulk = [self.heap.create_tensor((num_ranks * self.bh_cap * 132,), torch.float32, align=1024) for _ in range(2)]
            self.bulk_flags = self.heap.create_tensor((16,), torch.int32)
            self.bulk_sync = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._ws: dict = {}
        self.heap.barrier_all()
        torch.cuda.synchronize()

    @torch.no_grad()
    def forward(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, global_kv_lens: torch.Tensor,
                block_table: torch.Tensor, max_kv_len: int | None = None, kv_split: int = -1) -> torch.Tensor:
        """q [B, Hq, 128]; k_cache / v_cache: this rank's pages [num_blocks, page, Hkv, 128]; global_kv_lens int32
        [num_ranks, B] (tokens held by every rank); block_table int32 [B, max_blocks] for the local pages."""
        B, Hq, D = q.shape
        if B > self.max_allowed_batch:
            raise ValueError(f"batch {B} exceeds max_allowed_batch {self.max_allowed_batch}")
        kv_lens = global_kv_lens[self.rank].to(torch.int32).contiguous()
        if max_kv_len is None:
            max_kv_len = block_table.shape[1] * k_cache.shape[1]
        S = kv_split if kv_split > 0 else ops.choose_kv_splits(B, self.num_kv_heads, Hq // self.num_kv_heads, max_kv_len)
        need = B * Hq * S
        if self._ws.get("rows", 0) < need:  # grows to the largest (batch, splits) seen, then stays: nothing is
            self._ws = {"rows": need,        # allocated once the shapes of a serving loop have been met
                        "o": torch.empty(need * D, dtype=torch.float32, device=q.device),
                        "lse": torch.empty(need, dtype=torch.float32, device=q.device)}
        o_part, lse_part = self._ws["o"], self._ws["lse"]
        _lib.call("b200_decode_attn", ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.stride(0),
                  ptr(kv_lens), B, Hq, self.num_kv_heads, D, k_cache.shape[1], c_float(self.scale), c_float(self.soft_cap), S,
                  ptr(o_part), ptr(lse_part), None, None, None, dtype_code(q.dtype), -1, stream_ptr())
        out = torch.empty_like(q)
        if self.bulk and B * Hq > self.bulk_rows:
            _lib.call("b200_sp_decode_combine_bulk", self.heap.ctx, ptr(o_part), ptr(lse_part), B * Hq, S, ptr(self.bulk[0]),
                      ptr(self.bulk[1]), ptr(self.bulk_flags), ptr(self.bulk_sync), ptr(out), None, dtype_code(q.dtype),
                      stream_ptr())
        else:
            _lib.call("b200_sp_decode_combine", self.heap.ctx, ptr(o_part), ptr(lse_part), B * Hq, S, ptr(self.ll[0]),
                      ptr(self.ll[1]), ptr(self.sync), ptr(out), None, dtype_code(q.dtype), 1 if self.use_multicast else 0,
                      stream_ptr())
        ops._count(2)
        return out

    __call__ = forward

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.ll + self.bulk + ([self.bulk_flags] if self.bulk else []):
            self.heap.free(t)
        self.ll, self.bulk = [], []
