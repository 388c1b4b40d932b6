"""Paged KV cache, head-sharded over the tensor-parallel ranks.

Same interface as the reference's dense cache (``python/triton_dist/models/kv_cache.py:29-66``:
``update_kv_cache``, ``rand_fill_kv_cache``, ``inc_offset``, ``clear``, ``get_kv_len``) but stored as pages
``[layers, num_blocks, page, kv_heads / world, head_dim]`` with a block table, which is the layout the
decode-attention kernel reads. Sequence b owns blocks ``b * blocks_per_seq ...`` so the table is static
and a decode step can be captured in a CUDA graph.
"""
from __future__ import annotations

import torch


class KV_Cache:

    def __init__(self, num_layers: int = 32, batch_size: int = 1, max_length: int = 32 * 1024, kv_heads: int = 8,
                 head_dim: int = 128, dtype=torch.bfloat16, world_size: int = 8, page_size: int = 64,
                 device="cuda") -> None:
        self.num_layers, self.batch_size, self.max_length = num_layers, batch_size, max_length
        self.kv_heads, self.head_dim, self.dtype, self.world_size = kv_heads, head_dim, dtype, world_size
        self.page_size = page_size
        self.local_kv_heads = max(1, kv_heads // world_size)
        self.blocks_per_seq = (max_length + page_size - 1) // page_size
        nblk = batch_size * self.blocks_per_seq
        shape = (num_layers, nblk, page_size, self.local_kv_heads, head_dim)
        self.k_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.v_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.kv_offset = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.block_table = torch.arange(nblk, dtype=torch.int32, device=device).view(batch_size, self.blocks_per_seq)

    def layer(self, layer_idx: int):
        """(k pages, v pages) of one layer: [num_blocks, page, kv_heads_local, head_dim]."""
        return self.k_cache[layer_idx], self.v_cache[layer_idx]

    def slots(self, positions: torch.Tensor) -> torch.Tensor:
        """Flat slot index (block * page + offset) of token position [B, S] of every sequence -> int64 [B*S]."""
        B, S = positions.shape
        base = torch.arange(B, device=positions.device, dtype=torch.int64)[:, None] * (self.blocks_per_seq * self.page_size)
        return (base + positions.to(torch.int64)).reshape(-1)

    def update_kv_cache(self, new_k: torch.Tensor, new_v: torch.Tensor, layer_idx: int):
        """Append [B, S, kv_heads_local, D] at the current offsets (the fused rope kernel normally does this)."""
        B, S = new_k.shape[:2]
        pos = self.kv_offset[:, None].to(torch.int64) + torch.arange(S, device=new_k.device)[None, :]
        sl = self.slots(pos)
        self.k_cache[layer_idx].view(-1, self.local_kv_heads, self.head_dim)[sl] = new_k.reshape(-1, self.local_kv_heads, self.head_dim)
        self.v_cache[layer_idx].view(-1, self.local_kv_heads, self.head_dim)[sl] = new_v.reshape(-1, self.local_kv_heads, self.head_dim)
        return self.k_cache[layer_idx], self.v_cache[layer_idx], self.kv_offset

    def rand_fill_kv_cache(self, offset: int) -> None:
        self.k_cache.copy_(torch.rand_like(self.k_cache) / 10)
        self.v_cache.copy_(torch.rand_like(self.v_cache) / 10)
        self.kv_offset.fill_(offset)

    def inc_offset(self, n: int = 1) -> None:
        self.kv_offset += n

    def clear(self) -> None:
        self.kv_offset.zero_()

    def get_kv_len(self) -> torch.Tensor:
        return self.kv_offset
