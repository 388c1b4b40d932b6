"""Reference semantics of paged GQA decode attention and of the LSE-weighted merge of partial results."""
from __future__ import annotations

import torch
import torch.distributed as dist


def paged_decode_attention_ref(q, k_cache, v_cache, kv_lens, block_table, scale: float, soft_cap: float = 0.0):
    """q [B,Hq,D]; caches [num_blocks, page, Hkv, D]; kv_lens [B]; block_table [B, max_blocks].
    Returns (out fp32 [B,Hq,D], lse fp32 [B,Hq] natural log; -inf and zeros where kv_len == 0)."""
    B, Hq, D = q.shape
    page, Hkv = k_cache.shape[1], k_cache.shape[2]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    for b in range(B):
        L = int(kv_lens[b])
        if L == 0:
            continue
        nb = (L + page - 1) // page
        idx = block_table[b, :nb].long()
        k = k_cache[idx].reshape(-1, Hkv, D)[:L].float().repeat_interleave(G, dim=1)
        v = v_cache[idx].reshape(-1, Hkv, D)[:L].float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), k) * scale
        if soft_cap > 0:
            s = soft_cap * torch.tanh(s / soft_cap)
        lse[b] = torch.logsumexp(s, dim=-1)
        out[b] = torch.einsum("hl,lhd->hd", torch.softmax(s, dim=-1), v)
    return out, lse


def combine_partials_ref(o_parts: torch.Tensor, lse_parts: torch.Tensor):
    """o_parts [R, ..., D], lse_parts [R, ...]: merge over dim 0 with weights exp(lse - max); -inf parts are skipped."""
    m = lse_parts.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse_parts - m_safe)
    w = torch.where(torch.isinf(lse_parts), torch.zeros_like(w), w)
    den = w.sum(0)
    out = (w[..., None] * o_parts).sum(0) / den.clamp_min(1e-30)[..., None]
    out = torch.where(den[..., None] > 0, out, torch.zeros_like(out))
    lse = torch.where(den > 0, m_safe + torch.log(den.clamp_min(1e-30)), torch.full_like(den, float("-inf")))
    return out, lse


def sp_flash_decode_ref(q, k_cache, v_cache, kv_lens_local, block_table, scale: float, soft_cap: float = 0.0, group=None):
    """Sequence-parallel decode: every rank attends to its own KV shard; partials are gathered and merged.
    Returns fp32 [B, Hq, D] (identical on every rank)."""
    o, lse = paged_decode_attention_ref(q, k_cache, v_cache, kv_lens_local, block_table, scale, soft_cap)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        world = dist.get_world_size(group)
        os_ = [torch.empty_like(o) for _ in range(world)]
        ls = [torch.empty_like(lse) for _ in range(world)]
        dist.all_gather(os_, o, group=group)
        dist.all_gather(ls, lse, group=group)
        o, _ = combine_partials_ref(torch.stack(os_), torch.stack(ls))
    return o
