"""Tensor-parallel GQA attention block (Qwen3: per-head q/k RMSNorm, neox RoPE, paged KV cache).

API parity with ``python/triton_dist/layers/nvidia/tp_attn.py:60-274``: module helpers ``layer_norm``,
``_set_cos_sin_cache``; class ``TP_Attn`` with ``_init_parameters``, ``_init_ctx``, ``_init_AR_ctx`` and the
forward modes ``torch_fwd`` / ``dist_triton_fwd`` / ``dist_triton_AR_fwd``. Heads are sharded over ranks:
``wqkv = [q shard; k shard; v shard]`` (rows), ``wo`` column shard (:100-105).

The reference calls flashinfer for norm/rope and flash-attn for attention + cache append; here one native
kernel does head-norm + RoPE + cache write, the paged decode kernel does single-token attention and the tcgen05
prefill kernel does many-token attention. The ``torch`` mode keeps the library composition as golden and baseline.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import ops
from ...kernels.allreduce import AllReduceMethod
from ...kernels.nvidia import (ag_gemm, all_reduce, create_ag_gemm_context, create_allreduce_ctx,
                               create_gemm_rs_context, gemm_rs)
from . import golden
from .tp_mlp import shard_local


def layer_norm(hidden: torch.Tensor, eps: float, w: torch.Tensor) -> torch.Tensor:
    """RMSNorm (the reference names it layer_norm, tp_attn.py:60-66). Native on CUDA, torch on CPU."""
    if hidden.is_cuda:
        return ops.rmsnorm(hidden, w, eps)
    hf = hidden.float()
    return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(hidden.dtype)


def _set_cos_sin_cache(inv_freq: torch.Tensor, max_length: int) -> torch.Tensor:
    """fp32 [max_length, head_dim] = cos(half) | sin(half) (tp_attn.py:69-75)."""
    t = torch.arange(max_length, device=inv_freq.device, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq.float())
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous()


_rope_torch = golden.rope_torch

class TP_Attn:

    def __init__(self, rank: int = 0, world_size: int = 8, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.head_dim = 128
        self.wqkv = self.wo = self.q_norm_w = self.k_norm_w = None
        self.ag_ctx = self.rs_ctx = self.ar_ctx = None
        self.ar_method = None
        self._attn_ws: dict = {}

    def _init_parameters(self, attn=None, verbose: bool = False, *, q=None, k=None, v=None, o=None, q_norm=None,
                         k_norm=None, num_heads=None, num_kv_heads=None, eps: float = 1e-6):
        """From an HF-style module (full weights; ``config`` gives the head counts) or from sharded tensors."""
        if attn is not None:
            num_heads, num_kv_heads = attn.config.num_attention_heads, attn.config.num_key_value_heads
            D = self.head_dim
            q = attn.q_proj.weight.detach()[shard_local(num_heads * D, self.world_size, self.rank)]
            k = attn.k_proj.weight.detach()[shard_local(num_kv_heads * D, self.world_size, self.rank)]
            v = attn.v_proj.weight.detach()[shard_local(num_kv_heads * D, self.world_size, self.rank)]
            o = attn.o_proj.weight.detach()[:, shard_local(num_heads * D, self.world_size, self.rank)]
            q_norm, k_norm = attn.q_norm.weight.detach(), attn.k_norm.weight.detach()
            eps = getattr(attn.q_norm, "variance_epsilon", eps)
        dev = "cuda" if torch.cuda.is_available() else q.device
        self.wqkv = torch.cat([q, k, v], dim=0).to(dev).contiguous()
        self.wo = o.to(dev).contiguous()
        self.q_norm_w = q_norm.to(dev).contiguous() if q_norm is not None else None
        self.k_norm_w = k_norm.to(dev).contiguous() if k_norm is not None else None
        self.q_heads_local = num_heads // self.world_size
        self.kv_heads_local = max(1, num_kv_heads // self.world_size)
        self.hidden = self.wqkv.shape[1]
        self.dtype = self.wqkv.dtype
        self.eps = eps
        self.scale = 1.0 / math.sqrt(self.head_dim)

    def _init_ctx(self, max_M: int, ag_intranode_stream=None, ag_internode_stream=None, BLOCK_M=128, BLOCK_N=256,
                  BLOCK_K=64, stages=4, ag_ctx=None, rs_ctx=None):
        self.ag_ctx = ag_ctx or create_ag_gemm_context(
            torch.empty(max_M // self.world_size, self.hidden, dtype=self.dtype, device="cuda"), self.wqkv, self.rank,
            self.world_size, max_M)
        self.rs_ctx = rs_ctx or create_gemm_rs_context(max_M, self.hidden, self.rank, self.world_size, self.world_size,
                                                       self.dtype)

    def _init_AR_ctx(self, max_M: int, method: AllReduceMethod | None = None, dtype=None, ar_ctx=None):
        self.ar_method = method
        self.ar_ctx = ar_ctx or create_allreduce_ctx(3 * max_M * self.hidden * 2, self.rank, self.world_size, self.world_size)

    def finalize(self):
        for c in (self.ag_ctx, self.rs_ctx, self.ar_ctx):
            if c is not None:
                c.finalize()
        self.ag_ctx = self.rs_ctx = self.ar_ctx = None

    # ------------------------------------------------------------------ attention cores
    def apply_rotary_pos_emb(self, q, k, cos_sin_cache, position_ids):
        """q [T, Hq, D], k [T, Hkv, D] -> rotated copies (torch path; the native path fuses this)."""
        pos = position_ids.reshape(-1)
        return _rope_torch(q, cos_sin_cache, pos), _rope_torch(k, cos_sin_cache, pos)

    def _attn_native(self, qkv, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen, step=None):
        """qkv [B*S, (Hq + 2 Hkv) D] -> attention output [B*S, Hq*D] with k/v appended to the paged cache.
        `step` carries per-step tensors precomputed by the model (positions int32, slots, kv_lens)."""
        kp, vp = kv_cache.layer(layer_idx)
        if step is None:
            pos = position_ids.reshape(-1).to(torch.int32)
            step = {"pos": pos, "slots": kv_cache.slots(position_ids), "kv_lens": (position_ids[:, -1] + 1).to(torch.int32)}
        q = ops.qk_norm_rope(qkv, step["pos"], cos_sin_cache, self.q_heads_local, self.kv_heads_local,
                             kp.view(-1, self.kv_heads_local, self.head_dim), vp.view(-1, self.kv_heads_local, self.head_dim),
                             step["slots"], self.q_norm_w, self.k_norm_w, self.eps)
        if seqlen == 1:
            splits = step.get("splits") or ops.choose_kv_splits(bsz, self.kv_heads_local, self.q_heads_local // self.kv_heads_local,
                                                                kv_cache.max_length)
            out = ops.decode_attention(q, kp, vp, step["kv_lens"], kv_cache.block_table, self.scale, 0.0, splits,
                                       workspace=self._attn_ws)
            return out.view(bsz, -1)
        # prefill: the tcgen05 attention kernel reads this chunk's keys and values in place from the cache (sequence b
        # owns a contiguous run of slots), causal with bottom-right alignment, so a chunk after a cached prefix works too
        if self.head_dim != 128:
            raise NotImplementedError("the native prefill attention is specialised for head_dim 128")
        L = kv_cache.blocks_per_seq * kv_cache.page_size
        cu_q = torch.arange(0, (bsz + 1) * seqlen, seqlen, dtype=torch.int32, device=qkv.device)
        cu_k = torch.arange(0, (bsz + 1) * L, L, dtype=torch.int32, device=qkv.device)
        o = ops.prefill_attention(q, kp.view(-1, self.kv_heads_local, self.head_dim), vp.view(-1, self.kv_heads_local, self.head_dim),
                                  cu_q, cu_k, seqlen, min(L, kv_cache.max_length), self.scale, True, seqlens_k=step["kv_lens"])
        return o.reshape(bsz * seqlen, -1)

    def _attn_torch(self, qkv, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen):
        """The library composition of the reference's torch mode (tp_attn.py:159-195): q/k RMSNorm and RoPE from
        flashinfer, attention and the cache append from ``flash_attn_with_kvcache`` on this sequence's contiguous run
        of pages; each call falls back to its PyTorch statement when the library is unusable (see ``golden.py``)."""
        D, Hq, Hkv = self.head_dim, self.q_heads_local, self.kv_heads_local
        q, k, v = qkv.view(bsz * seqlen, -1).split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        q, k, v = q.reshape(-1, Hq, D).contiguous(), k.reshape(-1, Hkv, D).contiguous(), v.reshape(-1, Hkv, D)
        if self.q_norm_w is not None:
            q, k = golden.rmsnorm(q, self.q_norm_w, self.eps), golden.rmsnorm(k, self.k_norm_w, self.eps)
        q, k = golden.rope_(q, k, cos_sin_cache, position_ids.reshape(-1))
        kp, vp = kv_cache.layer(layer_idx)
        L = kv_cache.blocks_per_seq * kv_cache.page_size
        o = golden.attention_with_kvcache(q.view(bsz, seqlen, Hq, D), k.view(bsz, seqlen, Hkv, D),
                                          v.reshape(bsz, seqlen, Hkv, D), kp.view(bsz, L, Hkv, D), vp.view(bsz, L, Hkv, D),
                                          position_ids[:, 0].to(torch.int32).contiguous())
        return o.reshape(bsz * seqlen, Hq * D)

    # ------------------------------------------------------------------ forwards
    @torch.no_grad()
    def torch_fwd(self, x, position_ids, cos_sin_cache, kv_cache, layer_idx: int):
        """x [B, S, H] replicated -> [B, S, H] (cuBLAS + NCCL all-reduce)."""
        bsz, seqlen, _ = x.shape
        qkv = F.linear(x.reshape(bsz * seqlen, -1), self.wqkv)
        o = self._attn_torch(qkv, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen)
        out = F.linear(o, self.wo)
        if self.world_size > 1:
            dist.all_reduce(out, group=self.group)
        return out.view(bsz, seqlen, -1)

    @torch.no_grad()
    def partial_fwd(self, x2, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen, step=None):
        """Native path without the final reduction: x2 [B*S, H] -> partial o_proj output [B*S, H]."""
        qkv = ops.linear(x2, self.wqkv)
        o = self._attn_native(qkv, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen, step)
        return ops.linear(o, self.wo)

    @torch.no_grad()
    def dist_triton_AR_fwd(self, x, position_ids, cos_sin_cache, kv_cache, layer_idx: int):
        bsz, seqlen, _ = x.shape
        out = self.partial_fwd(x.reshape(bsz * seqlen, -1), position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen)
        if self.world_size > 1:
            out = all_reduce(out, None, self.ar_method, self.ar_ctx)
        return out.view(bsz, seqlen, -1)

    @torch.no_grad()
    def dist_triton_fwd(self, x, position_ids, cos_sin_cache, kv_cache, layer_idx: int, ag_gemm_persistent=True,
                        gemm_rs_persistent=True, autotune=False, step=None):
        """x: this rank's batch rows [B / world, S, H] -> [B / world, S, H]; attention runs on the gathered batch
        for the local heads, as in the reference (tp_attn.py:203-237)."""
        b_local, seqlen, _ = x.shape
        bsz = b_local * self.world_size
        qkv = ag_gemm(x.reshape(b_local * seqlen, -1), self.wqkv, self.ag_ctx)
        o = self._attn_native(qkv, position_ids, cos_sin_cache, kv_cache, layer_idx, bsz, seqlen, step)
        out = gemm_rs(o, self.wo, self.rs_ctx)
        return out.view(b_local, seqlen, -1)

    fwd = torch_fwd
