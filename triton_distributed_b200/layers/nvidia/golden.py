"""Library composition used by the ``torch`` forward mode: the baseline every native path is measured against.

The reference's torch mode is cuBLAS + NCCL plus ``flashinfer.norm.rmsnorm``,
``flashinfer.apply_rope_with_cos_sin_cache_inplace`` and ``flash_attn_with_kvcache``
(``python/triton_dist/layers/nvidia/tp_attn.py:60-75,159-195``). The same three library calls are used here when
they import and run on this GPU; each one is probed once on a tiny input and replaced by its plain PyTorch
statement when the probe fails (missing package, no kernel image for the device, JIT compiler absent).
``describe()`` says which ones are active so a benchmark can print it next to its baseline number.

Set ``B200DIST_GOLDEN_LIBS=0`` to force the plain PyTorch statements (they are the fp32-accurate oracle of the tests).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

_state: dict = {"probed": False, "rmsnorm": None, "rope": None, "attn": None, "notes": {}}


def _probe() -> None:
    if _state["probed"]:
        return
    _state["probed"] = True
    notes = _state["notes"]
    if os.environ.get("B200DIST_GOLDEN_LIBS", "1") == "0" or not torch.cuda.is_available():
        notes["libs"] = "disabled" if torch.cuda.is_available() else "no CUDA device"
        return
    dev = torch.device("cuda", torch.cuda.current_device())
    try:
        from flashinfer.norm import rmsnorm as fi_rmsnorm
        x = torch.randn(4, 128, device=dev, dtype=torch.bfloat16)
        w = torch.ones(128, device=dev, dtype=torch.bfloat16)
        y = fi_rmsnorm(x, w, 1e-6)
        torch.cuda.synchronize()
        ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
        if not torch.allclose(y.float(), ref.float(), atol=3e-2, rtol=3e-2):
            raise RuntimeError("flashinfer rmsnorm disagrees with the PyTorch statement")
        _state["rmsnorm"] = fi_rmsnorm
        notes["rmsnorm"] = "flashinfer.norm.rmsnorm"
    except Exception as e:  # noqa: BLE001
        notes["rmsnorm"] = f"torch ({type(e).__name__}: {str(e)[:80]})"
    try:
        from flashinfer import apply_rope_with_cos_sin_cache_inplace as fi_rope
        T, D = 4, 128
        q = torch.randn(T, 2 * D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
        cs = torch.randn(16, D, device=dev, dtype=torch.float32)
        pos = torch.arange(T, device=dev, dtype=torch.int64)
        want = rope_torch(q.view(T, 2, D), cs, pos)
        fi_rope(positions=pos, query=q, key=k, head_size=D, cos_sin_cache=cs, is_neox=True)
        torch.cuda.synchronize()
        if not torch.allclose(q.view(T, 2, D).float(), want.float(), atol=5e-2, rtol=5e-2):
            raise RuntimeError("flashinfer rope disagrees with the PyTorch statement")
        _state["rope"] = fi_rope
        notes["rope"] = "flashinfer.apply_rope_with_cos_sin_cache_inplace"
    except Exception as e:  # noqa: BLE001
        notes["rope"] = f"torch ({type(e).__name__}: {str(e)[:80]})"
    try:
        from flash_attn import flash_attn_with_kvcache
        q = torch.randn(1, 1, 2, 128, device=dev, dtype=torch.bfloat16)
        kc = torch.zeros(1, 256, 1, 128, device=dev, dtype=torch.bfloat16)
        vc = torch.zeros(1, 256, 1, 128, device=dev, dtype=torch.bfloat16)
        kn = torch.randn(1, 1, 1, 128, device=dev, dtype=torch.bfloat16)
        lens = torch.zeros(1, device=dev, dtype=torch.int32)
        o = flash_attn_with_kvcache(q, kc, vc, k=kn, v=kn, cache_seqlens=lens, causal=True)
        torch.cuda.synchronize()
        if not torch.allclose(o[0, 0, 0].float(), kn[0, 0, 0].float(), atol=2e-2, rtol=2e-2):
            raise RuntimeError("flash_attn_with_kvcache disagrees with the one-key case")
        _state["attn"] = flash_attn_with_kvcache
        notes["attention"] = "flash_attn.flash_attn_with_kvcache"
    except Exception as e:  # noqa: BLE001
        notes["attention"] = f"torch SDPA ({type(e).__name__}: {str(e)[:80]})"


def describe() -> dict:
    """Which library kernels the torch mode runs on this machine (after the one-time probe)."""
    _probe()
    return dict(_state["notes"])


def rmsnorm_torch(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def rope_torch(x: torch.Tensor, cos_sin: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """x [T, H, D] (any float dtype), neox style, cos_sin fp32 [max_pos, D] = cos | sin."""
    D = x.shape[-1]
    cs = cos_sin[pos.long()]
    cos, sin = cs[:, None, : D // 2], cs[:, None, D // 2:]
    xf = x.float()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last dimension of a tensor of any rank (library kernel when available)."""
    _probe()
    fn = _state["rmsnorm"]
    if fn is None or not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16):
        return rmsnorm_torch(x, w, eps)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return fn(x2, w, eps).view(x.shape)


def rope_(q: torch.Tensor, k: torch.Tensor, cos_sin: torch.Tensor, pos: torch.Tensor):
    """Rotate q [T, Hq, D] and k [T, Hkv, D] (contiguous); returns the rotated pair (in place when the library runs)."""
    _probe()
    fn = _state["rope"]
    if fn is None or not q.is_cuda:
        return rope_torch(q, cos_sin, pos), rope_torch(k, cos_sin, pos)
    T, Hq, D = q.shape
    q2, k2 = q.reshape(T, Hq * D), k.reshape(T, k.shape[1] * D)
    fn(positions=pos.to(torch.int64), query=q2, key=k2, head_size=D, cos_sin_cache=cos_sin, is_neox=True)
    return q2.view(T, Hq, D), k2.view(T, -1, D)


def attention_with_kvcache(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, cache_seqlens: torch.Tensor) -> torch.Tensor:
    """Append k_new / v_new [B, S, Hkv, D] to the dense caches [B, L, Hkv, D] at `cache_seqlens` (int32 [B]) and return
    causal attention of q [B, S, Hq, D] over the cache: the contract of ``flash_attn_with_kvcache``.

    The fallback has no host synchronisation, so either form can be captured in a CUDA graph."""
    _probe()
    fn = _state["attn"]
    if fn is not None and q.is_cuda:
        return fn(q, k_cache, v_cache, k=k_new, v=v_new, cache_seqlens=cache_seqlens, causal=True)
    B, S, Hq, D = q.shape
    L = k_cache.shape[1]
    pos = cache_seqlens.to(torch.int64)[:, None] + torch.arange(S, device=q.device)[None, :]      # [B, S]
    bidx = torch.arange(B, device=q.device)[:, None].expand(B, S)
    k_cache[bidx, pos] = k_new
    v_cache[bidx, pos] = v_new
    mask = (torch.arange(L, device=q.device)[None, None, :] <= pos[:, :, None])[:, None]            # [B, 1, S, L]
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k_cache.transpose(1, 2), v_cache.transpose(1, 2),
                                       attn_mask=mask, enable_gqa=True)
    return o.transpose(1, 2)
