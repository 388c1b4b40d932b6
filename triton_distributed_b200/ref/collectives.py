"""Reference semantics of the dense collectives and their fused GEMM forms (torch.distributed only)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def ag_gemm_ref(a_local: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """``all_gather(a_local)[M, K] @ b[N_local, K].T`` -> [M, N_local]; rows in rank order."""
    world = _world(group)
    if world == 1:
        full = a_local
    else:
        full = torch.empty((a_local.shape[0] * world, a_local.shape[1]), dtype=a_local.dtype, device=a_local.device)
        dist.all_gather_into_tensor(full, a_local.contiguous(), group=group)
    return (full.float() @ b.float().t()).to(a_local.dtype)


def gemm_rs_ref(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """``reduce_scatter(a[M, K_local] @ b[N, K_local].T)`` -> this rank's rows [M / world, N]."""
    world = _world(group)
    full = a.float() @ b.float().t()
    if world == 1:
        return full.to(a.dtype)
    out = torch.empty((a.shape[0] // world, b.shape[0]), dtype=torch.float32, device=a.device)
    dist.reduce_scatter_tensor(out, full.contiguous(), group=group) if a.is_cuda else _rs_via_allreduce(out, full, group)
    return out.to(a.dtype)


def _rs_via_allreduce(out: torch.Tensor, full: torch.Tensor, group) -> None:
    """gloo has no reduce_scatter: all-reduce and keep the own slice."""
    dist.all_reduce(full, group=group)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    per = full.shape[0] // world
    out.copy_(full[rank * per:(rank + 1) * per])


def all_reduce_ref(x: torch.Tensor, group=None) -> torch.Tensor:
    y = x.float().clone()
    if _world(group) > 1:
        dist.all_reduce(y, group=group)
    return y.to(x.dtype)


def all_reduce_rmsnorm_ref(x: torch.Tensor, residual: torch.Tensor | None, gamma: torch.Tensor, eps: float, group=None):
    """``h = all_reduce(x) + residual`` (stored in x's dtype); ``y = rmsnorm(h) * gamma``. Returns (y, h)."""
    s = x.float().clone()
    if _world(group) > 1:
        dist.all_reduce(s, group=group)
    if residual is not None:
        s = s + residual.float()
    h = s.to(x.dtype)
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    return y.to(x.dtype), h


def fast_allgather_ref(local: torch.Tensor, group=None) -> torch.Tensor:
    """[world, *local.shape] with slot r holding rank r's tensor."""
    world = _world(group)
    if world == 1:
        return local[None].clone()
    outs = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(outs, local.contiguous(), group=group)
    return torch.stack(outs)
