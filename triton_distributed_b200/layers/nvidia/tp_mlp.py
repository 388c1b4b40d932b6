"""Tensor-parallel SwiGLU MLP.

API parity with ``python/triton_dist/layers/nvidia/tp_mlp.py:51-241``: ``_init_parameters``, ``_init_ctx``,
``_init_AR_ctx``, the three forward modes ``torch_fwd`` (cuBLAS + NCCL all-reduce, the golden and the
baseline), ``dist_triton_fwd`` (AG-GEMM -> SwiGLU -> GEMM-RS on sequence-sharded activations) and
``dist_triton_AR_fwd`` (GEMM + AllReduce on replicated activations), and the unit ops used by its tests.

Column-parallel ``gate_up = [gate shard; up shard]`` (rows) and row-parallel ``down`` (columns), as in the
reference (:76-81). B200-specific: the decode path (<= 128 tokens) runs gate/up and SwiGLU as ONE kernel,
and ``partial_fwd`` exposes the un-reduced down projection so the model can fuse the all-reduce with the
residual add and the next RMSNorm.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import ops
from ...kernels.allreduce import AllReduceMethod
from ...kernels.nvidia import (ag_gemm, all_reduce, create_ag_gemm_context, create_allreduce_ctx,
                               create_gemm_rs_context, gemm_rs)


def shard_local(weight_rows: int, world_size: int, rank: int) -> slice:
    per = weight_rows // world_size
    return slice(rank * per, (rank + 1) * per)


class TP_MLP:

    def __init__(self, rank: int = 0, world_size: int = 8, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.act_fn = F.silu
        self.gate_up_proj: torch.Tensor | None = None  # [2 * I / world, H]
        self.down_proj: torch.Tensor | None = None     # [H, I / world]
        self.ag_ctx = self.rs_ctx = self.ar_ctx = None
        self.ar_method = None

    # ------------------------------------------------------------------ parameters
    def _init_parameters(self, mlp=None, verbose: bool = False, *, gate=None, up=None, down=None):
        """From an HF-style module (``gate_proj/up_proj/down_proj`` with full weights) or from already
        sharded tensors (``gate``/``up`` [I/world, H], ``down`` [H, I/world])."""
        if mlp is not None:
            I = mlp.gate_proj.weight.shape[0]
            rows = shard_local(I, self.world_size, self.rank)
            gate = mlp.gate_proj.weight.detach()[rows]
            up = mlp.up_proj.weight.detach()[rows]
            down = mlp.down_proj.weight.detach()[:, rows]
        self.gate_up_proj = torch.cat([gate, up], dim=0).to("cuda" if torch.cuda.is_available() else gate.device).contiguous()
        self.down_proj = down.to(self.gate_up_proj.device).contiguous()
        self.dtype = self.gate_up_proj.dtype
        self.inter_local = gate.shape[0]
        self.hidden = self.gate_up_proj.shape[1]

    def _init_ctx(self, max_M: int, ag_intranode_stream=None, ag_internode_stream=None, BLOCK_M=128, BLOCK_N=256,
                  BLOCK_K=64, stages=4, ag_ctx=None, rs_ctx=None):
        """Contexts may be shared between layers of equal shape (the reference shares two across 64 layers)."""
        self.ag_ctx = ag_ctx or create_ag_gemm_context(
            torch.empty(max_M // self.world_size, self.hidden, dtype=self.dtype, device="cuda"), self.gate_up_proj,
            self.rank, self.world_size, max_M)
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

    # ------------------------------------------------------------------ forwards
    @torch.no_grad()
    def torch_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Golden / baseline: cuBLAS GEMMs + NCCL all-reduce. x: [..., H] replicated."""
        gu = F.linear(x, self.gate_up_proj)
        g, u = gu.split(self.inter_local, dim=-1)
        out = F.linear(self.act_fn(g) * u, self.down_proj)
        if self.world_size > 1:
            dist.all_reduce(out, group=self.group)
        return out

    @torch.no_grad()
    def partial_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """Native GEMMs, no reduction: returns this rank's partial sum of the down projection. x: [T, H]."""
        T = x.shape[0]
        if T <= 128:
            act = ops.gemm_skinny(x, self.gate_up_proj, swiglu=True)
            return ops.gemm_skinny(act, self.down_proj)
        act = ops.silu_mul(ops.gemm(x, self.gate_up_proj))
        return ops.linear(act, self.down_proj)

    @torch.no_grad()
    def dist_triton_AR_fwd(self, x: torch.Tensor) -> torch.Tensor:
        """GEMM + AllReduce mode on replicated activations."""
        shape = x.shape
        out = self.partial_fwd(x.reshape(-1, shape[-1]))
        if self.world_size > 1:
            out = all_reduce(out, None, self.ar_method, self.ar_ctx)
        return out.reshape(shape)

    @torch.no_grad()
    def dist_triton_fwd(self, x: torch.Tensor, ag_gemm_persistent: bool = True, gemm_rs_persistent: bool = True,
                        autotune: bool = False) -> torch.Tensor:
        """AG-GEMM -> SwiGLU -> GEMM-RS. x: this rank's rows [M / world, H]; returns [M / world, H]."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        gu = ag_gemm(x2, self.gate_up_proj, self.ag_ctx)
        act = ops.silu_mul(gu)
        out = gemm_rs(act, self.down_proj, self.rs_ctx)
        return out.reshape(shape)

    fwd = torch_fwd

    # ------------------------------------------------------------------ unit ops (tests / benchmarks)
    @torch.no_grad()
    def torch_ag_gemm(self, x: torch.Tensor) -> torch.Tensor:
        full = torch.empty((x.shape[0] * self.world_size, x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(full, x.contiguous(), group=self.group)
        return F.linear(full, self.gate_up_proj)

    @torch.no_grad()
    def dist_triton_ag_gemm(self, x: torch.Tensor, persistent: bool = True, autotune: bool = False) -> torch.Tensor:
        return ag_gemm(x, self.gate_up_proj, self.ag_ctx)

    @torch.no_grad()
    def torch_gemm_rs(self, x: torch.Tensor) -> torch.Tensor:
        full = F.linear(x, self.down_proj)
        out = torch.empty((x.shape[0] // self.world_size, full.shape[1]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, full, group=self.group)
        return out

    @torch.no_grad()
    def dist_triton_gemm_rs(self, x: torch.Tensor, persistent: bool = True, autotune: bool = False) -> torch.Tensor:
        return gemm_rs(x, self.down_proj, self.rs_ctx)
