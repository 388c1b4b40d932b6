"""Qwen3-MoE-shaped decoder (Qwen3-30B-A3B / Qwen3-235B-A22B architectures): the dense model with every MLP replaced
by a tensor-parallel mixture-of-experts block (``layers/nvidia/tp_moe.py``: AG + grouped GEMM up-projection, grouped GEMM
+ top-k reduce + reduce-scatter down-projection). The reference has no MoE model class; it exercises its MoE kernels
only from tests (``python/triton_dist/test/nvidia/test_ag_moe.py``, ``test_moe_reduce_rs.py``).

This module owns what is specific to the MoE variant: reading the per-expert weights of an HF checkpoint into the
stacked, intermediate-sharded layout the grouped GEMMs consume, and the model class that insists on an MoE architecture.
"""
from __future__ import annotations

import torch

from ..layers.nvidia import TP_MoE
from .config import ArchConfig, ModelConfig
from .qwen import Qwen3
from .weights import WeightSource


def build_moe_block(src: WeightSource, prefix: str, arch: ArchConfig, rank: int, world: int, group) -> TP_MoE:
    """TP_MoE block of the layer whose parameter names start with `prefix` (``model.layers.N.``). Every expert's
    intermediate dimension is sharded over the ranks: ``w_gate_up`` [E, 2 * I / world, H] (gate rows, then up rows) and
    ``w_down`` [E, H, I / world]; the router weight [E, H] is replicated."""
    if arch.moe_intermediate_size % world:
        raise ValueError("moe_intermediate_size must be divisible by the world size")
    shard = slice(rank * arch.moe_intermediate_size // world, (rank + 1) * arch.moe_intermediate_size // world)
    block = TP_MoE(rank, world, group, arch.num_experts_per_tok, arch.norm_topk_prob)
    gate_up, down = [], []
    for e in range(arch.num_experts):
        q = f"{prefix}mlp.experts.{e}."
        gate_up.append(torch.cat([src.get(q + "gate_proj.weight", rows=shard), src.get(q + "up_proj.weight", rows=shard)], dim=0))
        down.append(src.get(q + "down_proj.weight", cols=shard))
    block._init_parameters(src.get(prefix + "mlp.gate.weight"), torch.stack(gate_up), torch.stack(down))
    return block


class Qwen3MoE(Qwen3):
    """``Qwen3`` restricted to architectures with experts; ``AutoLLM`` picks it for them."""

    def __init__(self, model_config: ModelConfig, group=None, source: WeightSource | None = None):
        if not model_config.arch().num_experts:
            raise ValueError(f"{model_config.model_name} has no experts; use Qwen3")
        super().__init__(model_config, group, source)

    def expert_parameter_bytes(self) -> int:
        """Bytes of expert weights this rank holds (what a decode step streams when every expert is hit)."""
        return sum(l.mlp.w_gate_up.numel() * l.mlp.w_gate_up.element_size() + l.mlp.w_down.numel() * l.mlp.w_down.element_size()
                   for l in self.layers)
