"""Model configuration.

``ModelConfig`` keeps the fields of the reference (``python/triton_dist/models/config.py:30-37``). The
architecture tables replace the Hugging Face hub lookup, which needs a network: they carry exactly the
numbers of the published ``config.json`` files of the Qwen3 dense family, plus a tiny shape for tests.
"""
from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass
class ArchConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int = 128
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    # MoE (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True


ARCHS: dict[str, ArchConfig] = {
    "Qwen/Qwen3-8B": ArchConfig(4096, 12288, 36, 32, 8),
    "Qwen/Qwen3-14B": ArchConfig(5120, 17408, 40, 40, 8),
    "Qwen/Qwen3-32B": ArchConfig(5120, 25600, 64, 64, 8),
    "Qwen/Qwen3-30B-A3B": ArchConfig(2048, 6144, 48, 32, 4, num_experts=128, num_experts_per_tok=8,
                                     moe_intermediate_size=768),
    "Qwen/Qwen3-235B-A22B": ArchConfig(4096, 12288, 94, 64, 4, num_experts=128, num_experts_per_tok=8,
                                       moe_intermediate_size=1536),
    # what ONE rank of a tensor-parallel Qwen3-32B computes at TP = 8 (heads, KV heads and intermediate size divided by
    # eight, vocabulary shard): a single-GPU stand-in for tuning the per-rank kernel chain without the collectives
    "Qwen3-32B-tp8-shard": ArchConfig(5120, 3200, 64, 8, 1, vocab_size=18992),
    # test shapes: same structure, divisible by 8 ranks
    "tiny-qwen3": ArchConfig(512, 1024, 2, 8, 8, vocab_size=1024),
    "tiny-qwen3-gqa": ArchConfig(1024, 2048, 3, 16, 8, vocab_size=2048),
    "tiny-qwen3-moe": ArchConfig(512, 1024, 2, 8, 8, vocab_size=1024, num_experts=16, num_experts_per_tok=4,
                                 moe_intermediate_size=256),
}


@dataclasses.dataclass
class ModelConfig:
    model_name: str = "Qwen/Qwen3-32B"
    max_length: int = 4096
    dtype: torch.dtype = torch.bfloat16
    local_only: bool = False
    rank: int = 0
    world_size: int = 8
    # extensions: a directory with HF-layout safetensors (config.json + shards); None = random initialisation
    checkpoint_dir: str | None = None
    seed: int = 0
    num_layers_override: int | None = None  # build fewer layers (tests only)

    def arch(self) -> ArchConfig:
        if self.checkpoint_dir is not None:
            from .weights import read_arch_from_checkpoint
            a = read_arch_from_checkpoint(self.checkpoint_dir)
        elif self.model_name in ARCHS:
            a = ARCHS[self.model_name]
        else:
            raise ValueError(f"unknown model {self.model_name!r}; known: {sorted(ARCHS)} (or pass checkpoint_dir)")
        if self.num_layers_override is not None:
            a = dataclasses.replace(a, num_hidden_layers=self.num_layers_override)
        return a
