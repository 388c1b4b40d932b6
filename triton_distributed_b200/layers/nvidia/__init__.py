"""Layers (exports follow ``python/triton_dist/layers/nvidia/__init__.py:25-29``)."""
from . import golden
from .ep_a2a_layer import EPAll2AllLayer
from .low_latency_allgather_layer import AllGatherLayer
from .sp_flash_decode_layer import SpGQAFlashDecodeAttention
from .tp_attn import TP_Attn, _set_cos_sin_cache, layer_norm
from .tp_moe import EP_MoE, TP_MoE
from .tp_mlp import TP_MLP, shard_local

__all__ = ["TP_MoE", "EP_MoE", "AllGatherLayer", "SpGQAFlashDecodeAttention", "EPAll2AllLayer", "TP_MLP", "TP_Attn", "layer_norm", "_set_cos_sin_cache", "shard_local", "golden"]
