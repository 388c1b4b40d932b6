"""Qwen3-MoE-shaped decoder (Qwen3-30B-A3B / Qwen3-235B-A22B architectures): the dense model with every MLP replaced
by a tensor-parallel mixture-of-experts block (``layers/nvidia/tp_moe.py``). The reference has no MoE model class; it
exercises its MoE kernels only from tests. ``Qwen3`` builds MoE layers whenever the architecture names experts, so
this class is that model under its own name."""
from __future__ import annotations

from .qwen import Qwen3


class Qwen3MoE(Qwen3):
    pass
