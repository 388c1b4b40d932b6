"""Weights: read Hugging Face safetensors checkpoints shard-by-shard, write random-initialised ones.

The reference loads the full ``Qwen3ForCausalLM`` on every rank and slices it
(``python/triton_dist/models/qwen.py:147-162``). Here each rank opens the shards named by
``model.safetensors.index.json`` and reads only the row/column ranges it owns
(``safe_open(...).get_slice``), so host memory per rank is one tensor slice, not the model.
``write_random_checkpoint`` produces a checkpoint in the same layout for machines without a network.
"""
from __future__ import annotations

import json
import os

import torch

from .config import ArchConfig


def hf_param_shapes(arch: ArchConfig) -> dict[str, tuple[int, ...]]:
    """Names and shapes of a Qwen3 (dense or MoE) ``state_dict`` in Hugging Face layout."""
    H, D = arch.hidden_size, arch.head_dim
    out = {"model.embed_tokens.weight": (arch.vocab_size, H), "model.norm.weight": (H,)}
    if not arch.tie_word_embeddings:
        out["lm_head.weight"] = (arch.vocab_size, H)
    for i in range(arch.num_hidden_layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (H,)
        out[p + "post_attention_layernorm.weight"] = (H,)
        out[p + "self_attn.q_proj.weight"] = (arch.num_attention_heads * D, H)
        out[p + "self_attn.k_proj.weight"] = (arch.num_key_value_heads * D, H)
        out[p + "self_attn.v_proj.weight"] = (arch.num_key_value_heads * D, H)
        out[p + "self_attn.o_proj.weight"] = (H, arch.num_attention_heads * D)
        out[p + "self_attn.q_norm.weight"] = (D,)
        out[p + "self_attn.k_norm.weight"] = (D,)
        if arch.num_experts:
            out[p + "mlp.gate.weight"] = (arch.num_experts, H)
            for e in range(arch.num_experts):
                q = p + f"mlp.experts.{e}."
                out[q + "gate_proj.weight"] = (arch.moe_intermediate_size, H)
                out[q + "up_proj.weight"] = (arch.moe_intermediate_size, H)
                out[q + "down_proj.weight"] = (H, arch.moe_intermediate_size)
        else:
            out[p + "mlp.gate_proj.weight"] = (arch.intermediate_size, H)
            out[p + "mlp.up_proj.weight"] = (arch.intermediate_size, H)
            out[p + "mlp.down_proj.weight"] = (H, arch.intermediate_size)
    return out


def _init_tensor(name: str, shape: tuple[int, ...], dtype: torch.dtype, seed: int, device="cpu") -> torch.Tensor:
    """N(0, 0.02) for matrices, ones for norm gains; the stream depends only on (seed, name)."""
    if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
        return torch.ones(shape, dtype=dtype, device=device)
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + sum(ord(c) * (i + 1) for i, c in enumerate(name))) % (2**31 - 1))
    return (torch.randn(shape, generator=g, dtype=torch.float32, device=device) * 0.02).to(dtype)


def write_random_checkpoint(path: str, arch: ArchConfig, dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                            max_shard_bytes: int = 2 << 30) -> None:
    """Write ``config.json``, ``model.safetensors.index.json`` and ``model-XXXXX-of-YYYYY.safetensors``."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    shapes = hf_param_shapes(arch)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, shape in shapes.items():
        t = _init_tensor(name, shape, dtype, seed)
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = t
        size += nbytes
    weight_map = {}
    for i, shard in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(path, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in shard})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    cfg = {
        "architectures": ["Qwen3MoeForCausalLM" if arch.num_experts else "Qwen3ForCausalLM"],
        "hidden_size": arch.hidden_size, "intermediate_size": arch.intermediate_size,
        "num_hidden_layers": arch.num_hidden_layers, "num_attention_heads": arch.num_attention_heads,
        "num_key_value_heads": arch.num_key_value_heads, "head_dim": arch.head_dim, "vocab_size": arch.vocab_size,
        "rms_norm_eps": arch.rms_norm_eps, "rope_theta": arch.rope_theta,
        "tie_word_embeddings": arch.tie_word_embeddings, "num_experts": arch.num_experts,
        "num_experts_per_tok": arch.num_experts_per_tok, "moe_intermediate_size": arch.moe_intermediate_size,
        "norm_topk_prob": arch.norm_topk_prob, "torch_dtype": str(dtype).replace("torch.", ""),
    }
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)


def read_arch_from_checkpoint(path: str) -> ArchConfig:
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    return ArchConfig(
        hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"],
        num_hidden_layers=c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
        num_key_value_heads=c["num_key_value_heads"],
        head_dim=c.get("head_dim", c["hidden_size"] // c["num_attention_heads"]), vocab_size=c["vocab_size"],
        rms_norm_eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e6),
        tie_word_embeddings=c.get("tie_word_embeddings", False), num_experts=c.get("num_experts", 0) or 0,
        num_experts_per_tok=c.get("num_experts_per_tok", 0) or 0,
        moe_intermediate_size=c.get("moe_intermediate_size", 0) or 0, norm_topk_prob=c.get("norm_topk_prob", True))


class WeightSource:
    """``get(name, rows=slice|None, cols=slice|None)`` -> tensor slice on `device`."""

    def get(self, name: str, rows: slice | None = None, cols: slice | None = None) -> torch.Tensor:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        raise NotImplementedError


class SafetensorsSource(WeightSource):
    """Reads slices out of a sharded HF checkpoint without materialising whole tensors."""

    def __init__(self, path: str, device="cuda", dtype: torch.dtype | None = None):
        from safetensors import safe_open
        self.path, self.device, self.dtype = path, device, dtype
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map = json.load(f)["weight_map"]
        else:
            self.weight_map = {}
            for fn in sorted(os.listdir(path)):
                if fn.endswith(".safetensors"):
                    with safe_open(os.path.join(path, fn), "pt") as f:
                        self.weight_map.update({k: fn for k in f.keys()})
        self._open = {}
        self._safe_open = safe_open

    def _file(self, fname: str):
        if fname not in self._open:
            self._open[fname] = self._safe_open(os.path.join(self.path, fname), "pt")
        return self._open[fname]

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def get(self, name, rows=None, cols=None):
        sl = self._file(self.weight_map[name]).get_slice(name)
        if rows is None and cols is None:
            t = sl[:]
        elif cols is None:
            t = sl[rows]
        else:
            t = sl[rows if rows is not None else slice(None), cols]
        t = t.to(self.device)
        return t.to(self.dtype) if self.dtype is not None else t


class RandomSource(WeightSource):
    """Random initialisation in HF layout.

    ``consistent=True`` draws every full tensor from a stream keyed by (seed, name) and slices it, so any
    tensor-parallel split sees the same model (tests). ``consistent=False`` draws only the requested slice,
    keyed additionally by the slice, which is what lets a 32B-parameter model be initialised per rank in
    seconds; the result is a valid random-init model, just not the same one for different world sizes.
    """

    def __init__(self, arch: ArchConfig, dtype: torch.dtype, seed: int = 0, device="cuda", consistent: bool = True):
        self.shapes = hf_param_shapes(arch)
        self.dtype, self.seed, self.device, self.consistent = dtype, seed, device, consistent

    def has(self, name: str) -> bool:
        return name in self.shapes

    def get(self, name, rows=None, cols=None):
        shape = self.shapes[name]
        if self.consistent:
            t = _init_tensor(name, shape, self.dtype, self.seed, device="cpu")
            if rows is not None:
                t = t[rows]
            if cols is not None:
                t = t[:, cols]
            return t.contiguous().to(self.device)
        r = range(shape[0])[rows] if rows is not None else range(shape[0])
        if len(shape) == 1:
            return _init_tensor(name, (len(r),), self.dtype, self.seed, device=self.device)
        c = range(shape[1])[cols] if cols is not None else range(shape[1])
        key = f"{name}[{r.start}:{r.stop},{c.start}:{c.stop}]"
        if name.endswith("norm.weight"):
            return torch.ones((len(r), len(c)), dtype=self.dtype, device=self.device)
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1000003 + sum(ord(ch) * (i + 1) for i, ch in enumerate(key))) % (2**31 - 1))
        out = torch.empty((len(r), len(c)), dtype=self.dtype, device=self.device)
        out.normal_(0.0, 0.02, generator=g)
        return out
