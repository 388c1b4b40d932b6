"""Qwen3 dense decoder with tensor parallelism and three forward modes.

API parity with ``python/triton_dist/models/qwen.py:54-229``: ``Qwen3(model_config, group)``,
``set_fwd(mode)``, ``init_triton_dist_ctx(max_M)``, ``init_triton_dist_AR_ctx(max_M, ar_method)``,
``inference(input_ids, position_ids, kv_cache, wo_lm_head)`` and ``finalize()``.

Modes:
  ``torch``           cuBLAS GEMMs, torch norms/rope/attention, NCCL all-reduce: golden and baseline.
  ``triton_dist``     AG-GEMM + GEMM-RS; hidden states stay batch-sharded between layers.
  ``triton_dist_AR``  native GEMMs on replicated activations; each all-reduce is fused with the residual
                      add and the following RMSNorm, so a layer is 8 launches at decode.

Weights come from HF safetensors shards or random initialisation (``models/weights.py``); each rank reads
only its slices. The vocabulary is sharded over ranks for ``lm_head`` (logits are all-gathered).
"""
from __future__ import annotations


import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..kernels.allreduce import AllReduceMethod
from ..kernels.nvidia import (all_reduce_rmsnorm, create_ag_gemm_context, create_allreduce_ctx,
                              create_fast_allgather_context, create_gemm_rs_context, fast_allgather)
from ..layers.nvidia import TP_MLP, TP_Attn, _set_cos_sin_cache, golden, layer_norm
from .config import ArchConfig, ModelConfig
from .kv_cache import KV_Cache
from .weights import RandomSource, SafetensorsSource, WeightSource



class Qwen3Layer:

    def __init__(self, layer_idx: int, rank: int, world_size: int, group):
        self.layer_idx = layer_idx
        self.attn = TP_Attn(rank, world_size, group)
        self.mlp = TP_MLP(rank, world_size, group)
        self.input_norm_w = self.post_norm_w = None
        self.eps = 1e-6

    def load(self, src: WeightSource, arch: ArchConfig, rank: int, world: int) -> None:
        p = f"model.layers.{self.layer_idx}."
        D = arch.head_dim
        qs = slice(rank * arch.num_attention_heads * D // world, (rank + 1) * arch.num_attention_heads * D // world)
        kv_per = max(1, arch.num_key_value_heads // world)
        kv_idx = rank * arch.num_key_value_heads // world if arch.num_key_value_heads >= world else rank * arch.num_key_value_heads // world
        ks = slice(kv_idx * D, (kv_idx + kv_per) * D)
        Is = slice(rank * arch.intermediate_size // world, (rank + 1) * arch.intermediate_size // world)
        self.attn._init_parameters(
            q=src.get(p + "self_attn.q_proj.weight", rows=qs), k=src.get(p + "self_attn.k_proj.weight", rows=ks),
            v=src.get(p + "self_attn.v_proj.weight", rows=ks), o=src.get(p + "self_attn.o_proj.weight", cols=qs),
            q_norm=src.get(p + "self_attn.q_norm.weight") if src.has(p + "self_attn.q_norm.weight") else None,
            k_norm=src.get(p + "self_attn.k_norm.weight") if src.has(p + "self_attn.k_norm.weight") else None,
            num_heads=arch.num_attention_heads, num_kv_heads=arch.num_key_value_heads, eps=arch.rms_norm_eps)
        if arch.num_experts:
            from .qwen_moe import build_moe_block  # (imports this module, hence not at the top)
            self.mlp = build_moe_block(src, p, arch, rank, world, self.attn.group)
        else:
            self.mlp._init_parameters(gate=src.get(p + "mlp.gate_proj.weight", rows=Is), up=src.get(p + "mlp.up_proj.weight", rows=Is),
                                      down=src.get(p + "mlp.down_proj.weight", cols=Is))
        self.input_norm_w = src.get(p + "input_layernorm.weight")
        self.post_norm_w = src.get(p + "post_attention_layernorm.weight")
        self.eps = arch.rms_norm_eps

    def set_fwd(self, mode: str) -> None:
        self.mode = mode

    @torch.no_grad()
    def fwd(self, hidden, position_ids, cos_sin_cache, kv_cache, step=None):
        """Unfused layer forward for the ``torch`` and ``triton_dist`` modes (pre-norm residual block)."""
        if self.mode == "torch":  # the library composition (flashinfer norm when usable)
            def norm(h, w): return golden.rmsnorm(h, w, self.eps)
        else:
            def norm(h, w): return layer_norm(h, self.eps, w)
        residual = hidden
        x = norm(hidden, self.input_norm_w)
        if self.mode == "torch":
            x = self.attn.torch_fwd(x, position_ids, cos_sin_cache, kv_cache, self.layer_idx)
        else:
            x = self.attn.dist_triton_fwd(x, position_ids, cos_sin_cache, kv_cache, self.layer_idx, step=step)
        hidden = residual + x
        residual = hidden
        x = norm(hidden, self.post_norm_w)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = self.mlp.torch_fwd(x2) if self.mode == "torch" else self.mlp.dist_triton_fwd(x2)
        return residual + x2.reshape(x.shape)


class Qwen3:

    def __init__(self, model_config: ModelConfig, group=None, source: WeightSource | None = None):
        self.model_config = model_config
        self.group = group
        self.rank, self.world_size = model_config.rank, model_config.world_size
        self.dtype = model_config.dtype
        self.arch = model_config.arch()
        a = self.arch
        if a.num_attention_heads % self.world_size or (a.num_experts == 0 and a.intermediate_size % self.world_size) or (
                a.num_experts and a.moe_intermediate_size % self.world_size):
            raise ValueError("heads and intermediate size must be divisible by the world size")
        self.device = "cuda" if torch.cuda.is_available() else "cpu"
        self.mode = "torch"
        self.ar_ctx = self.ag_ctx_qkv = self.ag_ctx_mlp = self.rs_ctx = self.moe_ctx = None
        self.gather_ctx = None      # small-message all-gather of the native modes (logits, last hidden rows)
        self.gather_rows = 0
        self.ar_method = None
        self.max_length = model_config.max_length
        self.init_parameters(source)

    # ------------------------------------------------------------------ weights
    def init_parameters(self, source: WeightSource | None = None) -> None:
        cfg, a = self.model_config, self.arch
        if source is None:
            if cfg.checkpoint_dir:
                source = SafetensorsSource(cfg.checkpoint_dir, self.device, self.dtype)
            else:
                big = a.hidden_size * a.intermediate_size * a.num_hidden_layers > 2e9
                source = RandomSource(a, self.dtype, cfg.seed, self.device, consistent=not big)
        r, w = self.rank, self.world_size
        self.embed_tokens = source.get("model.embed_tokens.weight")
        self.vocab_pad = (a.vocab_size + w - 1) // w * w
        vs = slice(r * self.vocab_pad // w, min(a.vocab_size, (r + 1) * self.vocab_pad // w))
        head_name = "lm_head.weight" if source.has("lm_head.weight") else "model.embed_tokens.weight"
        lm = source.get(head_name, rows=vs)
        rows_local = self.vocab_pad // w
        if lm.shape[0] < rows_local:  # pad the last rank's shard so that every rank computes the same shape
            lm = torch.cat([lm, torch.zeros(rows_local - lm.shape[0], lm.shape[1], dtype=lm.dtype, device=lm.device)])
        self.lm_head = lm.contiguous()
        self.norm_w = source.get("model.norm.weight")
        self.layers = []
        for i in range(a.num_hidden_layers):
            layer = Qwen3Layer(i, r, w, self.group)
            layer.load(source, a, r, w)
            layer.set_fwd(self.mode)
            self.layers.append(layer)
        inv_freq = 1.0 / (a.rope_theta ** (torch.arange(0, a.head_dim, 2, dtype=torch.float32, device=self.device) / a.head_dim))
        self.cos_sin_cache = _set_cos_sin_cache(inv_freq, self.max_length)
        self.num_layers = a.num_hidden_layers
        self.eps = a.rms_norm_eps

    def set_fwd(self, mode: str = "torch") -> None:
        if mode not in ("torch", "triton_dist", "triton_dist_AR"):
            raise ValueError(f"unknown forward mode {mode!r}")
        self.mode = mode
        for layer in self.layers:
            layer.set_fwd(mode)

    # ------------------------------------------------------------------ contexts (shared by all layers)
    def init_triton_dist_ctx(self, max_M: int) -> None:
        H = self.arch.hidden_size
        l0 = self.layers[0]
        self._init_gather_ctx()
        dummy = torch.empty(max_M // self.world_size, H, dtype=self.dtype, device="cuda")
        if self.ag_ctx_qkv is None:
            # one gather context serves both projections (same K); one scatter context serves o_proj and down
            self.ag_ctx_qkv = create_ag_gemm_context(dummy, l0.attn.wqkv, self.rank, self.world_size, max_M)
            self.rs_ctx = create_gemm_rs_context(max_M, H, self.rank, self.world_size, self.world_size, self.dtype)
        if self.arch.num_experts and self.moe_ctx is None:
            self.layers[0].mlp._init_ctx(max_M)  # one pair of MoE contexts serves every layer
            self.moe_ctx = (self.layers[0].mlp.ag_ctx, self.layers[0].mlp.rs_ctx)
        for layer in self.layers:
            layer.attn._init_ctx(max_M, ag_ctx=self.ag_ctx_qkv, rs_ctx=self.rs_ctx)
            if self.arch.num_experts:
                layer.mlp.ag_ctx, layer.mlp.rs_ctx = self.moe_ctx
            else:
                layer.mlp._init_ctx(max_M, ag_ctx=self.ag_ctx_qkv, rs_ctx=self.rs_ctx)

    _GATHER_ROWS = 32  # batch rows the native logits gather holds; larger batches take the NCCL all-gather

    def _init_gather_ctx(self) -> None:
        """Symmetric buffers for the per-step gathers of the native modes: the vocabulary-sharded logits and, in
        ``triton_dist`` mode, the last hidden row of every sequence (both a few hundred KB)."""
        if self.world_size == 1 or self.gather_ctx is not None:
            return
        from ..runtime.heap import get_heap
        heap, w = get_heap(), self.world_size
        rows, vloc, H = self._GATHER_ROWS, self.lm_head.shape[0], self.arch.hidden_size
        self.gather_rows = rows
        self.logit_buf = heap.create_tensor((w, rows, vloc), self.dtype, align=1024)
        self.hidden_buf = heap.create_tensor((w, rows, H), self.dtype, align=1024)
        self.gather_ctx = create_fast_allgather_context(self.rank, 0, w, 1, max_buffer_size=w * rows * max(vloc, H) * 2)
        self.gather_mode = "push2d_ll_multimem" if heap.has_multicast else "push2d_ll"

    def _gather_rows(self, buf: torch.Tensor, n_rows: int) -> torch.Tensor:
        """All-gather the first n_rows of every rank's slot of `buf` [world, rows, C]; returns [world, n_rows, C]."""
        if n_rows == buf.shape[1]:
            fast_allgather(buf, self.gather_ctx, mode=self.gather_mode)
            return buf
        # fewer rows than the buffer holds: gather a compact view of the same symmetric allocation
        view = buf.view(-1)[: self.world_size * n_rows * buf.shape[2]].view(self.world_size, n_rows, buf.shape[2])
        fast_allgather(view, self.gather_ctx, mode=self.gather_mode)
        return view

    def init_triton_dist_AR_ctx(self, max_M: int, ar_method: AllReduceMethod | None = None) -> None:
        self.ar_method = ar_method
        self._init_gather_ctx()
        if self.world_size > 1 and self.ar_ctx is None:
            # fixed-size workspace: larger inputs are processed in row chunks
            self.ar_ctx = create_allreduce_ctx(64 << 20, self.rank, self.world_size, self.world_size)
        for layer in self.layers:
            for sub in (layer.attn, layer.mlp):
                sub.ar_ctx, sub.ar_method = self.ar_ctx, ar_method
        # pre-size the split-K scratch so that nothing allocates inside a CUDA graph capture
        a = self.arch
        widest = max(self.lm_head.shape[0], a.intermediate_size // self.world_size, a.hidden_size)
        ops.reserve_skinny_scratch(torch.device("cuda", torch.cuda.current_device()),
                                   2 * ((min(max_M, 256) + 15) // 16 * 16) * ((widest + 127) // 128) * 128,
                                   (widest + 127) // 128)

    def finalize(self) -> None:
        for c in (self.ar_ctx, self.ag_ctx_qkv, self.rs_ctx, self.gather_ctx) + tuple(self.moe_ctx or ()):
            if c:
                c.finalize()
        if self.gather_ctx is not None:
            from ..runtime.heap import get_heap
            get_heap().free(self.logit_buf)
            get_heap().free(self.hidden_buf)
        self.ar_ctx = self.ag_ctx_qkv = self.rs_ctx = self.moe_ctx = self.gather_ctx = None

    # ------------------------------------------------------------------ forward
    def _reduce_norm(self, partial, residual, gamma):
        """h = all_reduce(partial) + residual (in place); returns rmsnorm(h) * gamma."""
        if self.world_size > 1:
            y, _ = all_reduce_rmsnorm(partial, residual, gamma, self.eps, self.ar_ctx, self.ar_method)
            return y
        return ops.rmsnorm(partial, gamma, self.eps, residual=residual)

    @torch.no_grad()
    def _inference_AR(self, input_ids, position_ids, kv_cache):
        """Returns the final-normed hidden states [B, S, H]."""
        bsz, seqlen = input_ids.shape
        step = {"pos": position_ids.reshape(-1).to(torch.int32), "slots": kv_cache.slots(position_ids),
                "kv_lens": (position_ids[:, -1] + 1).to(torch.int32)}
        residual = ops.embedding(input_ids.reshape(-1), self.embed_tokens)  # [T, H], becomes the residual stream
        x = ops.rmsnorm(residual, self.layers[0].input_norm_w, self.eps)
        for i, layer in enumerate(self.layers):
            part = layer.attn.partial_fwd(x, position_ids, self.cos_sin_cache, kv_cache, i, bsz, seqlen, step)
            x = self._reduce_norm(part, residual, layer.post_norm_w)
            part = layer.mlp.partial_fwd(x)
            nxt = self.layers[i + 1].input_norm_w if i + 1 < self.num_layers else self.norm_w
            x = self._reduce_norm(part, residual, nxt)
        return x.view(bsz, seqlen, -1)  # already final-normed

    @torch.no_grad()
    def inference(self, input_ids: torch.Tensor, position_ids: torch.Tensor, kv_cache: KV_Cache,
                  wo_lm_head: bool = False) -> torch.Tensor:
        """input_ids / position_ids [B, S] (full batch on every rank). Returns fp32 logits [B, 1, V] of the last
        position (or the normed hidden states with ``wo_lm_head``). ``triton_dist`` mode needs B % world == 0."""
        bsz, seqlen = input_ids.shape
        native_gather = self.world_size > 1 and self.gather_ctx is not None and bsz <= self.gather_rows
        if self.mode == "triton_dist_AR":
            hidden = self._inference_AR(input_ids, position_ids, kv_cache)
        else:
            native = self.mode == "triton_dist"
            hidden = ops.embedding(input_ids, self.embed_tokens) if native else F.embedding(input_ids, self.embed_tokens)
            step = None
            if native:
                bl = bsz // self.world_size
                hidden = hidden[self.rank * bl:(self.rank + 1) * bl].contiguous()
                step = {"pos": position_ids.reshape(-1).to(torch.int32), "slots": kv_cache.slots(position_ids),
                        "kv_lens": (position_ids[:, -1] + 1).to(torch.int32)}
            for layer in self.layers:
                hidden = layer.fwd(hidden, position_ids, self.cos_sin_cache, kv_cache, step)
            if native and not wo_lm_head and native_gather:
                # only the last position feeds the head: norm and gather b_local rows instead of the whole sequence
                last_local = layer_norm(hidden[:, -1, :].contiguous(), self.eps, self.norm_w)
                bl = last_local.shape[0]
                self.hidden_buf.view(-1)[: self.world_size * bl * last_local.shape[1]].view(self.world_size, bl, -1)[self.rank].copy_(last_local)
                hidden = self._gather_rows(self.hidden_buf, bl).reshape(bsz, 1, -1)
            else:
                hidden = (golden.rmsnorm(hidden, self.norm_w, self.eps) if self.mode == "torch"
                          else layer_norm(hidden, self.eps, self.norm_w))
                if native:
                    full = torch.empty((bsz, seqlen, hidden.shape[-1]), dtype=hidden.dtype, device=hidden.device)
                    dist.all_gather_into_tensor(full, hidden.contiguous(), group=self.group)
                    hidden = full
        if wo_lm_head:
            return hidden
        last = hidden[:, -1, :].contiguous()
        if self.mode == "torch":
            local = F.linear(last, self.lm_head)
        elif native_gather:
            # the head writes its vocabulary shard straight into this rank's slot of the symmetric gather buffer
            vloc = self.lm_head.shape[0]
            slot = self.logit_buf.view(-1)[: self.world_size * bsz * vloc].view(self.world_size, bsz, vloc)[self.rank]
            ops.linear(last, self.lm_head, out=slot)
            gathered = self._gather_rows(self.logit_buf, bsz)
            local = gathered.permute(1, 0, 2).reshape(bsz, -1)
            return local[:, : self.arch.vocab_size].float().unsqueeze(1)
        else:
            local = ops.linear(last, self.lm_head)
        if self.world_size > 1:
            gathered = torch.empty((self.world_size, bsz, local.shape[-1]), dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.group)
            local = gathered.permute(1, 0, 2).reshape(bsz, -1)
        return local[:, : self.arch.vocab_size].float().unsqueeze(1)
