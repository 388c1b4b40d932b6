"""Serving engine: prefill, then a CUDA-graph-captured decode step replayed per token.

API parity with ``python/triton_dist/models/engine.py:37-187``: ``Engine(model_config, temperature, top_p,
verbose, group)``, attributes ``backend`` / ``no_graph`` / ``enable_profile``, and ``serve(input_ids, gen_len)``.
The decode graph contains the whole forward (embedding to logits); sampling runs after each replay, as
in the reference (:164-177).
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..kernels.allreduce import AllReduceMethod
from .config import ModelConfig
from .kv_cache import KV_Cache
from .qwen import Qwen3
from .utils import logger, sample_token


class Engine:

    def __init__(self, model_config: ModelConfig, temperature: float = 0.6, top_p: float = 0.95, verbose: bool = False,
                 group=None, model: Qwen3 | None = None):
        self.model_config = model_config
        self.temperature, self.top_p, self.verbose, self.group = temperature, top_p, verbose, group
        self.backend = "triton_dist_AR"      # decode backend: torch | triton_dist | triton_dist_AR
        self.prefill_backend = None          # None = same as `backend`
        self.no_graph = False
        self.enable_profile = False
        self.ar_method: AllReduceMethod | None = None
        self.model = model if model is not None else Qwen3(model_config, group)
        self.kv_cache: KV_Cache | None = None
        self.graph = None
        self.bsz = None

    # ------------------------------------------------------------------ set-up
    def _init_kv_cache(self, bsz: int) -> None:
        a = self.model.arch
        if self.kv_cache is None or self.kv_cache.batch_size != bsz:
            self.kv_cache = KV_Cache(a.num_hidden_layers, bsz, self.model_config.max_length, a.num_key_value_heads,
                                     a.head_dim, self.model_config.dtype, self.model_config.world_size)
        self.kv_cache.clear()

    def _set_backend(self, backend: str, max_M: int) -> None:
        m = self.model
        if backend == "triton_dist":
            m.init_triton_dist_ctx(max_M)
        elif backend == "triton_dist_AR":
            m.init_triton_dist_AR_ctx(max_M, self.ar_method)
        m.set_fwd(backend)

    def _decode_step(self) -> None:
        self._static_pos.copy_(self.kv_cache.kv_offset.to(torch.int64)[:, None])
        self._static_logits = self.model.inference(self._static_ids, self._static_pos, self.kv_cache)

    def _init_cuda_graph(self) -> None:
        """Warm up on a side stream, then capture one decode step (static input / position / logits buffers)."""
        self.graph = None
        if self.no_graph:
            return
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                self._decode_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if dist.is_initialized() and self.model_config.world_size > 1:
            dist.barrier(group=self.group)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._decode_step()
        self.graph = g
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ steps
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        bsz, plen = input_ids.shape
        self.bsz = bsz
        self._init_kv_cache(bsz)
        backend = self.prefill_backend or self.backend
        self._set_backend(backend, max(bsz * plen, bsz))
        pos = torch.arange(plen, device=input_ids.device, dtype=torch.int64)[None, :].expand(bsz, plen).contiguous()
        logits = self.model.inference(input_ids, pos, self.kv_cache)
        self.kv_cache.kv_offset.fill_(plen)
        return sample_token(logits, self.temperature, self.top_p)

    @torch.no_grad()
    def prepare_decode(self, first_token: torch.Tensor) -> None:
        bsz = first_token.shape[0]
        self._set_backend(self.backend, max(bsz, self.model_config.world_size))
        self._static_ids = first_token.clone()
        self._static_pos = torch.zeros((bsz, 1), dtype=torch.int64, device=first_token.device)
        self._static_logits = None
        self._init_cuda_graph()

    @torch.no_grad()
    def decode_one(self, token: torch.Tensor | None = None) -> torch.Tensor:
        """One decode step: feed `token` (default: the previously sampled one), return the next token ids [B, 1]."""
        if token is not None:
            self._static_ids.copy_(token, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self._decode_step()
        nxt = sample_token(self._static_logits, self.temperature, self.top_p)
        self.kv_cache.inc_offset()
        self._static_ids.copy_(nxt)
        return nxt

    @torch.no_grad()
    def serve(self, input_ids: torch.Tensor, gen_len: int) -> torch.Tensor:
        """Prefill `input_ids` [B, S] and generate `gen_len` tokens. Returns [B, S + gen_len]."""
        if input_ids.shape[1] + gen_len > self.model_config.max_length:
            raise ValueError("prompt + generation exceeds max_length")
        t0 = time.time()
        nxt = self.prefill(input_ids)
        out = [input_ids, nxt]
        self.prepare_decode(nxt)
        torch.cuda.synchronize()
        t1 = time.time()
        prof = None
        if self.enable_profile:
            from ..utils import get_torch_prof_ctx
            prof = get_torch_prof_ctx(True)
            prof.__enter__()
        for _ in range(gen_len - 1):
            out.append(self.decode_one())
        torch.cuda.synchronize()
        from ..runtime.heap import get_heap, heap_initialized
        if heap_initialized():
            get_heap().check_status("Engine.serve")  # an expired wait means tokens computed from incomplete sums
        if prof is not None:
            prof.__exit__(None, None, None)
            prof.export_chrome_trace(f"decode_rank{self.model_config.rank}.json")
        t2 = time.time()
        if self.verbose and self.model_config.rank == 0:
            logger.info(f"prefill+setup {t1 - t0:.3f}s, decode {gen_len - 1} steps {t2 - t1:.3f}s "
                        f"({(t2 - t1) / max(gen_len - 1, 1) * 1e3:.3f} ms/step)")
        return torch.cat(out, dim=1)
