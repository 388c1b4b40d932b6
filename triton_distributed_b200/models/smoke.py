"""One tiny prefill + decode of the flagship architecture family on ``cuda:0`` through the native kernels."""
from __future__ import annotations

import os

import torch


def run_smoke() -> None:
    from .. import ops, utils
    from . import Engine, ModelConfig
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("LOCAL_RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"), os.environ.setdefault("MASTER_PORT", "29533")
    group = utils.initialize_distributed(seed=0, heap_bytes=256 << 20)
    cfg = ModelConfig(model_name="tiny-qwen3-gqa", max_length=256, rank=0, world_size=1)
    eng = Engine(cfg, temperature=0.0, group=group)
    ids = torch.randint(0, 2048, (2, 32), device="cuda")
    before = ops.launch_count
    out = eng.serve(ids, gen_len=4)
    torch.cuda.synchronize()
    assert out.shape == (2, 36), out.shape
    assert ops.launch_count > before, "native kernels did not run"
    # cross-check against the torch-mode model on the same weights
    ref = Engine(cfg, temperature=0.0, group=group, model=eng.model)
    ref.backend = "torch"
    ref.no_graph = True
    out_ref = ref.serve(ids, gen_len=4)
    assert torch.equal(out[:, :33], out_ref[:, :33]), "first generated token differs from the torch-mode model"
    print("smoke ok: generated", out[:, 32:].tolist())
    eng.model.finalize()
    utils.finalize_distributed()
