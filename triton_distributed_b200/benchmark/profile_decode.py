"""Per-kernel device time of one decode step of Qwen3-32B (or its first N layers), from torch.profiler over CUDA-graph
replays of ``Engine.decode_one()``. Rank 0 prints and writes a table ``us/step, calls/step, us/call, kernel``.

Run (1 GPU):  ``python -m triton_distributed_b200.benchmark.profile_decode --layers 8``
Run (N GPUs): ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m triton_distributed_b200.benchmark.profile_decode``
Role in the reference: the 64-step decode trace of ``python/triton_dist/models/engine.py:151-177``.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .. import utils
from ..models import Engine, ModelConfig


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=8, help="number of transformer layers to build (64 = the full model)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--out", default=None, help="text file for the table (rank 0)")
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29547")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=1 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = ModelConfig(model_name="Qwen/Qwen3-32B", max_length=args.prompt + 512, rank=rank, world_size=world,
                      num_layers_override=args.layers)
    eng = Engine(cfg, temperature=0.6, top_p=0.95, group=group)
    prompt = torch.randint(0, 151936, (args.batch, args.prompt), device="cuda")
    eng.prepare_decode(eng.prefill(prompt))
    for _ in range(4):
        eng.decode_one()
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(args.steps):
            eng.decode_one()
        torch.cuda.synchronize()
    if rank == 0:
        rows = []
        for e in prof.key_averages():
            t = getattr(e, "device_time_total", 0) or getattr(e, "cuda_time_total", 0)
            if t > 0 and e.device_type.name == "CUDA":
                rows.append((t / args.steps, e.count / args.steps, e.key[:90]))
        rows.sort(reverse=True)
        lines = [f"world={world} layers={args.layers}: total kernel us/step {sum(r[0] for r in rows):.1f}"]
        lines += [f"{t:10.1f} us/step  {c:7.1f} calls/step  {t / max(c, 1e-9):8.2f} us/call  {k}" for t, c, k in rows[:25]]
        print("\n".join(lines), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write("\n".join(lines) + "\n")
    os._exit(0)  # CUDA graphs that captured collectives do not survive an orderly process-group teardown


if __name__ == "__main__":
    main()
