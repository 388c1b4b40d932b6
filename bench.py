"""Flagship benchmark: end-to-end tensor-parallel decode throughput of a Qwen3-32B-shaped dense model.

Workload (fixed, strong scaling over N): batch 8, prompt 2048 uniform-random token ids, random-init bf16
weights, then decode steps through ``Engine`` (native GEMMs, fused AllReduce + residual + RMSNorm, paged
decode attention, CUDA graph, top-p sampling). ``--steps`` decode steps are timed after ``--warmup`` untimed
ones. Rank 0 prints ONE JSON line.

  value        decode tokens/s of the whole job, device-timed with CUDA events (max over ranks)
  e2e.value    the same through the public ``Engine.decode_one`` API with, every step, the host->device copy
               of the input token ids from pinned memory and the device->host read of the sampled ids
  torch_mode   the same decode loop with the model in ``torch`` mode (cuBLAS + NCCL all-reduce, torch
               norms/rope/attention, CUDA graph): the reference's own golden/baseline composition

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _reference_arm() -> None:
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference cannot be installed offline: its root has no installable package and python/setup.py "
                      "builds the empty 3rdparty/triton submodule and downloads LLVM (no network); nvshmem4py is absent"}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", default="Qwen/Qwen3-32B")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--no-baseline", action="store_true", help="skip the torch-mode (cuBLAS + NCCL) measurement")
    ap.add_argument("--prefill-backend", default="triton_dist_AR", choices=["torch", "triton_dist", "triton_dist_AR"])
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:  # one line per job, also when launched as N ranks
            _reference_arm()
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from triton_distributed_b200 import ops, utils
    from triton_distributed_b200.models import Engine, ModelConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1 (see the module docstring)")
        args.gpus = world
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("LOCAL_RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"), os.environ.setdefault("MASTER_PORT", "29541")
    group = utils.initialize_distributed(seed=0, heap_bytes=3 << 30)
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    max_len = args.prompt + args.steps * 2 + args.warmup * 2 + 64
    max_len = (max_len + 255) // 256 * 256
    cfg = ModelConfig(model_name=args.model, max_length=max_len, dtype=torch.bfloat16, rank=rank, world_size=world, seed=0)
    eng = Engine(cfg, temperature=0.6, top_p=0.95, group=group)
    eng.backend = "triton_dist_AR"
    eng.prefill_backend = args.prefill_backend
    torch.manual_seed(1234)  # same prompt and sampling stream on every rank
    arch = eng.model.arch
    prompt = torch.randint(0, arch.vocab_size, (args.batch, args.prompt), device=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()

    # ---------------- prefill (untimed part of the workload, reported separately) ----------------
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    first = eng.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = utils.max_over_ranks(e0.elapsed_time(e1), group)
    before = ops.launch_count
    eng.prepare_decode(first)
    launches_per_step = (ops.launch_count - before) // 4  # 3 warm-up steps + 1 captured step
    kv_after_prefill = eng.kv_cache.kv_offset.clone()

    def timed_decode(e2e: bool):
        """Returns (ms per step, clocks). Tokens stay on the device unless e2e."""
        pinned_in = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
        pinned_out = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
        pinned_in.copy_(first.cpu())
        eng.kv_cache.kv_offset.copy_(kv_after_prefill)
        for _ in range(args.warmup):
            eng.decode_one()
        sync_all()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            if e2e:
                tok = pinned_in.to(dev, non_blocking=True)
                nxt = eng.decode_one(tok)
                pinned_out.copy_(nxt, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                pinned_in.copy_(pinned_out)
            else:
                eng.decode_one()
        b.record()
        sync_all()
        clocks = sampler.stop()
        return utils.max_over_ranks(a.elapsed_time(b) / args.steps, group), clocks

    ms, clocks = timed_decode(False)
    ms_e2e, _ = timed_decode(True)
    toks = args.batch / (ms * 1e-3)
    out = {
        "metric": "e2e decode tok/s, Qwen3-32B TP=N, batch 8, prompt 2048", "value": toks, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random token ids, random-init weights)",
        "impl": "ours",
        "config": {"model": args.model, "global_batch": args.batch, "seq_len": args.prompt, "parallelism": f"tp{world}",
                   "decode_backend": eng.backend, "prefill_backend": args.prefill_backend, "cuda_graph": not eng.no_graph,
                   "sampling": "top-p 0.95, temperature 0.6", "l2": "per-step inputs (weight shards + KV cache) exceed the 126 MB L2",
                   "heap_mode": utils.get_heap().mode, "nvls": utils.get_heap().has_multicast},
        "clocks": clocks,
        "e2e": {"value": args.batch / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": args.batch * 8},
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_per_step": launches_per_step,
        "prefill_ms": prefill_ms,
    }
    if not args.no_baseline:
        ref = Engine(cfg, temperature=0.6, top_p=0.95, group=group, model=eng.model)
        ref.backend = "torch"
        ref.kv_cache, ref.bsz = eng.kv_cache, args.batch
        ref.kv_cache.kv_offset.copy_(kv_after_prefill)
        ref.prepare_decode(first)
        eng_saved, eng_ref = eng, ref
        eng = ref  # timed_decode closes over `eng`
        try:
            ms_t, _ = timed_decode(False)
            out["torch_mode"] = {"value": args.batch / (ms_t * 1e-3), "unit": "tokens/s", "ms_per_step": ms_t,
                                 "what": "same engine and CUDA graph with cuBLAS + NCCL all_reduce + torch ops"}
            out["speedup_vs_torch_mode"] = ms_t / ms
        finally:
            eng = eng_saved
    if rank == 0:
        print(json.dumps(out), flush=True)
    # Teardown must never outlive the measurement: CUDA graphs that captured NCCL kernels are dropped before the
    # communicator, and a watchdog ends the process if a collective teardown stalls.
    sys.stdout.flush()
    watchdog = threading.Timer(30.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    try:
        for e in (eng, locals().get("eng_ref"), locals().get("eng_saved")):
            if e is not None:
                e.graph = None
        import gc
        gc.collect()
        torch.cuda.synchronize()
        utils.finalize_distributed()
    finally:
        watchdog.cancel()
    os._exit(0)


if __name__ == "__main__":
    main()
