"""Flagship benchmark: end-to-end tensor-parallel decode throughput of a Qwen3-32B-shaped dense model.

Workload (fixed, strong scaling over N): batch 8, prompt 2048 uniform-random token ids, random-init bf16 weights.
The prompt is prefilled with AG-GEMM + GEMM-RS on sequence-sharded activations (``triton_dist`` mode, N >= 2) and the
native prefill attention; decode runs through ``Engine`` in ``triton_dist_AR`` mode (native decode GEMMs, fused
all-reduce + residual + RMSNorm, paged decode attention, CUDA graph, top-p sampling). ``--steps`` decode steps are
timed after ``--warmup`` untimed ones. Rank 0 prints ONE JSON line.

  value        decode tokens/s of the whole job, device-timed with CUDA events (max over ranks)
  e2e.value    the same through the public ``Engine.decode_one`` API with, every step, the host->device copy of the
               input token ids from pinned memory and the device->host read of the sampled ids
  torch_mode   the same decode loop with the model in ``torch`` mode: cuBLAS + NCCL all-reduce + flashinfer RMSNorm /
               RoPE + flash-attn (the library composition the reference uses as golden and baseline), CUDA graph
  kernels      (N >= 2) the fused compute + collective kernels of the headline metric on their named shapes, each next to
               its NCCL (+ cuBLAS) composition, measured after the decode loops

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N``.
"""
from __future__ import annotations

import argparse
import atexit
import gc
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

    def wait_first_sample(self, timeout_s: float) -> None:
        """Block until nvidia-smi has printed its first line (its initialisation is over) or `timeout_s` has passed."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout_s:
            time.sleep(0.02)

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


def emit_result(out: dict, heap, rank: int) -> None:
    """Print the JSON line, but only if no kernel of this rank recorded an expired wait: a bounded wait that ran out
    makes its kernel return early with incomplete data, so a number measured after that is not a measurement.
    Raises ``SymmTimeoutError`` (non-zero exit) instead of printing."""
    if heap is not None:
        heap.check_status("bench.py timed region")
    if rank == 0:
        print(json.dumps(out), flush=True)


def _teardown(engines) -> None:
    """Orderly shutdown: captured graphs (which hold NCCL kernels) go first, then the heap, then the process group.
    Should a collective teardown stall, a watchdog runs the interpreter's exit hooks and ends the process, so a
    finished measurement is never held hostage by a peer that is already gone."""
    import torch

    from triton_distributed_b200 import utils

    def last_resort():
        sys.stderr.write("bench.py: teardown stalled for 90 s; exiting without it\n")
        sys.stderr.flush()
        try:
            atexit._run_exitfuncs()
        finally:
            os._exit(0)

    watchdog = threading.Timer(90.0, last_resort)
    watchdog.daemon = True
    watchdog.start()
    try:
        for e in engines:
            if e is not None and getattr(e, "graph", None) is not None:
                e.graph.reset()
                e.graph = None
        gc.collect()
        torch.cuda.synchronize()
        utils.finalize_distributed()
    finally:
        watchdog.cancel()


def _kernel_extras(args, group, world: int, budget_s: float = 120.0) -> dict:
    """The fused kernels of the headline metric on their named shapes next to their NCCL (+ cuBLAS) compositions:
    AG-GEMM and GEMM-RS (Llama-3-70B MLP, M = 8192), EP dispatch + combine (128 tokens per rank, hidden 7168, fp8),
    the all-reduce (+ residual + RMSNorm) at a few sizes, SP flash-decode and the TP-MoE pair. Microseconds, device
    timed, L2 flushed per call, min over iterations, max over ranks. A failing row is reported, not fatal."""
    import types

    import torch

    from triton_distributed_b200 import utils
    from triton_distributed_b200.benchmark import bench_collectives as bc
    from triton_distributed_b200.benchmark import bench_comm_gemm as bg

    heap = utils.get_heap()
    heap.set_timeout_ms(3000)  # a lost signal in one of these rows costs seconds, not the default ten per wait
    out: dict = {}
    t_start = time.time()
    a = types.SimpleNamespace(iters=args.kernel_iters, warmup=3, ar_max_bytes=args.ar_max_bytes, ep_tokens=128,
                              moe_tokens=8192, sp_batches=(1, 8), sp_kv=(128 << 10, 1 << 20),
                              ar_tokens=(8, 2048))
    steps = [("comm_gemm", lambda rows: bg.bench_pair(group, 8192, a.iters, a.warmup, rows)),
             ("ep_a2a", lambda rows: bc.bench_ep_a2a(a, group, rows)),
             ("allreduce", lambda rows: bc.bench_allreduce(a, group, rows)),
             ("sp_decode", lambda rows: bc.bench_sp_decode(a, group, rows)),
             ("tp_moe", lambda rows: bc.bench_tp_moe(a, group, rows))]
    for name, fn in steps:
        if name in args.skip_kernels:
            continue
        over = torch.tensor([1.0 if time.time() - t_start > budget_s else 0.0], device="cuda")
        torch.distributed.all_reduce(over, group=group)  # every rank takes the same decision
        if over.item() > 0:
            out[name] = {"skipped": "time budget"}
            continue
        rows: list = []
        try:
            fn(rows)
            torch.cuda.synchronize()
            heap.check_status(name)
            out[name] = rows
        except Exception as e:  # noqa: BLE001
            out[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}", "rows": rows}
            break  # the ranks may no longer agree on what comes next
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", default="Qwen/Qwen3-32B")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--no-baseline", action="store_true", help="skip the torch-mode (library composition) measurement")
    ap.add_argument("--prefill-backend", default="auto", choices=["auto", "torch", "triton_dist", "triton_dist_AR"],
                    help="auto: triton_dist (AG-GEMM + GEMM-RS) when N >= 2 and the batch divides, else triton_dist_AR")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel measurements at N >= 2")
    ap.add_argument("--skip-kernels", nargs="*", default=[], help="names of per-kernel groups to leave out")
    ap.add_argument("--kernel-iters", type=int, default=8)
    ap.add_argument("--ar-max-bytes", type=int, default=64 << 20)
    ap.add_argument("--settle-steps", type=int, default=24,
                    help="untimed decode steps right after graph capture (clocks, link state), before any timed phase")
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
    from triton_distributed_b200.layers.nvidia import golden
    from triton_distributed_b200.models import Engine, ModelConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1 (see the module docstring)")
        args.gpus = world
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("LOCAL_RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"), os.environ.setdefault("MASTER_PORT", "29541")
    group = utils.initialize_distributed(seed=0, heap_bytes=(3 << 30) if world == 1 else (8 << 30))
    heap = utils.get_heap()
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    # every timed phase restarts from the end of the prompt, so the cache holds the longest single phase
    max_len = (args.prompt + max(args.settle_steps, args.steps + args.warmup) + 16 + 255) // 256 * 256
    cfg = ModelConfig(model_name=args.model, max_length=max_len, dtype=torch.bfloat16, rank=rank, world_size=world, seed=0)
    eng = Engine(cfg, temperature=0.6, top_p=0.95, group=group)
    eng.backend = "triton_dist_AR"
    prefill_backend = args.prefill_backend
    if prefill_backend == "auto":
        prefill_backend = "triton_dist" if world > 1 and args.batch % world == 0 else "triton_dist_AR"
    eng.prefill_backend = prefill_backend
    torch.manual_seed(1234)  # same prompt and sampling stream on every rank
    arch = eng.model.arch
    prompt = torch.randint(0, arch.vocab_size, (args.batch, args.prompt), device=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()

    # ---------------- prefill (not part of the timed decode metric; reported separately, cold and warm) ----------------
    prefill_ms = []
    for _ in range(2):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        first = eng.prefill(prompt)
        e1.record()
        torch.cuda.synchronize()
        prefill_ms.append(utils.max_over_ranks(e0.elapsed_time(e1), group))
    heap.check_status("prefill")
    before = ops.launch_count
    eng.prepare_decode(first)
    launches_per_step = (ops.launch_count - before) // 4  # 3 warm-up steps + 1 captured step
    kv_after_prefill = eng.kv_cache.kv_offset.clone()
    for _ in range(args.settle_steps):
        eng.decode_one()
    sync_all()

    def timed_decode(e2e: bool):
        """Returns (ms per step, clocks, per-step stats). Tokens stay on the device unless e2e."""
        pinned_in = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
        pinned_out = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
        pinned_in.copy_(first.cpu())
        eng.kv_cache.kv_offset.copy_(kv_after_prefill)
        # the sampler starts BEFORE the warm-up steps: nvidia-smi's start-up (driver queries from one process per rank at
        # once) stalls kernel launches for tens of milliseconds, which must not land inside the timed steps
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        sampler.wait_first_sample(3.0)
        for _ in range(args.warmup):
            eng.decode_one()
        sync_all()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        marks[0].record()
        for i in range(args.steps):
            if e2e:
                tok = pinned_in.to(dev, non_blocking=True)
                nxt = eng.decode_one(tok)
                pinned_out.copy_(nxt, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                pinned_in.copy_(pinned_out)
            else:
                eng.decode_one()
            marks[i + 1].record()
        sync_all()
        clocks = sampler.stop()
        per = [marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps)]
        ms = utils.max_over_ranks(marks[0].elapsed_time(marks[-1]) / args.steps, group)
        stats = {"step_ms_min": utils.max_over_ranks(min(per), group),
                 "step_ms_median": utils.max_over_ranks(statistics.median(per), group),
                 "step_ms_max": utils.max_over_ranks(max(per), group)}
        return ms, clocks, stats

    ms, clocks, stats = timed_decode(False)
    ms_e2e, _, stats_e2e = timed_decode(True)
    heap.check_status("decode")
    toks = args.batch / (ms * 1e-3)
    out = {
        "metric": "e2e decode tok/s, Qwen3-32B TP=N, batch 8, prompt 2048", "value": toks, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random token ids, random-init weights)",
        "impl": "ours",
        "config": {"model": args.model, "global_batch": args.batch, "seq_len": args.prompt, "parallelism": f"tp{world}",
                   "decode_backend": eng.backend, "prefill_backend": prefill_backend, "cuda_graph": not eng.no_graph,
                   "sampling": "top-p 0.95, temperature 0.6", "l2": "per-step inputs (weight shards + KV cache) exceed the 126 MB L2",
                   "heap_mode": heap.mode, "nvls": heap.has_multicast, "settle_steps": args.settle_steps},
        "clocks": clocks,
        "e2e": {"value": args.batch / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": args.batch * 8, **stats_e2e},
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_per_step": launches_per_step,
        "prefill_ms": prefill_ms[1], "prefill_cold_ms": prefill_ms[0],
        **stats,
    }
    engines = [eng]
    if not args.no_baseline:
        ref = Engine(cfg, temperature=0.6, top_p=0.95, group=group, model=eng.model)
        ref.backend = "torch"
        ref.kv_cache, ref.bsz = eng.kv_cache, args.batch
        ref.kv_cache.kv_offset.copy_(kv_after_prefill)
        ref.prepare_decode(first)
        engines.append(ref)
        eng_saved, eng = eng, ref  # timed_decode closes over `eng`
        try:
            for _ in range(args.settle_steps):
                eng.decode_one()
            ms_t, _, stats_t = timed_decode(False)
            out["torch_mode"] = {"value": args.batch / (ms_t * 1e-3), "unit": "tokens/s", "ms_per_step": ms_t, **stats_t,
                                 "what": "same engine and CUDA graph on cuBLAS + NCCL all_reduce + the libraries below",
                                 "libraries": golden.describe()}
            out["speedup_vs_torch_mode"] = ms_t / ms
        finally:
            eng = eng_saved
    if world > 1 and not args.no_kernels:
        for e in engines:  # free the decode graphs' NCCL work before the kernels' own collectives
            if e.graph is not None:
                e.graph.reset()
                e.graph = None
        out["kernels"] = _kernel_extras(args, group, world)
    emit_result(out, heap, rank)
    sys.stdout.flush()
    _teardown(engines)


if __name__ == "__main__":
    main()
