"""Host runtime helpers: distributed bring-up, symmetric tensors, timing, printing, comparison,
profiling and capability probes.

API parity with ``python/triton_dist/utils.py`` of the reference (names and call signatures are kept
so that scripts written against it run unchanged): ``initialize_distributed`` (:174), ``TP_GROUP``
(:197), ``nvshmem_create_tensor(s)`` (:122-144), ``nvshmem_free_tensor_sync`` (:147),
``nvshmem_barrier_all_on_stream`` (:169), ``finalize_distributed`` (:153), ``perf_func`` (:269),
``dist_print`` (:284), ``assert_allclose`` (:865), ``generate_data`` (:252), ``group_profile`` (:500),
``sleep_async`` (:1010) and the capability probes (:704-1000). NVSHMEM is replaced by the CUDA VMM
symmetric heap of :mod:`triton_distributed_b200.runtime.heap`; the ``nvshmem_*`` names are aliases.
"""
from __future__ import annotations

import contextlib
import datetime
import functools
import json
import os
import random
import tarfile
from pathlib import Path
from typing import Callable, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .runtime.heap import (SymmHeap, SymmHeapError, SymmTimeoutError, finalize_symm_heap, get_heap,
                           heap_initialized, init_symm_heap)

__all__ = [
    "initialize_distributed", "finalize_distributed", "TP_GROUP", "init_seed", "init_symm_heap_by_torch_process_group",
    "init_nvshmem_by_torch_process_group", "symm_create_tensor", "symm_create_tensors", "symm_free_tensor_sync",
    "symm_barrier_all_on_stream", "nvshmem_create_tensor", "nvshmem_create_tensors", "nvshmem_free_tensor_sync",
    "nvshmem_barrier_all_on_stream", "NVSHMEM_SIGNAL_DTYPE", "SIGNAL_DTYPE", "perf_func", "dist_print",
    "assert_allclose", "generate_data", "group_profile", "get_torch_prof_ctx", "sleep_async",
    "is_nvshmem_multimem_supported", "is_multimem_supported", "get_has_fullmesh_nvlink", "get_intranode_max_speed",
    "get_nvlink_max_speed", "check_p2p_native_atomic_supported", "get_device_max_shared_memory_size", "is_tma_support",
    "get_numa_world_size", "requires", "SymmHeap", "SymmHeapError", "SymmTimeoutError", "get_heap",
]

_TP_GROUP = None
# Flags of this library are 32-bit epochs; the reference's NVSHMEM signals are int64.
SIGNAL_DTYPE = torch.int32
NVSHMEM_SIGNAL_DTYPE = SIGNAL_DTYPE


# ------------------------------------------------------------------------------------------------
# bring-up / teardown
# ------------------------------------------------------------------------------------------------
def init_seed(seed: int = 0) -> None:
    """Seed every RNG and select deterministic, TF32-free math (reference: utils.py:75-94)."""
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    np.random.seed(seed)
    random.seed(seed)


def init_symm_heap_by_torch_process_group(pg=None, size_bytes: int | None = None) -> SymmHeap:
    return init_symm_heap(pg, size_bytes)


init_nvshmem_by_torch_process_group = init_symm_heap_by_torch_process_group


def initialize_distributed(seed: int | None = None, heap_bytes: int | None = None, backend: str | None = None):
    """One process per GPU: bind the device, create the NCCL process group (gloo without CUDA), the
    all-ranks TP group, seed the RNGs and build the symmetric heap. Returns the TP group."""
    global _TP_GROUP
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kw = {}
        if cuda and backend in (None, "nccl"):
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend or ("nccl" if cuda else "gloo"), world_size=world, rank=rank,
                                timeout=datetime.timedelta(seconds=int(os.environ.get("B200DIST_PG_TIMEOUT_S", 1800))),
                                **kw)
    _TP_GROUP = dist.new_group(ranks=list(range(world)), backend=backend or ("nccl" if cuda else "gloo"))
    init_seed(rank if seed is None else seed)
    if cuda:
        dist.barrier(group=_TP_GROUP)
        init_symm_heap(_TP_GROUP, heap_bytes)
    return _TP_GROUP


def TP_GROUP():
    return _TP_GROUP


def finalize_distributed() -> None:
    finalize_symm_heap()
    if dist.is_initialized():
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# symmetric tensors
# ------------------------------------------------------------------------------------------------
def symm_create_tensor(shape: Sequence[int] | int, dtype: torch.dtype) -> torch.Tensor:
    """Zero-filled tensor at the same heap offset on every rank (call it collectively, same order)."""
    return get_heap().create_tensor(shape, dtype)


def symm_create_tensors(shape, dtype, rank: int | None = None, local_world_size: int | None = None) -> list[torch.Tensor]:
    """Like the reference's ``nvshmem_create_tensors``: one symmetric allocation, returned as the list
    of every rank's view of it (entry ``rank`` is the local tensor, the others are peer mappings)."""
    return get_heap().create_tensors(shape, dtype)


def symm_free_tensor_sync(t: torch.Tensor) -> None:
    torch.cuda.synchronize()
    get_heap().free(t)


def symm_barrier_all_on_stream(stream: torch.cuda.Stream | None = None) -> None:
    get_heap().barrier_all(stream)


nvshmem_create_tensor = symm_create_tensor
nvshmem_create_tensors = symm_create_tensors
nvshmem_free_tensor_sync = symm_free_tensor_sync
nvshmem_barrier_all_on_stream = symm_barrier_all_on_stream


# ------------------------------------------------------------------------------------------------
# timing / data / printing / comparison
# ------------------------------------------------------------------------------------------------
def perf_func(func: Callable, iters: int, warmup_iters: int):
    """CUDA-event timing on the current stream: returns (last output, mean milliseconds per call)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = None
    for n in range(iters + warmup_iters):
        if n == warmup_iters:
            start.record()
        out = func()
    stop.record()
    start.wait()
    stop.wait()
    torch.cuda.current_stream().synchronize()
    return out, start.elapsed_time(stop) / max(iters, 1)


_l2_flush_buf: torch.Tensor | None = None


def flush_l2() -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    global _l2_flush_buf
    if _l2_flush_buf is None:
        _l2_flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _l2_flush_buf.zero_()


def perf_func_cold(func: Callable, iters: int, warmup_iters: int, head_start_us: float = 500.0):
    """Like perf_func but with an L2 flush before every timed call; each call is timed separately.
    Returns (last output, mean ms, list of per-call ms).

    The device spins for `head_start_us` before the first event, so the host has enqueued the call by the time the
    device reaches it: the interval then holds device time only, not the host's launch latency (which otherwise
    puts a floor of tens of microseconds under every small kernel)."""
    out = None
    for _ in range(warmup_iters):
        out = func()
    times = []
    spin = int(head_start_us * 1.9e3)  # cycles at the boost clock; the exact length does not matter
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if spin > 0:
            torch.cuda._sleep(spin)
        a.record()
        out = func()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return out, float(np.mean(times)) if times else 0.0, times


def max_over_ranks(value: float, group=None) -> float:
    """Device-timed numbers are reported as the maximum over ranks."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def _make_tensor(shape, dtype, init_args, device="cuda"):
    if isinstance(init_args, (int, float)):
        return torch.full(shape, init_args, dtype=dtype, device=device)
    if isinstance(init_args, (tuple, list)) and len(init_args) == 2:
        scale, bias = init_args
        if dtype in (torch.float16, torch.bfloat16, torch.float32):
            return (torch.rand(shape, dtype=dtype, device=device) * 2 - 1) * scale + bias
        if dtype == torch.int8:
            return torch.randint(-127, 128, shape, dtype=torch.int8, device=device)
        return ((torch.rand(shape, dtype=torch.float32, device=device) * 2 - 1) * scale + bias).to(dtype)
    raise ValueError(f"unsupported init_args {init_args!r}")


def generate_data(configs):
    """Infinite generator of tensor lists; each config is (shape, dtype, (scale, bias) | constant)."""
    while True:
        yield [_make_tensor(*c) if c is not None else None for c in configs]


def dist_print(*args, allowed_ranks: Sequence[int] | str = (0,), prefix: bool = False, need_sync: bool = False, **kw):
    """print() filtered by rank; with need_sync the ranks print in order separated by barriers."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    if allowed_ranks == "all":
        allowed_ranks = list(range(world))
    for r in range(world) if need_sync else [rank]:
        if need_sync and world > 1:
            dist.barrier()
        if r == rank and rank in allowed_ranks:
            if prefix:
                print(f"[rank:{rank}]", *args, **kw)
            else:
                print(*args, **kw)


def assert_allclose(x: torch.Tensor, y: torch.Tensor, rtol: float, atol: float, verbose: bool = True) -> None:
    """torch.allclose with a readable report of the worst mismatches (raises RuntimeError)."""
    if x.shape != y.shape:
        raise RuntimeError(f"shape mismatch {tuple(x.shape)} vs {tuple(y.shape)}")
    xf, yf = x.detach().float(), y.detach().float()
    bad = ~torch.isclose(xf, yf, rtol=rtol, atol=atol)
    nbad = int(bad.sum().item())
    if nbad == 0:
        if verbose:
            print("✅ all close!")
        return
    diff = (xf - yf).abs()
    idx = torch.nonzero(bad)[:8]
    lines = [f"❌ {nbad}/{x.numel()} mismatches (rtol={rtol}, atol={atol}), max abs diff {diff.max().item():.5g}"]
    for i in idx:
        t = tuple(int(v) for v in i)
        lines.append(f"  at {t}: {xf[t].item():.6g} vs {yf[t].item():.6g}")
    raise RuntimeError("\n".join(lines))


_sleep_buf = None


def sleep_async(duration_ms: int) -> None:
    """Keep the current stream busy for about `duration_ms` without blocking the host (used to create
    stragglers in correctness tests, reference: utils.py:1010)."""
    torch.cuda._sleep(int(duration_ms * 1.5e6))


# ------------------------------------------------------------------------------------------------
# profiling: per-rank torch.profiler traces merged into one chrome trace on rank 0
# ------------------------------------------------------------------------------------------------
def get_torch_prof_ctx(do_prof: bool):
    if not do_prof:
        return contextlib.nullcontext()
    return torch.profiler.profile(
        activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA], record_shapes=True)


def _remap_trace(trace: dict, rank: int) -> list[dict]:
    """Shift pids/tids into a per-rank range and tag names so that ranks do not collide when merged."""
    off = rank * 100_000_000
    out = []
    for ev in trace.get("traceEvents", []):
        ev = dict(ev)
        for key in ("pid", "tid"):
            if isinstance(ev.get(key), int):
                ev[key] = ev[key] + off
            elif key in ev:
                ev[key] = f"{ev[key]}_rank{rank}"
        if ev.get("ph") == "M" and isinstance(ev.get("args"), dict) and "name" in ev["args"]:
            ev["args"] = dict(ev["args"], name=f"{ev['args']['name']}_rank{rank}")
        out.append(ev)
    return out


def merge_traces(traces: list[dict]) -> dict:
    merged = {"traceEvents": []}
    for rank, tr in enumerate(traces):
        merged["traceEvents"].extend(_remap_trace(tr, rank))
    for k, v in traces[0].items():
        if k != "traceEvents":
            merged[k] = v
    return merged


@contextlib.contextmanager
def group_profile(name: str | None = None, do_prof: bool = True, merge_group: bool = True,
                  keep_merged_only: bool = True, compress: bool = True, group=None):
    """Profile the enclosed region on every rank and write ``prof/<name>_merged.json(.tar.gz)`` on rank 0."""
    if not do_prof:
        yield None
        return
    prof = get_torch_prof_ctx(True)
    with prof:
        yield prof
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    out_dir = Path("prof")
    out_dir.mkdir(exist_ok=True)
    mine = out_dir / f"{name or 'trace'}_rank{rank}.json"
    prof.export_chrome_trace(str(mine))
    if not merge_group:
        return
    with open(mine) as f:
        trace = json.load(f)
    gathered = [None] * world if rank == 0 else None
    if world > 1:
        dist.gather_object(trace, gathered, dst=dist.get_global_rank(group, 0) if group else 0, group=group)
    else:
        gathered = [trace]
    if rank == 0:
        merged_path = out_dir / f"{name or 'trace'}_merged.json"
        with open(merged_path, "w") as f:
            json.dump(merge_traces(gathered), f)
        if compress:
            with tarfile.open(str(merged_path) + ".tar.gz", "w:gz") as tar:
                tar.add(merged_path, arcname=merged_path.name)
            merged_path.unlink()
    if keep_merged_only:
        mine.unlink(missing_ok=True)


# ------------------------------------------------------------------------------------------------
# capability probes
# ------------------------------------------------------------------------------------------------
def is_multimem_supported() -> bool:
    """True when the symmetric heap is bound to an NVLS multicast object (multimem.* usable)."""
    return heap_initialized() and get_heap().has_multicast


is_nvshmem_multimem_supported = is_multimem_supported


@functools.lru_cache()
def get_has_fullmesh_nvlink() -> bool:
    """Every pair of visible GPUs can reach each other peer-to-peer (true behind an NVSwitch)."""
    n = torch.cuda.device_count()
    return all(torch.cuda.can_device_access_peer(i, j) for i in range(n) for j in range(n) if i != j)


def get_nvlink_max_speed(gpu_index: int = 0) -> float:
    """Per-direction NVLink bandwidth of one GPU in GB/s summed over active links (0 when unknown)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        total = 0.0
        for link in range(18):
            try:
                if pynvml.nvmlDeviceGetNvLinkState(h, link):
                    total += 50.0  # NVLink 5: 50 GB/s per direction per link
            except pynvml.NVMLError:
                break
        return total
    except Exception:
        return 0.0


def get_intranode_max_speed() -> float:
    """GB/s per direction between two GPUs of the node: NVLink if present, else a PCIe 5 x16 figure."""
    v = get_nvlink_max_speed()
    return v if v > 0 else 64.0


def get_numa_world_size() -> int:
    return torch.cuda.device_count()


def check_p2p_native_atomic_supported() -> bool:
    if torch.cuda.device_count() < 2:
        return True
    try:
        from cuda.bindings import runtime as rt
        err, v = rt.cudaDeviceGetP2PAttribute(rt.cudaDeviceP2PAttr.cudaDevP2PAttrNativeAtomicSupported, 0, 1)
        return bool(v)
    except Exception:
        return get_has_fullmesh_nvlink()


def get_device_max_shared_memory_size(device: int = 0) -> int:
    return torch.cuda.get_device_properties(device).shared_memory_per_block_optin


def is_tma_support() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 9


def requires(check: Callable[[], bool], reason: str = ""):
    """Decorator: the wrapped function raises unless `check()` holds (reference: utils.py:991)."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            if not check():
                raise RuntimeError(f"{fn.__name__} is not supported here: {reason or check.__name__}")
            return fn(*a, **k)
        return wrapped
    return deco
