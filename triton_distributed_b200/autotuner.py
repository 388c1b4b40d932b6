"""Contextual autotuner: tune a whole thunk (several kernels, side effects, collectives) instead of one kernel.

API parity with ``python/triton_dist/autotuner.py:33-256`` (``contextual_autotune(is_dist=...)`` decorator). The
reference hooks Triton's per-kernel autotuner and interleaves one benchmark step per invocation; here the tunables
are explicit: the decorated function receives ``config=`` chosen from ``configs``; every candidate is timed with CUDA
events for ``iters`` calls, timings are all-reduced with MAX over ranks so that every rank picks the same winner, and
the choice is cached per key (and optionally persisted as JSON).
"""
from __future__ import annotations

import functools
import json
import os
from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist

_LOG_DIR = ".autotune_logs"


def _log(msg: str) -> None:
    os.makedirs(_LOG_DIR, exist_ok=True)
    rank = dist.get_rank() if dist.is_initialized() else 0
    with open(os.path.join(_LOG_DIR, f"rank-{rank}.log"), "a") as f:
        f.write(msg + "\n")


def contextual_autotune(configs: Sequence[Any], key: Callable[..., Any] | None = None, is_dist: bool = False,
                        iters: int = 5, warmup: int = 2, cache_file: str | None = None):
    """Decorate ``fn(*args, config=..., **kw)``. The first call per key times every config and keeps the fastest."""
    def deco(fn):
        cache: dict[str, int] = {}
        if cache_file and os.path.exists(cache_file):
            with open(cache_file) as f:
                cache.update(json.load(f))

        @functools.wraps(fn)
        def wrapped(*args, **kw):
            k = repr(key(*args, **kw)) if key else "default"
            if k not in cache:
                times = []
                for cfg in configs:
                    for _ in range(warmup):
                        fn(*args, config=cfg, **kw)
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(iters):
                        fn(*args, config=cfg, **kw)
                    b.record()
                    b.synchronize()
                    times.append(a.elapsed_time(b) / iters)
                t = torch.tensor(times, dtype=torch.float64, device="cuda")
                if is_dist and dist.is_initialized() and dist.get_world_size() > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                best = int(torch.argmin(t).item())
                cache[k] = best
                _log(f"{fn.__name__} key={k} times_ms={[round(x, 4) for x in t.tolist()]} best={configs[best]!r}")
                if cache_file and (not dist.is_initialized() or dist.get_rank() == 0):
                    with open(cache_file, "w") as f:
                        json.dump(cache, f)
            return fn(*args, config=configs[cache[k]], **kw)

        wrapped.cache = cache
        return wrapped
    return deco
