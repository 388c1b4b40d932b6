"""Reference-semantics plumbing on CPU: world_size=2 over gloo, fp32, seed 0. Each output is checked against
torch.distributed collectives composed with plain matmuls."""
import multiprocessing as mp
import os
import random

import pytest

from _gloo_cases import CASES, worker


def _run(name: str, world: int = 2, timeout: int = 120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = random.randint(20000, 40000)
    procs = [ctx.Process(target=worker, args=(r, world, port, name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=timeout) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    errs = [f"rank {r}:\n{e}" for r, e in results if e]
    assert not errs, "\n".join(errs)


@pytest.mark.parametrize("name", [n for n in CASES])
def test_gloo_case(name):
    _run(name)
