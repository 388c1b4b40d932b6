"""Launches the multi-rank GPU cases (tests/dist_cases.py) under torchrun when >= 2 GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc: int, script: str, args=(), timeout=900, env_extra=None):
    port = 29700 + os.getpid() % 200
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script), *args]
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_multi_rank_cases():
    n = min(torch.cuda.device_count(), 8)
    n = 1 << (n.bit_length() - 1)
    res = _run(n, "dist_cases.py")
    sys.stdout.write(res.stdout[-6000:])
    sys.stderr.write(res.stderr[-3000:])
    assert res.returncode == 0, "multi-rank cases failed (see output)"
    assert "FAIL" not in res.stdout
