"""The tutorials run as written (one rank, small shapes): each one checks its own result and exits non-zero on a mismatch."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,args", [
    ("01_notify_wait.py", []),
    ("02_overlapping_allgather_gemm.py", ["--m", "1024", "--n", "2048", "--k", "1024"]),
    ("03_overlapping_gemm_reduce_scatter.py", ["--m", "1024", "--n", "1024", "--k", "2048"]),
    ("04_ep_all2all_fp8.py", []),
    ("05_allgather.py", []),
    ("06_reduce_scatter.py", []),
])
def test_tutorial_runs(script, args):
    env = dict(os.environ)
    env.update({"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                "MASTER_PORT": str(29800 + os.getpid() % 100)})
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tutorials", script), *args], capture_output=True, text=True,
                         timeout=600, env=env, cwd=ROOT)
    sys.stdout.write(res.stdout[-2000:])
    sys.stderr.write(res.stderr[-2000:])
    assert res.returncode == 0 and "tutorial" in res.stdout
