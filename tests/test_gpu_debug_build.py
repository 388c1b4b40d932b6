"""The checking build (``python -m triton_distributed_b200.build --debug``): bounds-checked symmetric address
translation and random delays in front of every notify / wait / barrier. Runs in child processes, because the library
variant is chosen when the package is first imported (``B200DIST_DEBUG_LIB=1``)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG_LIB = os.path.join(ROOT, "triton_distributed_b200", "lib", "libb200dist_debug.so")

_BAD_POINTER = r"""
import ctypes, os, sys, torch
sys.path.insert(0, os.getcwd())
from triton_distributed_b200 import _lib, utils
from triton_distributed_b200.runtime.heap import SymmTimeoutError
lib = _lib.load(build_if_missing=False)
assert lib.b200_debug_checks() == 1, "the regular library was loaded: the bad-pointer call below must not run on it"
utils.initialize_distributed(seed=0, heap_bytes=64 << 20)
heap = utils.get_heap()
good = heap.create_tensor((4,), torch.int32)
ok = torch.zeros(1, dtype=torch.int32, device="cuda")
_lib.call("b200_test_notify_add", heap.ctx, _lib.ptr(good), 0, 1, _lib.ptr(ok), _lib.stream_ptr())
torch.cuda.synchronize()
heap.check_status("in-heap notify")            # a pointer inside the heap passes the check
assert int(good[0]) == 1 and int(ok) == 1
stray = torch.zeros(4, dtype=torch.int32, device="cuda")   # NOT in the symmetric heap
_lib.call("b200_test_notify_add", heap.ctx, _lib.ptr(stray), 0, 1, _lib.ptr(ok), _lib.stream_ptr())
torch.cuda.synchronize()
try:
    heap.check_status("stray notify")
except SymmTimeoutError as e:
    assert "bad kernel argument" in str(e), e
    assert int(stray[0]) == 1                  # the access fell back to the local address
    print("bad pointer reported:", e)
else:
    raise AssertionError("the checking build did not report a pointer outside the heap")
heap.free(good)
utils.finalize_distributed()
print("debug build ok")
"""


def _env():
    env = dict(os.environ)
    env.update({"B200DIST_DEBUG_LIB": "1", "B200DIST_NO_BUILD": "1", "RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1",
                "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(29900 + os.getpid() % 90)})
    return env


@pytest.mark.skipif(not os.path.exists(DEBUG_LIB), reason="the checking library has not been built (build --debug)")
def test_checking_build_reports_a_pointer_outside_the_heap():
    res = subprocess.run([sys.executable, "-c", _BAD_POINTER], capture_output=True, text=True, timeout=300, env=_env(), cwd=ROOT)
    sys.stdout.write(res.stdout[-1500:])
    sys.stderr.write(res.stderr[-1500:])
    assert res.returncode == 0 and "debug build ok" in res.stdout


@pytest.mark.skipif(not os.path.exists(DEBUG_LIB), reason="the checking library has not been built (build --debug)")
def test_world1_cases_pass_under_the_checking_build():
    """Every single-rank case of the heap, the primitives and the fused kernels with the checks and the delays on."""
    res = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_dist_world1.py", "-x", "-q", "-m", "gpu",
                          "-p", "no:cacheprovider"], capture_output=True, text=True, timeout=900, env=_env(), cwd=ROOT)
    sys.stdout.write(res.stdout[-1500:])
    assert res.returncode == 0, res.stdout[-3000:]
