"""The decode GEMM entry point for callers that cannot allocate device memory.

Some hosts of this library (a runtime whose memory plan is frozen, a pool that owns the whole device) treat
any cudaMalloc after start-up as an error, so ``b200_gemm_skinny_static`` keeps its split-accumulation area
inside the library image. The test calls it through its exported C symbol, twice in a row (the second call
relies on the first having left the shared area zeroed), and compares with the regular entry point.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, x, w, out, dual):
    M, K = x.shape
    N = out.shape[1]
    rc = lib.b200_gemm_skinny_static(
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(out.data_ptr()), M, N, K,
        x.stride(0), w.stride(0), out.stride(0), 1 if dual else 0, 0,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.b200_last_error().decode()


@pytest.mark.parametrize("M,N,K,dual", [(8, 5120, 1024, False), (16, 1280, 5120, False), (8, 3200, 5120, True)])
def test_static_entry_matches_regular_entry_twice(M, N, K, dual):
    from triton_distributed_b200 import _lib, ops
    lib = ctypes.CDLL(str(_lib.LIB_PATH))  # the exported C symbol, not the Python wrapper
    lib.b200_last_error.restype = ctypes.c_char_p
    torch.manual_seed(11)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn((2 * N if dual else N), K, device="cuda", dtype=torch.bfloat16) * 0.05
    want = ops.gemm_skinny(x, w, swiglu=dual)
    for _ in range(2):
        got = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        _call_static(lib, x, w, got, dual)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    ref = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:] if dual else ref
    torch.testing.assert_close(got.float(), ref, rtol=3e-2, atol=3e-2)


def test_static_entry_rejects_oversized_problems():
    from triton_distributed_b200 import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    lib.b200_last_error.restype = ctypes.c_char_p
    lib.b200_gemm_skinny_static_capacity_floats.restype = ctypes.c_longlong
    assert lib.b200_gemm_skinny_static_capacity_floats() == 1 << 20
    x = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(65536, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(256, 65536, device="cuda", dtype=torch.bfloat16)
    rc = lib.b200_gemm_skinny_static(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                                     ctypes.c_void_p(out.data_ptr()), 256, 65536, 64, 64, 64, 65536, 0, 0,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"built-in area" in lib.b200_last_error()
