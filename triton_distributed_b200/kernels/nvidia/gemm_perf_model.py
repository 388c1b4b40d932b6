"""Speed-of-light estimates for GEMMs on the current GPU.

API parity with ``python/triton_dist/kernels/nvidia/gemm_perf_model.py:61-236`` (``get_tensorcore_tflops``,
``get_dram_gbps``, ``estimate_gemm_sol_time_ms``). B200 figures are the measured ones of this pool (cuBLAS bf16 burst
and STREAM-style copy); other devices fall back to their datasheet numbers.
"""
from __future__ import annotations

import torch

_DEVICE_TABLE = {  # name fragment -> (dense bf16 TFLOP/s, HBM GB/s)
    "B200": (1605.6, 6531.9),
    "H100": (989.0, 3350.0), "H800": (989.0, 3350.0), "H200": (989.0, 4800.0), "A100": (312.0, 2039.0), "L40": (181.0, 864.0),
}
_DTYPE_SCALE = {torch.bfloat16: 1.0, torch.float16: 1.0, torch.float8_e4m3fn: 2.0, torch.float8_e5m2: 2.0, torch.int8: 2.0,
                torch.float32: 0.5}


def _lookup(device=None):
    name = torch.cuda.get_device_name(device) if torch.cuda.is_available() else "B200"
    for frag, v in _DEVICE_TABLE.items():
        if frag in name:
            return v
    return _DEVICE_TABLE["B200"]


def get_tensorcore_tflops(dtype: torch.dtype = torch.bfloat16, device=None, num_ctas: int | None = None) -> float:
    tf = _lookup(device)[0] * _DTYPE_SCALE.get(dtype, 1.0)
    if num_ctas is not None and torch.cuda.is_available():
        sms = torch.cuda.get_device_properties(device or 0).multi_processor_count
        tf *= min(1.0, num_ctas / sms)
    return tf


def get_dram_gbps(device=None) -> float:
    return _lookup(device)[1]


def estimate_gemm_sol_time_ms(M: int, N: int, K: int, dtype: torch.dtype = torch.bfloat16, device=None) -> float:
    """max(compute at tensor-core peak, operand + result traffic at HBM bandwidth) in milliseconds."""
    es = torch.empty((), dtype=dtype).element_size()
    t_compute = 2.0 * M * N * K / (get_tensorcore_tflops(dtype, device) * 1e12)
    t_mem = (M * K + N * K + M * N) * es / (get_dram_gbps(device) * 1e9)
    return max(t_compute, t_mem) * 1e3
