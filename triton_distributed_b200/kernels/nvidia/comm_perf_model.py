"""Speed-of-light estimates for intra-node collectives over NVLink 5 / NVSwitch.

API parity with ``python/triton_dist/kernels/nvidia/comm_perf_model.py:34-114``. The link figure is the measured
peer-copy bandwidth of this pool (770 GB/s per direction per GPU; 900 nominal).
"""
from __future__ import annotations

NVLINK_GBPS_PER_DIRECTION = 770.0


def get_nic_gbps_per_gpu() -> float:
    """No NIC is modelled: this library spans one node."""
    return 0.0


def estimate_all_gather_time_ms(nbytes_per_rank: int, world_size: int, local_world_size: int | None = None) -> float:
    """Every GPU receives (world - 1) shards through its own NVLink ports."""
    return (world_size - 1) * nbytes_per_rank / (NVLINK_GBPS_PER_DIRECTION * 1e9) * 1e3


def estimate_reduce_scatter_time_ms(nbytes_total: int, world_size: int, local_world_size: int | None = None) -> float:
    """Every GPU sends (world - 1) / world of its partial and receives as much."""
    return (world_size - 1) / world_size * nbytes_total / (NVLINK_GBPS_PER_DIRECTION * 1e9) * 1e3


def fused_roofline_ms(flops: float, nvlink_bytes: float, peak_tflops: float = 1605.6) -> float:
    """Target time of a fused compute + collective kernel: the slower of its math at the measured GEMM peak and
    its NVLink bytes at the measured link bandwidth."""
    return max(flops / (peak_tflops * 1e12), nvlink_bytes / (NVLINK_GBPS_PER_DIRECTION * 1e9)) * 1e3
