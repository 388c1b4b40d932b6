"""A Blackwell-native (sm_100a) framework for compute-communication overlap.

PyTorch on top, hand-written CUDA underneath: a CUDA-VMM symmetric heap with NVLS multicast instead
of NVSHMEM, device primitives (wait / notify / symm_at / put / get / barriers) as C++ device
functions, and fused tcgen05 kernels for AG-GEMM, GEMM-RS, AllReduce(+RMSNorm), MoE and decode
attention. The public names follow the reference package ``triton_dist``.
"""
__version__ = "0.1.0"
