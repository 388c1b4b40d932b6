"""Kernel library: context factories and op entry points (module layout follows ``python/triton_dist/kernels``)."""
