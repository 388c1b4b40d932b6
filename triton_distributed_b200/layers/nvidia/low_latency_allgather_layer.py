"""All-gather layer over a staged symmetric buffer.

API parity with ``python/triton_dist/layers/nvidia/low_latency_allgather_layer.py:30-187``
(``AllGatherLayer(nnodes, world_size, rank, max_buffer_size, stages)`` and its ``forward_*`` methods). On one
NVSwitch node the 3D / NUMA variants have no topology to exploit and run the 2D kernels.
"""
from __future__ import annotations

import torch

from ...kernels.nvidia.low_latency_allgather import create_fast_allgather_context, fast_allgather
from ...runtime.heap import get_heap


class AllGatherLayer:

    def __init__(self, nnodes: int, world_size: int, rank: int, max_buffer_size: int = 2 * 32 * 1024 * 1024, stages: int = 2):
        if nnodes != 1:
            raise NotImplementedError("single node only")
        self.heap = get_heap()
        self.world_size, self.rank, self.stages = world_size, rank, max(1, stages)
        self.max_buffer_size = max_buffer_size
        self.ctx = create_fast_allgather_context(rank, 0, world_size, 1, max_buffer_size)
        self.buffers = [self.heap.create_tensor((max_buffer_size,), torch.uint8, align=1024) for _ in range(self.stages)]
        self.calls = 0

    def _run(self, local: torch.Tensor, mode: str) -> torch.Tensor:
        """local: this rank's contribution (any shape). Returns [world, *local.shape] (a view of a staging buffer,
        valid for `stages` further calls)."""
        nbytes = local.numel() * local.element_size()
        if nbytes * self.world_size > self.max_buffer_size:
            raise ValueError("message exceeds the layer's buffer")
        buf = self.buffers[self.calls % self.stages]
        self.calls += 1
        view = buf[: nbytes * self.world_size].view(local.dtype).view(self.world_size, *local.shape)
        view[self.rank].copy_(local)
        fast_allgather(view, self.ctx, mode=mode)
        return view

    def forward_pull(self, local):
        return self._run(local, "pull")

    def forward_push_2d(self, local):
        return self._run(local, "push2d")

    def forward_push_2d_ll(self, local):
        return self._run(local, "push2d_ll")

    def forward_push_2d_ll_multimem(self, local):
        return self._run(local, "push2d_ll_multimem" if self.heap.has_multicast else "push2d_ll")

    forward_push_3d = forward_push_numa_2d = forward_push_2d
    forward_push_3d_ll = forward_push_numa_2d_ll = forward_push_numa_2d_ll_multinode = forward_push_2d_ll

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for b in self.buffers:
            self.heap.free(b)
        self.buffers = []
        self.ctx.finalize()
