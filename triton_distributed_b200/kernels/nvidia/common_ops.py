"""Host-visible synchronisation helpers.

API parity with ``python/triton_dist/kernels/nvidia/common_ops.py:209-277`` (``BarrierAllContext``,
``barrier_all_on_stream``, ``wait_eq``, ``set_signal``). The device-side helpers of that module
(grid barrier, barrier_all, bisect, vector loads) are C++ device functions in
``csrc/include/b200/primitives.cuh``.
"""
from __future__ import annotations

import torch

from ...runtime.heap import get_heap


class BarrierAllContext:
    """Kept for API parity: the barrier state (flags + device-resident epoch) lives in the heap."""

    def __init__(self, is_intra_node: bool = True):
        if not is_intra_node:
            raise NotImplementedError("single node only")
        self.is_intra_node = True
        self.heap = get_heap()


def barrier_all_on_stream(ctx: BarrierAllContext | None = None, stream: torch.cuda.Stream | None = None) -> None:
    (ctx.heap if ctx is not None else get_heap()).barrier_all(stream)


def set_signal(tensor: torch.Tensor, index: int, value: int, stream: torch.cuda.Stream | None = None) -> None:
    """Stream-ordered store of `value` into ``tensor[index]`` (a local or peer-mapped flag)."""
    with torch.cuda.stream(stream or torch.cuda.current_stream()):
        tensor[index : index + 1].fill_(value)


def wait_eq(tensor: torch.Tensor, index: int, value: int, stream: torch.cuda.Stream | None = None,
            timeout_ms: int = 10000) -> None:
    """Block the HOST until ``tensor[index] == value`` (bounded). Device code should use the bounded
    device-side waits instead; a stream-blocking wait has no timeout and is not offered."""
    import time
    (stream or torch.cuda.current_stream()).synchronize()
    t0 = time.time()
    while int(tensor[index].item()) != value:
        if (time.time() - t0) * 1000 > timeout_ms:
            raise TimeoutError(f"flag[{index}] did not reach {value} within {timeout_ms} ms")
        time.sleep(0.0005)
