"""GEMM-RS: ``out[M/r, N] = reduce_scatter(A[M, K/r] @ B[N, K/r].T)`` in one fused sm_100a kernel.

API parity with ``python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py`` (``create_gemm_rs_context``
:79, ``gemm_rs`` :576). The reference's producer GEMM writes into a symmetric buffer and a second
stream scatters and ring-reduces; here the tcgen05 epilogue stores every output row straight into
the owner rank's slot over NVLink, bumps the owner's arrival counters with a release, and the same
kernel finishes with the owner-side fp32 reduction of its rows (``csrc/kernels/gemm_sm100.cu``).
The sum order is fixed (slot 0..r-1), so results are reproducible run to run.

With an NVLS multicast mapping the reduction can run inside the switch instead (``ctx.nvls`` / ``B200DIST_RS_NVLS``:
True / 1 to enable; the default is the slot reduction):
the epilogue keeps every partial row in this rank's own memory at the owner's offset, and the owner issues one
``multimem.ld_reduce`` per 16 bytes that returns the sum over the ranks (fp32 accumulation in the switch), the role of
the multimem reduce-scatter in ``kernels/nvidia/moe_reduce_rs.py:1128-1152`` of the reference. The owner then receives
one copy of its rows over NVLink instead of ``world - 1`` and sums nothing itself.
"""
from __future__ import annotations

import dataclasses
import os

import torch

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap



@dataclasses.dataclass
class GEMMReduceScatterTensorParallelContext:
    rank: int
    world_size: int
    local_world_size: int
    max_M: int
    N: int
    output_dtype: torch.dtype
    heap: SymmHeap
    slots: list[torch.Tensor]     # two parity buffers [world, max_M / world, N]
    rs_cnt: torch.Tensor          # symmetric u32 [world, rs_blocks] arrival counters (remote-incremented)
    rs_base: torch.Tensor         # local counter bases
    sync: torch.Tensor
    rs_blocks: int
    BLOCK_M: int = 128
    BLOCK_N: int = 256
    BLOCK_K: int = 64
    stages: int = 4
    group_m: int = 8
    max_ctas: int = 0
    nvls: bool | None = None      # reduce in the switch (needs the heap's multicast mapping); None / False = slots

    def use_nvls(self, M: int) -> bool:
        """Whether a call with M rows sums in the switch: only when asked to (``nvls=True`` or ``B200DIST_RS_NVLS=1``).
        Measured on the Llama-3-70B down-projection (N = 8192): at two ranks the in-switch reduction wins from a few
        thousand rows (M = 8192: 1452 us against 1684 us with slots; M = 2048: 397 against 375 us), at four ranks the
        slots win (714 against 740 us). An automatic switch at two ranks and M >= 4096 made the Qwen3-32B prefill
        (N = 5120) 4 % slower, so there is none."""
        return bool(self.nvls) and self.heap.has_multicast

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.slots + [self.rs_cnt]:
            self.heap.free(t)
        self.slots = []


def create_gemm_rs_context(max_M: int, N: int, rank: int, world_size: int, local_world_size: int,
                           output_dtype: torch.dtype, rs_stream=None, BLOCK_M: int = 128, BLOCK_N: int = 256,
                           BLOCK_K: int = 64, GROUP_M: int = 8, stages: int = 4) -> GEMMReduceScatterTensorParallelContext:
    heap = get_heap()
    if world_size != heap.world:
        raise ValueError("GEMM-RS spans the ranks of the symmetric heap (single node)")
    if max_M % world_size != 0:
        raise ValueError("max_M must be divisible by the world size")
    mr_cap = max_M // world_size
    rs_blocks = (mr_cap + 127) // 128 + 2
    slots = [heap.create_tensor((world_size, mr_cap, N), output_dtype, align=1024) for _ in range(2)]
    rs_cnt = heap.create_tensor((world_size * rs_blocks,), torch.int32)
    ctx = GEMMReduceScatterTensorParallelContext(
        rank=rank, world_size=world_size, local_world_size=local_world_size, max_M=max_M, N=N, output_dtype=output_dtype,
        heap=heap, slots=slots, rs_cnt=rs_cnt,
        rs_base=torch.zeros(world_size * rs_blocks, dtype=torch.int32, device="cuda"),
        sync=torch.zeros(4, dtype=torch.int32, device="cuda"), rs_blocks=rs_blocks, group_m=GROUP_M,
        nvls={"1": True, "0": False}.get(os.environ.get("B200DIST_RS_NVLS", ""), None))
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def gemm_rs(a: torch.Tensor, b: torch.Tensor, ctx: GEMMReduceScatterTensorParallelContext, persistent: bool = True,
            fuse_scatter: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """a: [M, K/r]; b: [N, K/r]. Returns this rank's rows [M/r, N] of the summed product."""
    M, K = a.shape
    N = b.shape[0]
    if N != ctx.N or M > ctx.max_M:
        raise ValueError(f"problem [{M},{N}] does not fit the context ([{ctx.max_M},{ctx.N}])")
    if M % ctx.world_size != 0:
        raise ValueError("M must be divisible by the world size")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("a and b must be row-major")
    if b.shape[1] != K:
        raise ValueError(f"a [{M},{K}] and b [{N},{b.shape[1]}] disagree on K")
    if a.dtype != ctx.output_dtype or b.dtype != a.dtype:
        raise TypeError(f"a ({a.dtype}) and b ({b.dtype}) must have the context's dtype ({ctx.output_dtype}): the slots "
                        "that peers write hold the output dtype")
    if out is None:
        out = torch.empty((M // ctx.world_size, N), dtype=ctx.output_dtype, device=a.device)
    elif tuple(out.shape) != (M // ctx.world_size, N) or out.dtype != ctx.output_dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [M / world, N] tensor of the context's dtype")
    _lib.call("b200_gemm_rs", ctx.heap.ctx, ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0),
              dtype_code(a.dtype), ptr(ctx.slots[0]), ptr(ctx.slots[1]), ptr(ctx.rs_cnt), ptr(ctx.rs_base), ptr(ctx.sync),
              ctx.max_M // ctx.world_size, ctx.rs_blocks, ctx.group_m, ctx.max_ctas, 1 if ctx.use_nvls(M) else 0, stream_ptr())
    ops._count()
    return out
