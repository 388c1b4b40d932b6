"""AG-GEMM: ``C[M, N/r] = all_gather(A)[M, K] @ B[N/r, K].T`` in one fused sm_100a kernel.

API parity with ``python/triton_dist/kernels/nvidia/allgather_gemm.py`` (``create_ag_gemm_context``
:489, ``ag_gemm`` :534, ``gemm_persistent`` :660, ``gemm_non_persistent`` :707). The reference runs a
copy-engine all-gather on a side stream and a consumer GEMM that spins on per-rank flags; here the
communication warps of the GEMM kernel itself move the shards over NVLink while the tcgen05 mainloop
consumes row blocks as they land (``csrc/kernels/gemm_sm100.cu``). No side stream, no flag reset, no
barrier: flags are epochs and counters only grow.

Two gathers. ``sm_push_fused`` stores this rank's shard into every peer's buffer in the order in which the
peers' tile schedules need it and bumps the destination's per-block row counters: posted stores run at link
speed however small M is, but while they drain they compete with the epilogue's stores. ``sm_pull_fused``
pulls the peers' shards with 16-byte loads after a "shard published" flag: free when one rank's share of the
GEMM is long enough to cover the first pull, latency-bound when it is not. ``auto`` (default) picks per call
from the world size and the bytes to move; ``B200DIST_AG_PUSH=1`` / ``0`` forces one. Calls of both kinds can
share a context (separate flags and counters, common epoch).
"""
from __future__ import annotations

import dataclasses
import os

import torch

from ... import _lib, ops
from ..._lib import dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap


PUSH_MAX_OUTGOING_BYTES = 64 << 20


@dataclasses.dataclass
class AllGatherGEMMTensorParallelContext:
    rank: int
    num_ranks: int
    num_local_ranks: int
    max_M: int
    N_per_rank: int
    K: int
    dtype: torch.dtype
    heap: SymmHeap
    symm_workspaces: list[torch.Tensor]   # the two parity gather buffers [max_M, K]
    symm_ready: torch.Tensor              # u32[world] "shard of rank s published" epochs (remote-written)
    blk_cnt: torch.Tensor                 # local row-arrival counters per 128-row block
    blk_flag: torch.Tensor                # local block epochs
    sync: torch.Tensor                    # local [epoch, done counter, local chunk counter, -]
    symm_blk_cnt: torch.Tensor | None = None   # push gather: u32[2, nblk] rows landed per block and parity (remote-added)
    blk_base: torch.Tensor | None = None       # push gather: local u32[2, nblk] counter values before the next call
    BLOCK_M: int = 128
    BLOCK_N: int = 256
    BLOCK_K: int = 64
    stages: int = 4
    group_m: int = 8
    max_ctas: int = 0
    for_correctness: bool = False
    is_multinode: bool = False
    all_gather_method: str = "auto"

    def method_for(self, Mr: int) -> str:
        """The gather used for a call with Mr rows per rank."""
        if self.all_gather_method != "auto":
            return self.all_gather_method
        outgoing = (self.num_ranks - 1) * Mr * self.K * self.dtype.itemsize
        # many ranks: small problems are latency-bound (push), large ones back-pressure the store path (pull).
        # two ranks: one peer, so pushed rows land as one stream while the local half is multiplied (measured at
        # M = 8192, K = 8192: 2630 us pushed against 3095 us pulled)
        if self.num_ranks == 2:
            return "sm_push_fused"
        return "sm_push_fused" if self.num_ranks >= 4 and outgoing <= PUSH_MAX_OUTGOING_BYTES else "sm_pull_fused"

    @property
    def symm_workspace(self) -> torch.Tensor:
        return self.symm_workspaces[0]

    @property
    def phase(self) -> int:
        """Number of calls completed (the device-resident epoch)."""
        return int(self.sync[0].item())

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.symm_workspaces + [self.symm_ready] + ([self.symm_blk_cnt] if self.symm_blk_cnt is not None else []):
            self.heap.free(t)
        self.symm_workspaces = []
        self.symm_blk_cnt = None

    finailize = finalize  # the reference spells it this way (allgather_gemm.py:483)


def create_ag_gemm_context(tensor_A: torch.Tensor, tensor_B: torch.Tensor, rank: int, num_ranks: int, max_M: int,
                           num_local_ranks: int = 8, BLOCK_M: int = 128, BLOCK_N: int = 256, BLOCK_K: int = 64,
                           stages: int = 4, ag_intranode_stream=None, ag_internode_stream=None,
                           for_correctness: bool = False) -> AllGatherGEMMTensorParallelContext:
    """tensor_A: this rank's shard [M/r, K]; tensor_B: [N/r, K]; max_M: largest gathered M the context serves."""
    heap = get_heap()
    if num_ranks != heap.world:
        raise ValueError("AG-GEMM spans the ranks of the symmetric heap (single node)")
    K = tensor_A.shape[1]
    if tensor_B.shape[1] != K:
        raise ValueError("A and B disagree on K")
    if max_M % num_ranks != 0:
        raise ValueError("max_M must be divisible by the number of ranks")
    ws = [heap.create_tensor((max_M, K), tensor_A.dtype, align=1024) for _ in range(2)]
    ready = heap.create_tensor((16,), torch.int32)
    nblk = (max_M + 127) // 128 + 2
    dev = tensor_A.device
    ctx = AllGatherGEMMTensorParallelContext(
        rank=rank, num_ranks=num_ranks, num_local_ranks=num_local_ranks, max_M=max_M, N_per_rank=tensor_B.shape[0], K=K,
        dtype=tensor_A.dtype, heap=heap, symm_workspaces=ws, symm_ready=ready,
        blk_cnt=torch.zeros(nblk, dtype=torch.int32, device=dev), blk_flag=torch.zeros(nblk, dtype=torch.int32, device=dev),
        sync=torch.zeros(4, dtype=torch.int32, device=dev), for_correctness=for_correctness)
    ctx.symm_blk_cnt = heap.create_tensor((2, nblk), torch.int32)
    ctx.symm_blk_cnt.zero_()
    ctx.blk_base = torch.zeros((2, nblk), dtype=torch.int32, device=dev)
    forced = os.environ.get("B200DIST_AG_PUSH")
    if forced is not None:
        ctx.all_gather_method = "sm_pull_fused" if forced == "0" else "sm_push_fused"
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def ag_gemm(a: torch.Tensor, b: torch.Tensor, ctx: AllGatherGEMMTensorParallelContext, rank: int | None = None,
            num_ranks: int | None = None, persistent: bool = True, autotune: bool = False,
            straggler_option=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """a: local shard [M/r, K]; b: [N/r, K]. Returns C [M, N/r] (rows in rank order)."""
    if ctx is None:
        raise ValueError("ag_gemm needs a context from create_ag_gemm_context")
    Mr, K = a.shape
    N = b.shape[0]
    M = Mr * ctx.num_ranks
    if M > ctx.max_M or K != ctx.K:
        raise ValueError(f"problem [{M},{K}] exceeds the context ([{ctx.max_M},{ctx.K}])")
    if not a.is_contiguous() or b.stride(1) != 1:
        raise ValueError("a must be contiguous and b row-major")
    if b.shape[1] != K:
        raise ValueError(f"a [{Mr},{K}] and b [{N},{b.shape[1]}] disagree on K")
    if a.dtype != ctx.dtype or b.dtype != a.dtype:
        raise TypeError(f"a ({a.dtype}) and b ({b.dtype}) must have the context's dtype ({ctx.dtype})")
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    elif tuple(out.shape) != (M, N) or out.dtype != a.dtype or out.stride(1) != 1:
        raise ValueError("out must be a row-major [M, N] tensor of the input dtype")
    if straggler_option is not None and straggler_option[0] == ctx.rank:
        torch.cuda._sleep(int(straggler_option[1]))
    _lib.call("b200_ag_gemm", ctx.heap.ctx, ptr(a), ptr(ctx.symm_workspaces[0]), ptr(ctx.symm_workspaces[1]), ptr(b),
              ptr(out), Mr, N, K, b.stride(0), out.stride(0), dtype_code(a.dtype), ptr(ctx.symm_ready), ptr(ctx.blk_cnt),
              ptr(ctx.blk_flag), ptr(ctx.sync), ctx.group_m, ctx.max_ctas, 1 if ctx.method_for(Mr) == "sm_push_fused" else 0,
              ptr(ctx.symm_blk_cnt), ptr(ctx.blk_base), ctx.symm_blk_cnt.shape[1], stream_ptr())
    ops._count()
    return out


def gemm_persistent(a: torch.Tensor, b: torch.Tensor, ctx=None, autotune: bool = False) -> torch.Tensor:
    """Local GEMM ``a[M,K] @ b[N,K].T`` on the same tcgen05 mainloop, without communication."""
    return ops.gemm(a, b)


def gemm_non_persistent(a: torch.Tensor, b: torch.Tensor, ctx=None) -> torch.Tensor:
    """Kept for API parity; the persistent kernel already degrades to one tile per CTA for small problems."""
    return ops.gemm(a, b)
