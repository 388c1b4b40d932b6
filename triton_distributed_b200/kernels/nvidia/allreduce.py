"""AllReduce over the symmetric heap, optionally fused with residual-add + RMSNorm.

API parity with ``python/triton_dist/kernels/nvidia/allreduce.py`` (``create_allreduce_ctx`` :114,
``all_reduce`` :1054, ``get_auto_allreduce_method`` :1039). Method mapping on one NVSwitch node:

  =====================  =====================================================================
  reference method       kernel used here (``csrc/kernels/allreduce.cu``)
  =====================  =====================================================================
  OneShot, OneShot_TMA   ONE_SHOT push (plain 16-byte P2P stores; TMA adds nothing for a push)
  TwoShot                TWO_SHOT pull-reduce + push-broadcast
  OneShot_Multimem       multimem.ld_reduce over the whole buffer
  TwoShot_Multimem(_ST)  multimem.ld_reduce of the own slice + multimem.st broadcast
  DoubleTree             ONE_SHOT for <= 64 KiB else TWO_SHOT: behind an NVSwitch every peer is one
                         hop away, so a tree only adds hops; the name is kept for API parity
  =====================  =====================================================================

Fused calls of at most 512 KB (the decode path) take a low-latency packet kernel (``csrc/kernels/allreduce_ll.cu``:
8-byte {data, epoch} packets that the receiver polls, so there is no flag exchange, fence or barrier; one
``multimem.st`` per packet when the heap has an NVLS mapping). ``B200DIST_AR_LL=0`` / ``B200DIST_AR_LL_MC=0`` switch the
packet path / its multicast stores off.

Unlike the reference there is no staging memcpy outside the kernel and no host-side call counter:
the kernel stages, synchronises CTA-by-CTA with its peers, reduces and (optionally) normalises, and
its epoch lives in device memory, so every method — chunked or not — can be captured in a CUDA graph.
"""
from __future__ import annotations

import dataclasses
import os

import torch

from ... import _lib, ops
from ..._lib import c_float, dtype_code, ptr, stream_ptr
from ...runtime.heap import SymmHeap, get_heap
from ..allreduce import AllReduceMethod

_NATIVE = {
    AllReduceMethod.OneShot: 0, AllReduceMethod.OneShot_TMA: 0,
    AllReduceMethod.TwoShot: 1,
    AllReduceMethod.OneShot_Multimem: 2,
    AllReduceMethod.TwoShot_Multimem: 3, AllReduceMethod.TwoShot_Multimem_ST: 3,
}


@dataclasses.dataclass
class AllReduceContext:
    workspace_nbytes: int
    rank: int
    world_size: int
    local_world_size: int
    heap: SymmHeap
    workspaces: list[torch.Tensor]  # two parity buffers (uint8)
    flags: torch.Tensor             # symmetric u32 CTA-level barrier epochs
    sync: torch.Tensor              # local [epoch, done counter]
    max_ctas: int

    def finalize(self) -> None:
        self.heap.sync_and_check(type(self).__name__)
        for t in self.workspaces + [self.flags] + list(getattr(self, "ll_ws", None) or []):
            self.heap.free(t)
        self.workspaces = []
        self.ll_ws = None


_AR_LL = os.environ.get("B200DIST_AR_LL", "1") != "0"
_AR_LL_MC = os.environ.get("B200DIST_AR_LL_MC", "1") != "0"
_LL_MAX_BYTES = 512 * 1024   # input bytes per call served by the low-latency packet path


def create_allreduce_ctx(workspace_nbytes: int, rank: int, world_size: int, local_world_size: int) -> AllReduceContext:
    """`workspace_nbytes` bounds the bytes one call can move per parity buffer; larger inputs are chunked."""
    heap = get_heap()
    if world_size != heap.world:
        raise ValueError("all_reduce spans the ranks of the symmetric heap (single node)")
    lib = _lib.load()
    max_ctas = lib.b200_allreduce_max_ctas()
    ws = [heap.create_tensor((workspace_nbytes,), torch.uint8, align=1024) for _ in range(2)]
    flags = heap.create_tensor((2 * max_ctas * 8,), torch.int32)
    ctx = AllReduceContext(workspace_nbytes, rank, world_size, local_world_size, heap, ws, flags,
                           torch.zeros(4, dtype=torch.int32, device="cuda"), max_ctas)
    if _AR_LL and world_size > 1:
        # dedicated packet buffers (data and flag share a word, so they must never hold anything else)
        ctx.ll_ws = [heap.create_tensor((world_size * _LL_MAX_BYTES * 2,), torch.uint8, align=1024) for _ in range(2)]
        ctx.ll_sync = torch.zeros(256, dtype=torch.int32, device="cuda")  # one call counter per CTA
    heap.barrier_all()
    torch.cuda.synchronize()
    return ctx


def get_auto_allreduce_method(nbytes: int, has_multicast: bool | None = None, world: int | None = None) -> AllReduceMethod:
    """Small messages are latency-bound: the one-shot push (one meeting point) wins up to 1 MB at eight ranks, 2 MB at
    four and 8 MB at two, where it moves no more data than a two-shot. Beyond that the two-shot forms are
    bandwidth-bound, with the reduction in the switch when the heap has an NVLS mapping and more than two ranks share
    it. (Measured at 2, 4 and 8 GPUs; the NVLS one-shot never beat the plain one-shot on this machine.)"""
    heap = get_heap() if (has_multicast is None or world is None) else None
    if has_multicast is None:
        has_multicast = heap.has_multicast
    if world is None:
        world = heap.world
    if nbytes <= (8 << 20 if world <= 2 else 2 << 20 if world <= 4 else 1 << 20):
        return AllReduceMethod.OneShot
    return AllReduceMethod.TwoShot_Multimem if (has_multicast and world > 2) else AllReduceMethod.TwoShot


def _resolve(method: AllReduceMethod | None, nbytes: int, ctx: AllReduceContext) -> int:
    if method is None or method == AllReduceMethod.Unknown:
        method = get_auto_allreduce_method(nbytes, ctx.heap.has_multicast, ctx.world_size)
    if method == AllReduceMethod.DoubleTree:
        method = AllReduceMethod.OneShot if nbytes <= 64 * 1024 else AllReduceMethod.TwoShot
    if method in (AllReduceMethod.OneShot_Multimem, AllReduceMethod.TwoShot_Multimem,
                  AllReduceMethod.TwoShot_Multimem_ST) and not ctx.heap.has_multicast:
        raise RuntimeError(f"{method.name} needs an NVLS multicast mapping, which this heap does not have")
    return _NATIVE[method]


def _ws_factor(native: int, world: int, fused: bool) -> int:
    return {0: world, 2: 1}.get(native, 3 if fused else 2)


def _num_ctas(nbytes: int, ctx: AllReduceContext, max_sm: int) -> int:
    n = max(1, min(ctx.max_ctas, nbytes // (32 * 1024)))
    if max_sm > 0:
        n = min(n, max_sm)
    return int(n)


def all_reduce(x: torch.Tensor, output: torch.Tensor | None = None, method: AllReduceMethod | None = None,
               ctx: AllReduceContext | None = None, max_sm: int = -1, straggler_option=None) -> torch.Tensor:
    """Sum `x` over all ranks into `output` (allocated when None)."""
    if ctx is None:
        raise ValueError("all_reduce needs a context from create_allreduce_ctx")
    if not x.is_contiguous():
        x = x.contiguous()
    if output is None:
        output = torch.empty_like(x)
    if straggler_option is not None and straggler_option[0] == ctx.rank:
        torch.cuda._sleep(int(straggler_option[1]))
    es = x.element_size()
    native = _resolve(method, x.numel() * es, ctx)
    factor = _ws_factor(native, ctx.world_size, False)
    unit = (16 // es) * ctx.world_size
    max_elems = (ctx.workspace_nbytes // (factor * es)) // unit * unit
    if max_elems <= 0:
        raise ValueError("allreduce workspace is too small for a single vector per rank")
    n = x.numel()
    xf, of = x.view(-1), output.view(-1)
    done = 0
    while done < n:
        cur = min(max_elems, n - done)
        cur_native = native
        if cur % unit != 0:  # ragged tail: the one-shot push has no divisibility requirement beyond 16 bytes
            if cur % (16 // es) != 0:
                raise ValueError("all_reduce needs a multiple of 16 bytes")
            cur_native = 0
            cap = (ctx.workspace_nbytes // (ctx.world_size * es)) // (16 // es) * (16 // es)
            cur = min(cur, cap)
        _lib.call("b200_allreduce", ctx.heap.ctx, ptr(xf[done:]), ptr(of[done:]), _lib.c_u64(cur), dtype_code(x.dtype),
                  cur_native, ptr(ctx.workspaces[0]), ptr(ctx.workspaces[1]), ptr(ctx.flags), ptr(ctx.sync), 0, None, None,
                  None, None, c_float(0.0), _num_ctas(cur * es, ctx, max_sm), stream_ptr())
        ops._count()
        done += cur
    return output


def all_reduce_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, gamma: torch.Tensor, eps: float,
                       ctx: AllReduceContext, method: AllReduceMethod | None = None,
                       normed_out: torch.Tensor | None = None, residual_out: torch.Tensor | None = None,
                       max_sm: int = -1):
    """Fused ``h = all_reduce(x) + residual; y = rmsnorm(h) * gamma``. x: [rows, hidden].

    Returns (y, h). `residual_out` defaults to `residual` (in place) when a residual is given.
    """
    rows, hidden = x.shape
    es = x.element_size()
    if (method is None and getattr(ctx, "ll_ws", None) is not None and es == 2 and x.numel() * es <= _LL_MAX_BYTES
            and hidden % 2 == 0 and hidden <= 8192 and x.is_contiguous()):
        # low-latency path: 8-byte {data, epoch} packets, no flag exchange, no fence
        if normed_out is None:
            normed_out = torch.empty_like(x)
        if residual_out is None:
            residual_out = residual if residual is not None else torch.empty_like(x)
        _lib.call("b200_allreduce_ll", ctx.heap.ctx, ptr(x), rows, hidden, dtype_code(x.dtype), ptr(ctx.ll_ws[0]),
                  ptr(ctx.ll_ws[1]), ptr(ctx.ll_sync), ptr(residual), ptr(residual_out), ptr(gamma), ptr(normed_out),
                  c_float(eps), 1 if (_AR_LL_MC and ctx.heap.has_multicast) else 0, stream_ptr())
        ops._count()
        return normed_out, residual_out
    if method is None and x.numel() * es <= 512 * 1024:
        # latency-bound: one push, one meeting point, one pass (a two-shot costs two meetings and three passes)
        method = AllReduceMethod.OneShot
    native = _resolve(method, x.numel() * es, ctx)
    if native in (1, 3) and rows % ctx.world_size != 0:
        native = 0 if native == 1 else 2  # row ownership needs rows divisible by the world size
    factor = _ws_factor(native, ctx.world_size, True)
    cap = ctx.workspace_nbytes // (factor * hidden * es)
    if native in (1, 3):
        cap = cap // ctx.world_size * ctx.world_size
    if cap <= 0:
        raise ValueError("allreduce workspace is too small for one row per rank")
    if normed_out is None:
        normed_out = torch.empty_like(x)
    if residual_out is None:
        residual_out = residual if residual is not None else torch.empty_like(x)
    for r0 in range(0, rows, cap):  # row chunks are independent calls
        r1 = min(rows, r0 + cap)
        nr = r1 - r0
        cur = native
        if cur in (1, 3) and nr % ctx.world_size != 0:
            cur = 0 if cur == 1 else 2
            if nr * hidden * es * _ws_factor(cur, ctx.world_size, True) > ctx.workspace_nbytes:
                raise ValueError("ragged tail does not fit the allreduce workspace")
        n_ctas = min(ctx.max_ctas, nr if cur in (0, 2) else max(1, nr // ctx.world_size))
        if max_sm > 0:
            n_ctas = min(n_ctas, max_sm)
        _lib.call("b200_allreduce", ctx.heap.ctx, ptr(x[r0:r1]), None, _lib.c_u64(nr * hidden), dtype_code(x.dtype), cur,
                  ptr(ctx.workspaces[0]), ptr(ctx.workspaces[1]), ptr(ctx.flags), ptr(ctx.sync), hidden,
                  ptr(residual[r0:r1]) if residual is not None else None, ptr(residual_out[r0:r1]), ptr(gamma),
                  ptr(normed_out[r0:r1]), c_float(eps), max(1, n_ctas), stream_ptr())
        ops._count()
    return normed_out, residual_out
