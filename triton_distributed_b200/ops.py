"""Single-GPU hot ops backed by the sm_100a kernels in ``csrc/kernels``.

Every function here launches native code on the current CUDA stream and fails loudly when the
native library or a GPU is missing: there is no silent PyTorch fallback (the CPU reference
semantics live in :mod:`triton_distributed_b200.ref`).

Replaces in the reference: cuBLAS ``F.linear``, ``flashinfer.norm.rmsnorm``,
``flashinfer.apply_rope_with_cos_sin_cache_inplace``, ``act_fn(gate) * up`` and the softmax/topk router
(``layers/nvidia/tp_mlp.py:159-186``, ``tp_attn.py:60-75,159-195``, ``kernels/nvidia/moe_reduce_rs.py:172-189``).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import c_float, dtype_code, ptr, stream_ptr

# number of native kernel launches issued through this module (bench.py reports it)
launch_count = 0


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _check_2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D tensor with unit inner stride, got shape {tuple(t.shape)} stride {t.stride()}")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[N,K].T`` on the persistent tcgen05 kernel (128x256x64 tiles, fp32 accumulation)."""
    _lib.require_cuda()
    _check_2d(a, "a"), _check_2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K or a.dtype != b.dtype:
        raise ValueError("gemm: shape/dtype mismatch")
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    _lib.call("b200_gemm", ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
              dtype_code(a.dtype), max_ctas, stream_ptr())
    _count()
    return out


class _SkinnyScratch:
    """Per-device split-K scratch shared by all skinny GEMM calls of a stream (each call re-zeroes it)."""

    def __init__(self):
        self.bufs: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    def get(self, device: torch.device, floats: int, tiles: int):
        key = device.index if device.index is not None else torch.cuda.current_device()
        cur = self.bufs.get(key)
        if cur is None or cur[0].numel() < floats or cur[1].numel() < tiles:
            if cur is not None:
                torch.cuda.synchronize()
            nf = max(floats, 4 << 20, 0 if cur is None else cur[0].numel())
            nt = max(tiles, 4096, 0 if cur is None else cur[1].numel())
            cur = (torch.zeros(nf, dtype=torch.float32, device=device), torch.zeros(nt, dtype=torch.int32, device=device))
            self.bufs[key] = cur
        return cur


_skinny_scratch = _SkinnyScratch()


def reserve_skinny_scratch(device, floats: int, tiles: int) -> None:
    """Pre-size the split-K scratch (call before CUDA-graph capture so no allocation happens inside)."""
    _skinny_scratch.get(torch.device(device), floats, tiles)


class SkinnyEpilogue(ctypes.Structure):
    """Mirror of ``b200::SkinnyEpilogue`` (csrc/kernels/gemm_skinny_sm100.cu): what the decode GEMM does with a
    finished tile besides storing it. Build one with ``skinny_row_scale``, ``skinny_qkv_heads`` or ``skinny_residual``."""
    _fields_ = [("kind", ctypes.c_int), ("sumsq_in", ctypes.c_void_p), ("scale_dim", ctypes.c_float), ("eps", ctypes.c_float),
                ("Hq", ctypes.c_int), ("Hkv", ctypes.c_int), ("positions", ctypes.c_void_p), ("slots", ctypes.c_void_p),
                ("cos_sin", ctypes.c_void_p), ("q_gamma", ctypes.c_void_p), ("k_gamma", ctypes.c_void_p),
                ("q_out", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("head_eps", ctypes.c_float), ("residual_in", ctypes.c_void_p), ("residual_out", ctypes.c_void_p),
                ("next_gamma", ctypes.c_void_p), ("scaled_out", ctypes.c_void_p), ("sumsq_out", ctypes.c_void_p)]

    def __init__(self, **kw):
        super().__init__()
        self._keep = []  # tensors referenced by raw pointers stay alive as long as the description does
        for k, v in kw.items():
            if isinstance(v, torch.Tensor):
                self._keep.append(v)
                v = v.data_ptr()
            setattr(self, k, v)


def _dptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def skinny_row_scale(sumsq: torch.Tensor, dim: int, eps: float, base: SkinnyEpilogue | None = None) -> SkinnyEpilogue:
    """Epilogue ``out[m, :] *= rsqrt(sumsq[m] / dim + eps)``: the RMSNorm of the GEMM's input when its producer already
    applied the gain. `sumsq` fp32 [>= M]. Combines with another epilogue when `base` is given."""
    ep = base if base is not None else SkinnyEpilogue(kind=0)
    ep.sumsq_in, ep.scale_dim, ep.eps = sumsq.data_ptr(), float(dim), float(eps)
    ep._keep.append(sumsq)
    return ep


def skinny_qkv_heads(positions: torch.Tensor, slots: torch.Tensor | None, cos_sin: torch.Tensor, num_q_heads: int,
                     num_kv_heads: int, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     q_gamma: torch.Tensor | None, k_gamma: torch.Tensor | None, eps: float) -> SkinnyEpilogue:
    """Epilogue of the fused qkv projection (head dim 128): per-head RMSNorm of q / k, neox RoPE, q to ``q_out``
    [M, Hq, 128] and k / v into the caches viewed as [slots, Hkv, 128] at ``slots`` (int64 [M], None = identity)."""
    if positions.dtype != torch.int32 or cos_sin.dtype != torch.float32 or (slots is not None and slots.dtype != torch.int64):
        raise ValueError("positions must be int32, slots int64 and cos_sin float32")
    ep = SkinnyEpilogue(kind=1, Hq=num_q_heads, Hkv=num_kv_heads, positions=positions, cos_sin=cos_sin, q_out=q_out,
                        k_cache=k_cache, v_cache=v_cache, head_eps=float(eps))
    for name, t in (("slots", slots), ("q_gamma", q_gamma), ("k_gamma", k_gamma)):
        if t is not None:
            setattr(ep, name, t.data_ptr())
            ep._keep.append(t)
    return ep


def skinny_residual(residual: torch.Tensor, sumsq_out: torch.Tensor | None, next_gamma: torch.Tensor | None = None,
                    scaled_out: torch.Tensor | None = None, residual_out: torch.Tensor | None = None) -> SkinnyEpilogue:
    """Epilogue ``h = out + residual``: writes h to ``residual_out`` (default: in place), ``h * next_gamma`` to
    ``scaled_out`` and adds ``sum(h^2)`` per token to ``sumsq_out`` (fp32, zeroed by the caller once per step)."""
    ro = residual if residual_out is None else residual_out
    ep = SkinnyEpilogue(kind=2, residual_in=residual, residual_out=ro)
    for name, t in (("sumsq_out", sumsq_out), ("next_gamma", next_gamma), ("scaled_out", scaled_out)):
        if t is not None:
            setattr(ep, name, t.data_ptr())
            ep._keep.append(t)
    return ep


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, swiglu: bool = False,
                splits: int = 0, epilogue: SkinnyEpilogue | None = None) -> torch.Tensor | None:
    """Decode GEMM for ``M <= 256`` tokens: ``x[M,K] @ w[N,K].T`` with the weights streamed once.

    With ``swiglu=True``, ``w`` is ``[gate; up]`` (2*I rows) and the result is ``silu(x gate^T) * (x up^T)`` [M, I].
    With ``epilogue`` (M <= 16) the finished tiles go through a fused epilogue instead of (or before) the plain store;
    the qkv-heads and residual kinds write their own outputs and return None unless ``out`` is given. The models do
    not use the epilogues: a decode step chained through them (5 launches per layer instead of 9) measured 15.6 ms
    against 13.8 ms on one B200 (Qwen3-32B, batch 8), because the epilogue runs on the one CTA that finishes each tile,
    on the critical path, while the separate small kernels spread over the machine and start early under programmatic
    dependent launch. They remain available for callers whose chain is launch-bound (no PDL, no graph).
    """
    _lib.require_cuda()
    _check_2d(x, "x"), _check_2d(w, "w")
    M, K = x.shape
    n_rows = w.shape[0]
    N = n_rows // 2 if swiglu else n_rows
    own_output = epilogue is not None and epilogue.kind in (1, 2)
    if out is None and not own_output:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    lib.b200_gemm_skinny_scratch_floats.restype = ctypes.c_longlong
    floats = lib.b200_gemm_skinny_scratch_floats(M, N, 1 if swiglu else 0)
    tiles = (N + 127) // 128
    scratch, tickets = _skinny_scratch.get(x.device, floats, tiles)
    ldc = out.stride(0) if out is not None else (epilogue._keep[0].stride(0) if epilogue.kind == 2 else N)
    if epilogue is None:
        _lib.call("b200_gemm_skinny", ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0), w.stride(0), ldc,
                  1 if swiglu else 0, dtype_code(x.dtype), ptr(scratch), ptr(tickets), splits, stream_ptr())
    else:
        if ctypes.sizeof(SkinnyEpilogue) != lib.b200_gemm_skinny_epilogue_bytes():
            raise RuntimeError("SkinnyEpilogue layout differs between the Python binding and the native library")
        _lib.call("b200_gemm_skinny_fused", ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0), w.stride(0), ldc,
                  1 if swiglu else 0, dtype_code(x.dtype), ptr(scratch), ptr(tickets), ctypes.byref(epilogue), stream_ptr())
    _count()
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T`` for any leading shape, routed to the skinny kernel for <= 256 rows, else the tiled one."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    o2 = out.reshape(-1, w.shape[0]) if out is not None else None
    y = gemm_skinny(x2, w, o2) if x2.shape[0] <= 256 else gemm(x2, w, o2)
    return y.reshape(*lead, w.shape[0])


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm over the last dim. With `residual`, computes ``residual += x`` in place first and normalises the sum.

    ``gamma`` is treated as a weight: the kernel fetches it before it waits for the kernel launched just before it
    (programmatic dependent launch), so it must not be an output of that kernel. The same holds for the gains of
    ``qk_norm_rope`` and of the fused all-reduce + RMSNorm."""
    _lib.require_cuda()
    hidden = x.shape[-1]
    x2 = x.reshape(-1, hidden)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, hidden)
    r2 = residual.reshape(-1, hidden) if residual is not None else None
    _lib.call("b200_rmsnorm", ptr(x2), ptr(r2), ptr(r2), ptr(gamma), ptr(o2), x2.shape[0], hidden, c_float(eps),
              dtype_code(x.dtype), stream_ptr())
    _count()
    return o2.reshape(x.shape)


def qk_norm_rope(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, num_q_heads: int,
                 num_kv_heads: int, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor | None,
                 q_gamma: torch.Tensor | None, k_gamma: torch.Tensor | None, eps: float = 1e-6,
                 q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-head RMSNorm of q/k, neox RoPE, and the write of k/v into the KV cache at `slots`, in one kernel.

    qkv: [T, (Hq + 2 Hkv) * 128]; positions: int32 [T]; cos_sin: fp32 [max_pos, 128] (cos | sin);
    caches: [num_slots, Hkv, 128] (any view whose first dim is the slot); slots: int64 [T] (None = identity).
    Returns q [T, Hq, 128].
    """
    _lib.require_cuda()
    T = qkv.shape[0]
    D = 128
    if qkv.shape[1] != (num_q_heads + 2 * num_kv_heads) * D or not qkv.is_contiguous():
        raise ValueError("qkv must be contiguous [T, (Hq + 2*Hkv) * 128]")
    if positions.dtype != torch.int32 or cos_sin.dtype != torch.float32:
        raise ValueError("positions must be int32 and cos_sin float32")
    if q_out is None:
        q_out = torch.empty((T, num_q_heads, D), dtype=qkv.dtype, device=qkv.device)
    _lib.call("b200_qk_norm_rope", ptr(qkv), ptr(positions), ptr(slots), ptr(q_gamma), ptr(k_gamma), ptr(cos_sin),
              ptr(q_out), ptr(k_cache), ptr(v_cache), T, num_q_heads, num_kv_heads, D, c_float(eps),
              dtype_code(qkv.dtype), stream_ptr())
    _count()
    return q_out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None, gamma: torch.Tensor | None = None,
              scaled_out: torch.Tensor | None = None, sumsq_out: torch.Tensor | None = None) -> torch.Tensor:
    """``table[ids]`` for int64 ids of any shape -> [*ids.shape, H] (ids outside the table give zero rows).

    For a following RMSNorm folded into the consumer GEMM: ``sumsq_out`` (fp32 [T]) receives every row's sum of
    squares and ``scaled_out`` ([T, H]) the row times ``gamma``."""
    _lib.require_cuda()
    if not table.is_contiguous() or table.dim() != 2:
        raise ValueError("embedding table must be a contiguous [V, H] tensor")
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    V, H = table.shape
    if out is None:
        out = torch.empty((flat.numel(), H), dtype=table.dtype, device=table.device)
    _lib.call("b200_embedding", ptr(flat), ptr(table), ptr(out), flat.numel(), ctypes.c_longlong(V), H, dtype_code(table.dtype),
              ptr(gamma), ptr(scaled_out), ptr(sumsq_out), stream_ptr())
    _count()
    return out.reshape(*ids.shape, H)


def silu_mul(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(x[..., :I]) * x[..., I:]`` for the fused [gate | up] projection."""
    _lib.require_cuda()
    inter = x.shape[-1] // 2
    x2 = x.reshape(-1, x.shape[-1])
    _check_2d(x2, "x")
    if out is None:
        out = torch.empty((x2.shape[0], inter), dtype=x.dtype, device=x.device)
    _lib.call("b200_silu_mul", ptr(x2), ptr(out), x2.shape[0], inter, x2.stride(0), dtype_code(x.dtype), stream_ptr())
    _count()
    return out.reshape(*x.shape[:-1], inter)


def silu_mul_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """SwiGLU gate fused with block quantisation: x [T, 2 * I] (gate | up, I % 128 == 0) -> (e4m3 [T, I], fp32 scales
    [T, I / 128]) with scale = amax / 448 per 128 channels, the activation format of ``grouped_gemm_fp8``."""
    _lib.require_cuda()
    x2 = x.reshape(-1, x.shape[-1])
    _check_2d(x2, "x")
    inter = x2.shape[1] // 2
    out8 = torch.empty((x2.shape[0], inter), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty((x2.shape[0], inter // 128), dtype=torch.float32, device=x.device)
    _lib.call("b200_silu_mul_fp8", ptr(x2), ptr(out8), ptr(scale), x2.shape[0], inter, x2.stride(0), dtype_code(x.dtype),
              stream_ptr())
    _count()
    return out8, scale


def topk_softmax(logits: torch.Tensor, k: int, renormalize: bool = False):
    """Router: softmax over experts then top-k. Returns (ids int32 [T,k], weights fp32 [T,k])."""
    _lib.require_cuda()
    T, E = logits.shape
    logits = logits.contiguous()
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    _lib.call("b200_topk_softmax", ptr(logits), dtype_code(logits.dtype), T, E, k, ptr(ids), ptr(w),
              1 if renormalize else 0, stream_ptr())
    _count()
    return ids, w


def top_p_sample(logits: torch.Tensor, temperature: float, top_p: float, uniform: torch.Tensor | None = None) -> torch.Tensor:
    """Nucleus sampling without a sort. logits fp32 [B, V]; returns int64 token ids [B, 1]."""
    _lib.require_cuda()
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        logits = logits.float().contiguous()
    B, V = logits.shape
    if uniform is None:
        uniform = torch.rand(B, dtype=torch.float32, device=logits.device)
    out = torch.empty((B, 1), dtype=torch.int64, device=logits.device)
    _lib.call("b200_top_p_sample", ptr(logits), logits.stride(0), B, V, c_float(temperature), c_float(top_p),
              ptr(uniform), ptr(out), stream_ptr())
    _count()
    return out


_attn_tickets: dict = {}


def choose_kv_splits(batch: int, num_kv_heads: int, group: int, max_kv_len: int, sm_count: int = 148) -> int:
    """Split count for the decode kernel: one wave of CTAs at two per SM (the per-warp-ring kernel keeps 96 KB of
    shared memory per CTA) and at least 128 tokens (two 64-token tiles) per split. With few (batch, KV head) groups,
    as under tensor parallelism, the kernel is bound by the latency of its serial tile loop, not by bytes: measured on
    the per-rank shapes of an 8-way split (batch 8, one KV head, 2 K tokens) 16 splits beat 4 by 0.42 ms per 64-layer
    step. ``B200DIST_KV_SPLITS`` forces a value (for experiments)."""
    forced = os.environ.get("B200DIST_KV_SPLITS")
    if forced:
        return max(1, int(forced))
    ctas = batch * num_kv_heads * ((group + 15) // 16)
    by_machine = max(1, (2 * sm_count) // max(ctas, 1))
    by_len = max(1, max_kv_len // 128)
    return int(max(1, min(by_machine, by_len, 64)))


# measured on the end-to-end decode step (one GPU, CUDA graph): the in-kernel merge costs 0.3 ms per step more than the
# separate combine launch, whose start overlaps the split kernel under programmatic dependent launch
_FUSED_COMBINE_DEFAULT = os.environ.get("B200DIST_ATTN_FUSED_COMBINE", "0") == "1"


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_lens: torch.Tensor,
                     block_table: torch.Tensor, scale: float, soft_cap: float = 0.0, num_splits: int = 1,
                     out: torch.Tensor | None = None, return_lse: bool = False, workspace: dict | None = None,
                     fused_combine: bool | None = None, ring: int = -1):
    """Paged GQA decode attention. q [B,Hq,128]; caches [num_blocks, page, Hkv, 128]; kv_lens int32 [B];
    block_table int32 [B, max_blocks]. Returns out [B,Hq,128] (and natural-log LSE fp32 [B,Hq]).

    With ``num_splits > 1`` the last CTA of every (batch, head group) merges the split partials inside the same
    launch (``fused_combine=False`` runs the separate combine kernel instead). ``ring`` selects the K/V pipeline:
    0 = two-stage CTA-wide, 3 / 6 = per-warp rings of that depth, -1 = the library default."""
    _lib.require_cuda()
    B, Hq, D = q.shape
    page, Hkv = k_cache.shape[1], k_cache.shape[2]
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous() and block_table.stride(1) == 1):
        raise ValueError("decode_attention needs contiguous q / caches and a row-major block table")
    if out is None:
        out = torch.empty_like(q)
    if fused_combine is None:
        fused_combine = _FUSED_COMBINE_DEFAULT
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if return_lse else None
    tickets = None
    if num_splits > 1:
        if workspace is not None and "o_part" in workspace and workspace["o_part"].numel() >= B * Hq * num_splits * D:
            o_part, lse_part = workspace["o_part"], workspace["lse_part"]
        else:
            o_part = torch.empty(B * Hq * num_splits * D, dtype=torch.float32, device=q.device)
            lse_part = torch.empty(B * Hq * num_splits, dtype=torch.float32, device=q.device)
            if workspace is not None:
                workspace["o_part"], workspace["lse_part"] = o_part, lse_part
        if fused_combine:
            n_groups = B * Hkv * ((Hq // Hkv + 15) // 16)
            holder = workspace if workspace is not None else _attn_tickets.setdefault(q.device, {})
            tickets = holder.get("tickets")
            if tickets is None or tickets.numel() < n_groups or tickets.device != q.device:
                tickets = torch.zeros(max(n_groups, 1024), dtype=torch.int32, device=q.device)
                holder["tickets"] = tickets
    else:
        o_part = lse_part = None
    _lib.call("b200_decode_attn", ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.stride(0),
              ptr(kv_lens), B, Hq, Hkv, D, page, c_float(scale), c_float(soft_cap), num_splits, ptr(o_part),
              ptr(lse_part), ptr(tickets), ptr(out), ptr(lse), dtype_code(q.dtype), ring, stream_ptr())
    _count()
    if num_splits > 1 and tickets is None:
        _lib.call("b200_decode_combine", ptr(o_part), ptr(lse_part), ctypes.c_longlong(num_splits * D),
                  ctypes.c_longlong(D), ctypes.c_longlong(num_splits), ctypes.c_longlong(1), B * Hq, num_splits,
                  ptr(out), None, ptr(lse), dtype_code(q.dtype), stream_ptr())
        _count()
    return (out, lse) if return_lse else out


_pipe_status: dict = {}


def _pipeline_status(device: torch.device) -> torch.Tensor:
    """One int32 word per device that single-GPU pipeline kernels raise when an internal wait expires."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _pipe_status.get(key)
    if st is None:
        st = _pipe_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return st


def check_pipeline_status(device=None) -> None:
    """Synchronise and raise if a pipeline kernel of this device gave up on an internal wait since the last check."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _pipe_status.get(key)
    if st is None:
        return
    code = int(st.item())
    if code != 0:
        st.zero_()
        raise RuntimeError(f"a pipeline kernel on {dev} gave up on an internal wait (status {code}); its output is incomplete")


def prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                      cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, scale: float,
                      causal: bool = True, out: torch.Tensor | None = None,
                      seqlens_k: torch.Tensor | None = None) -> torch.Tensor:
    """Variable-length attention on the tcgen05 prefill kernel. q [total_q, Hq, 128]; k, v [total_k, Hkv, 128];
    cu_seqlens_* int32 [B + 1] on the device. With ``causal`` query i of a sequence attends keys <= i + (k_len - q_len).

    Packed sequences: leave ``seqlens_k`` None (lengths are differences of ``cu_seqlens_k``). Keys in place: give
    ``seqlens_k`` int32 [B]; sequence b then reads rows ``cu_seqlens_k[b] ... + seqlens_k[b]`` of k / v, which may be the
    slot view of a paged KV cache whose sequences own contiguous runs of slots. Returns [total_q, Hq, 128]."""
    _lib.require_cuda()
    total_q, Hq, D = q.shape
    total_k, Hkv, _ = k.shape
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()) or k.shape != v.shape or D != 128:
        raise ValueError("prefill_attention needs contiguous q / k / v with head dim 128")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("prefill_attention handles bf16 / f16")
    B = cu_seqlens_q.numel() - 1
    cu_q = cu_seqlens_q.to(device=q.device, dtype=torch.int32).contiguous()
    cu_k = cu_seqlens_k.to(device=q.device, dtype=torch.int32).contiguous()
    k_lens = seqlens_k.to(device=q.device, dtype=torch.int32).contiguous() if seqlens_k is not None else None
    lib = _lib.load()
    lib.b200_prefill_attention_scratch_bytes.restype = ctypes.c_longlong
    nbytes = int(lib.b200_prefill_attention_scratch_bytes(B, Hkv, int(max_seqlen_k)))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    if out is None:
        out = torch.empty_like(q)
    _lib.call("b200_prefill_attention", ptr(q), ptr(k), ptr(v), ptr(cu_q), ptr(cu_k), ptr(k_lens), B, total_q, total_k,
              int(max_seqlen_q), int(max_seqlen_k), Hq, Hkv, D, c_float(scale), 1 if causal else 0, ptr(scratch), ptr(out),
              dtype_code(q.dtype), ptr(_pipeline_status(q.device)), stream_ptr())
    _count(2)
    return out


def combine_partials(o_part: torch.Tensor, lse_part: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Merge attention partials over dim 0: o_part fp32 [R, BH, 128], lse_part fp32 [R, BH] -> [BH, 128]."""
    _lib.require_cuda()
    R, BH, D = o_part.shape
    out = torch.empty((BH, D), dtype=out_dtype, device=o_part.device)
    _lib.call("b200_decode_combine", ptr(o_part), ptr(lse_part), ctypes.c_longlong(o_part.stride(1)),
              ctypes.c_longlong(o_part.stride(0)), ctypes.c_longlong(lse_part.stride(1)),
              ctypes.c_longlong(lse_part.stride(0)), BH, R, ptr(out), None, None, dtype_code(out_dtype), stream_ptr())
    _count()
    return out
