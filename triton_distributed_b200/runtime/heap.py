"""Symmetric heap of one node: the Python driver of ``csrc/runtime/symm_heap.cc``.

Each rank owns one physical allocation (CUDA VMM) and maps every peer's allocation into a single
virtual-address window, so a pointer into the local heap translates to a peer by adding a
per-rank base difference. When the GPUs sit behind an NVSwitch with multicast support the same
allocations are also bound to an NVLS multicast object (``multimem`` loads reduce over ranks,
stores broadcast). File descriptors of the allocations travel over abstract unix sockets;
the torch process group only carries small Python objects (socket names, verdicts).

Role in the reference: NVSHMEM initialised from the torch process group and the symmetric tensor
helpers (``python/triton_dist/utils.py:107-171``: ``init_nvshmem_by_torch_process_group``,
``nvshmem_create_tensor(s)``, ``nvshmem_free_tensor_sync``, ``nvshmem_barrier_all_on_stream``).

Fallbacks, chosen collectively so that all ranks end in the same mode:
  * file-descriptor export or exchange refused  -> cudaMalloc + CUDA IPC heap (no multicast);
  * multicast unsupported or any step of it fails on any rank -> heap without multicast.
"""
from __future__ import annotations

import ctypes
import math
import os
import secrets
from typing import Sequence

import torch
import torch.distributed as dist

from .. import _lib
from .dlpack import tensor_from_pointer


class SymmTimeoutError(RuntimeError):
    """A bounded device-side wait expired (lost signal, dead peer, mismatched call order)."""


class SymmHeapError(RuntimeError):
    pass


_STATUS_NAMES = {1: "flag wait timed out", 2: "barrier timed out", 3: "kernel pipeline wait timed out",
                 4: "bad kernel argument"}


def _all_agree(group, ok: bool) -> bool:
    if group is None or dist.get_world_size(group) == 1:
        return ok
    verdicts = [None] * dist.get_world_size(group)
    dist.all_gather_object(verdicts, bool(ok), group=group)
    return all(verdicts)


class SymmHeap:
    """One symmetric heap per process. Create through :func:`init_symm_heap`."""

    def __init__(self, group=None, size_bytes: int | None = None, use_multicast: bool | None = None,
                 timeout_ms: int | None = None):
        _lib.require_cuda()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 8:
            raise SymmHeapError("the symmetric heap spans one node of at most 8 GPUs")
        self.device = torch.cuda.current_device()
        if size_bytes is None:
            size_bytes = int(float(os.environ.get("B200DIST_HEAP_SIZE", 2 * 1024**3)))
        if use_multicast is None:
            use_multicast = os.environ.get("B200DIST_DISABLE_NVLS", "0") != "1"
        if timeout_ms is None:
            timeout_ms = int(os.environ.get("B200DIST_WAIT_TIMEOUT_MS", "10000"))
        self._lib = _lib.load()
        self._h = ctypes.c_void_p()
        self._tensors: dict[int, int] = {}  # data_ptr -> offset
        self.mode = "vmm"
        self.has_multicast = False

        force_ipc = os.environ.get("B200DIST_FORCE_IPC", "0") == "1"
        ok = False
        if not force_ipc:
            rc = self._lib.b200_heap_create(self.device, self.rank, self.world, ctypes.c_uint64(size_bytes),
                                            1 if use_multicast else 0, ctypes.byref(self._h))
            ok = rc == 0
            self._create_error = "" if ok else self._lib.b200_last_error().decode()
        if _all_agree(group, ok) and not force_ipc:
            ok = self._exchange_fds()
            if not _all_agree(group, ok):
                self._destroy_handle()
                ok = False
        elif ok:
            self._destroy_handle()
            ok = False
        if not ok:
            self.mode = "ipc"
            _lib.call("b200_heap_create_ipc", self.device, self.rank, self.world, ctypes.c_uint64(size_bytes),
                      ctypes.byref(self._h))
            self._exchange_ipc()
        elif use_multicast and self.world > 1:
            self.has_multicast = self._setup_multicast()
        self._lib.b200_heap_set_timeout_ms(self._h, ctypes.c_uint64(timeout_ms))
        self.bytes = int(self._lib.b200_heap_bytes(self._h))
        self._refresh_ctx()
        # 64 KiB of the heap is reserved for runtime flags (barrier epochs etc.)
        self._barrier_flags = self.create_tensor((64,), torch.int32)
        self._barrier_sync = torch.zeros(4, dtype=torch.int32, device="cuda")
        # The first device barrier also pays for every rank's first kernel launch out of the native library (module
        # load on a cold machine can take many seconds and differs between ranks): meet on the host first and give
        # this one barrier a generous budget, then restore the configured one.
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        self._lib.b200_heap_set_timeout_ms(self._h, ctypes.c_uint64(max(timeout_ms, 120000)))
        self._refresh_ctx()
        self.barrier_all()
        torch.cuda.synchronize()
        self._lib.b200_heap_set_timeout_ms(self._h, ctypes.c_uint64(timeout_ms))
        self._refresh_ctx()
        self.check_status("heap bootstrap barrier")

    # ------------------------------------------------------------------ bootstrap pieces
    def _sock_name(self, rank: int) -> bytes:
        return f"b200dist-{self._uid}-{rank}".encode()

    def _exchange_fds(self) -> bool:
        if self.world == 1:
            return True
        uid = [secrets.token_hex(8) if self.rank == 0 else None]
        dist.broadcast_object_list(uid, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)
        self._uid = uid[0]
        self._sock = ctypes.c_int(-1)
        rc = self._lib.b200_fd_socket_open(self._sock_name(self.rank), ctypes.byref(self._sock))
        if not _all_agree(self.group, rc == 0):
            return False
        ok = True
        fd = ctypes.c_int(-1)
        if self._lib.b200_heap_export_fd(self._h, ctypes.byref(fd)) != 0:
            ok = False
        if not _all_agree(self.group, ok):
            return False
        for k in range(1, self.world):
            peer = (self.rank + k) % self.world
            if self._lib.b200_fd_send(self._sock, self._sock_name(peer), fd, 0, self.rank) != 0:
                ok = False
        os.close(fd.value)
        for _ in range(self.world - 1):
            rfd, tag, aux = ctypes.c_int(-1), ctypes.c_int(0), ctypes.c_int(0)
            if self._lib.b200_fd_recv(self._sock, 20000, ctypes.byref(rfd), ctypes.byref(tag), ctypes.byref(aux)) != 0:
                ok = False
                break
            if tag.value != 0 or self._lib.b200_heap_import_fd(self._h, aux.value, rfd.value) != 0:
                ok = False
        return ok

    def _exchange_ipc(self) -> None:
        if self.world == 1:
            return
        handle = (ctypes.c_char * 64)()
        _lib.call("b200_heap_export_ipc", self._h, handle)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        for peer, hb in enumerate(handles):
            if peer != self.rank:
                _lib.call("b200_heap_import_ipc", self._h, peer, ctypes.create_string_buffer(hb, 64))

    def _setup_multicast(self) -> bool:
        if not _all_agree(self.group, bool(self._lib.b200_heap_multicast_supported(self._h))):
            return False
        ok = True
        if self.rank == 0:
            fd = ctypes.c_int(-1)
            ok = self._lib.b200_heap_mc_create(self._h, ctypes.byref(fd)) == 0
            if ok:
                for peer in range(1, self.world):
                    ok = ok and self._lib.b200_fd_send(self._sock, self._sock_name(peer), fd, 1, 0) == 0
                os.close(fd.value)
        created = [ok]
        dist.broadcast_object_list(created, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                                   group=self.group)
        if not created[0]:
            return False
        if self.rank != 0:
            rfd, tag, aux = ctypes.c_int(-1), ctypes.c_int(0), ctypes.c_int(0)
            ok = self._lib.b200_fd_recv(self._sock, 20000, ctypes.byref(rfd), ctypes.byref(tag), ctypes.byref(aux)) == 0
            ok = ok and tag.value == 1 and self._lib.b200_heap_mc_import(self._h, rfd.value) == 0
        ok = ok and self._lib.b200_heap_mc_add_device(self._h) == 0
        if not _all_agree(self.group, ok):  # doubles as the "all devices added" barrier
            self._lib.b200_heap_mc_release(self._h)
            return False
        ok = self._lib.b200_heap_mc_bind(self._h) == 0
        if not _all_agree(self.group, ok):
            self._lib.b200_heap_mc_release(self._h)
            return False
        return True

    def _refresh_ctx(self) -> None:
        n = self._lib.b200_symm_ctx_size()
        self._ctx_buf = ctypes.create_string_buffer(n)
        _lib.call("b200_heap_get_ctx", self._h, self._ctx_buf)
        self.base = [int(self._lib.b200_heap_base(self._h, k)) for k in range(self.world)]
        self.mc_base = int(self._lib.b200_heap_mc_base(self._h))

    @property
    def ctx(self) -> ctypes.Array:
        """The by-value kernel argument (``b200::SymmCtx``) as a ctypes buffer."""
        return self._ctx_buf

    def set_timeout_ms(self, ms: int) -> None:
        self._lib.b200_heap_set_timeout_ms(self._h, ctypes.c_uint64(ms))
        self._refresh_ctx()

    # ------------------------------------------------------------------ tensors
    def create_tensor(self, shape: Sequence[int] | int, dtype: torch.dtype, align: int = 256,
                      sync: bool = True) -> torch.Tensor:
        """Allocate a zero-filled symmetric tensor. Collective: every rank must issue the same sequence of
        create/free calls so that offsets agree. With ``sync`` (default) a device barrier is enqueued behind the
        zero-fill on the current stream, so that work enqueued after this call can never have its remote writes
        wiped by a slower peer's zero-fill (the role of the barrier inside ``nvshmem_malloc``)."""
        if isinstance(shape, int):
            shape = (shape,)
        nbytes = max(1, math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        off = ctypes.c_uint64(0)
        rc = self._lib.b200_heap_alloc(self._h, ctypes.c_uint64(nbytes), ctypes.c_uint64(align), ctypes.byref(off))
        if rc != 0:
            raise SymmHeapError(self._lib.b200_last_error().decode())
        t = tensor_from_pointer(self.base[self.rank] + off.value, nbytes, self.device).view(dtype)
        t = t[: math.prod(shape)].view(*shape)
        t.zero_()
        self._tensors[t.data_ptr()] = off.value
        if sync and self.world > 1 and getattr(self, "_barrier_flags", None) is not None:
            self.barrier_all()
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base[self.rank]
        if not (0 <= off < self.bytes):
            raise SymmHeapError("tensor does not live in the local symmetric heap")
        return off

    def is_symmetric(self, t: torch.Tensor) -> bool:
        return t.is_cuda and 0 <= t.data_ptr() - self.base[self.rank] < self.bytes

    def peer_tensor(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        """View of `t`'s counterpart on `peer` (same shape/stride), addressed through the peer mapping.
        Only element-wise torch ops and copies may touch it; library GEMM/attention kernels must not."""
        if peer == self.rank:
            return t
        off = self.offset_of(t)
        nbytes = t.untyped_storage().nbytes() - (t.data_ptr() - t.untyped_storage().data_ptr())
        span = (sum((s - 1) * st for s, st in zip(t.shape, t.stride())) + 1) * t.element_size() if t.numel() else 0
        nbytes = min(nbytes, span) if span else nbytes
        raw = tensor_from_pointer(self.base[peer] + off, max(nbytes, t.element_size()), self.device).view(t.dtype)
        return raw.as_strided(t.shape, t.stride())

    def create_tensors(self, shape, dtype) -> list[torch.Tensor]:
        """Allocate symmetrically and return the views of all ranks (index = rank; own = local tensor)."""
        t = self.create_tensor(shape, dtype)
        return [self.peer_tensor(t, k) for k in range(self.world)]

    def multicast_tensor(self, t: torch.Tensor) -> torch.Tensor:
        if not self.has_multicast:
            raise SymmHeapError("no NVLS multicast mapping on this heap")
        off = self.offset_of(t)
        raw = tensor_from_pointer(self.mc_base + off, t.numel() * t.element_size(), self.device).view(t.dtype)
        return raw.view(t.shape)

    def free(self, t: torch.Tensor) -> None:
        off = self._tensors.pop(t.data_ptr(), None)
        if off is None:
            raise SymmHeapError("not a tensor returned by create_tensor (or already freed)")
        _lib.call("b200_heap_free", self._h, ctypes.c_uint64(off))

    def live_bytes(self) -> int:
        return int(self._lib.b200_heap_live_bytes(self._h))

    # ------------------------------------------------------------------ sync + status
    def barrier_all(self, stream: torch.cuda.Stream | None = None) -> None:
        """Cross-rank barrier enqueued on `stream`: kernels of all ranks enqueued before it have
        finished (and their stores are visible system-wide) before anything enqueued after it runs."""
        _lib.call("b200_barrier_all", self._ctx_buf, _lib.ptr(self._barrier_flags), _lib.ptr(self._barrier_sync),
                  _lib.stream_ptr(stream))

    def status(self) -> list[int]:
        out = (ctypes.c_uint32 * 16)()
        self._lib.b200_heap_status(self._h, out)
        return list(out)

    def check_status(self, what: str = "") -> None:
        """Raise if any kernel of this rank recorded an expired wait since the last clear."""
        st = self.status()
        if st[0] != 0:
            self._lib.b200_heap_status_clear(self._h)
            raise SymmTimeoutError(
                f"{what or 'kernel'}: {_STATUS_NAMES.get(st[0], f'status {st[0]}')} on rank {self.rank} "
                f"(who={st[1]}, expected={st[2]}, seen={st[3]}, line={st[4]})")

    def sync_and_check(self, what: str = "") -> None:
        """Wait for this device's work, then raise if one of its kernels gave up on a wait. Contexts call this when
        they are finalised, so an expired wait cannot pass unnoticed even if the caller never looks at the status."""
        torch.cuda.synchronize()
        self.check_status(what)

    # ------------------------------------------------------------------ teardown
    def _destroy_handle(self) -> None:
        if self._h:
            self._lib.b200_heap_destroy(self._h)
            self._h = ctypes.c_void_p()

    def finalize(self) -> None:
        if not self._h:
            return
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        if getattr(self, "_sock", None) is not None and self._sock.value >= 0:
            self._lib.b200_fd_socket_close(self._sock)
            self._sock = ctypes.c_int(-1)
        self._tensors.clear()
        self._destroy_handle()


_HEAP: SymmHeap | None = None


def init_symm_heap(group=None, size_bytes: int | None = None, **kw) -> SymmHeap:
    global _HEAP
    if _HEAP is None:
        _HEAP = SymmHeap(group, size_bytes, **kw)
    return _HEAP


def get_heap() -> SymmHeap:
    if _HEAP is None:
        raise SymmHeapError("symmetric heap not initialised; call initialize_distributed() first")
    return _HEAP


def heap_initialized() -> bool:
    return _HEAP is not None


def finalize_symm_heap() -> None:
    global _HEAP
    if _HEAP is not None:
        _HEAP.finalize()
        _HEAP = None
