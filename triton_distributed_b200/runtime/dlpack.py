"""Wrap a raw device address as a torch tensor without copying and without asking the driver who
owns the address.

Peer mappings of the symmetric heap are addresses of *this* process that resolve to another GPU's
memory. ``__cuda_array_interface__`` import would query the pointer's owner and label the tensor
with the peer's device index; a hand-built DLPack capsule lets us state the device ourselves, so
peer views behave like ordinary tensors of the current device for copies and element-wise ops.

Role in the reference: ``nvshmem.core.tensor`` / ``get_peer_tensor`` (``python/triton_dist/utils.py:122-144``).
"""
from __future__ import annotations

import ctypes

import torch

_kDLCUDA = 2
_kDLUInt = 1


class _DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class _DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class _DLTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("device", _DLDevice),
        ("ndim", ctypes.c_int32),
        ("dtype", _DLDataType),
        ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
        ("byte_offset", ctypes.c_uint64),
    ]


class _DLManagedTensor(ctypes.Structure):
    pass


_DELETER = ctypes.CFUNCTYPE(None, ctypes.POINTER(_DLManagedTensor))
_DLManagedTensor._fields_ = [("dl_tensor", _DLTensor), ("manager_ctx", ctypes.c_void_p), ("deleter", _DELETER)]

# Keeps the ctypes objects of every exported tensor alive until torch calls the deleter.
_live: dict[int, tuple] = {}


@_DELETER
def _deleter(managed_ptr):
    _live.pop(ctypes.addressof(managed_ptr.contents), None)


_PyCapsule_New = ctypes.pythonapi.PyCapsule_New
_PyCapsule_New.restype = ctypes.py_object
_PyCapsule_New.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]


def tensor_from_pointer(address: int, nbytes: int, device_index: int) -> torch.Tensor:
    """Return a 1-D ``torch.uint8`` CUDA tensor of `nbytes` bytes that aliases `address`.

    The memory is not owned: the caller (the symmetric heap) keeps it mapped for the tensor's lifetime.
    """
    shape = (ctypes.c_int64 * 1)(nbytes)
    managed = _DLManagedTensor()
    managed.dl_tensor.data = ctypes.c_void_p(address)
    managed.dl_tensor.device = _DLDevice(_kDLCUDA, device_index)
    managed.dl_tensor.ndim = 1
    managed.dl_tensor.dtype = _DLDataType(_kDLUInt, 8, 1)
    managed.dl_tensor.shape = ctypes.cast(shape, ctypes.POINTER(ctypes.c_int64))
    managed.dl_tensor.strides = None
    managed.dl_tensor.byte_offset = 0
    managed.manager_ctx = None
    managed.deleter = _deleter
    _live[ctypes.addressof(managed)] = (managed, shape)
    capsule = _PyCapsule_New(ctypes.addressof(managed), b"dltensor", None)
    return torch.from_dlpack(capsule)
