"""Device arrays for the host side: the mirror of ``CUDAnative.CuHostArray``.

Reference: src/array.jl of CUDAnative.jl -- ``CuHostArray{T,N}`` holds a device pointer and its
dims (:4-7), allocates on construction (:20-37), uploads / downloads with ``copyto!`` and
``Array(x)`` (:50-60) and converts to a raw device pointer for ``ccall`` (:15).  Arrays are dense
and column-major, as Julia's are (src/device/array.jl:104).

Memory comes from the library's own ``b200_malloc`` so the package works without PyTorch; a
``torch.Tensor`` on the device can be wrapped without copying through ``DevicePtr.of``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

Float16 = np.float16
Float32 = np.float32


class DevicePtr:
    """A typed device address: the mirror of ``DevicePtr{T,AS.Global}``
    (src/device/pointer.jl:46-50).  ``keep`` pins the owner of the memory."""

    __slots__ = ("dtype", "addr", "keep")

    def __init__(self, dtype, addr: int, keep=None):
        self.dtype = np.dtype(dtype)
        self.addr = int(addr)
        self.keep = keep

    def __add__(self, n_elements: int) -> "DevicePtr":
        return DevicePtr(self.dtype, self.addr + int(n_elements) * self.dtype.itemsize, self.keep)

    @staticmethod
    def of(obj) -> "DevicePtr":
        """Pointer to the first element of a CuHostArray or of a CUDA torch.Tensor."""
        if isinstance(obj, DevicePtr):
            return obj
        if isinstance(obj, CuHostArray):
            return DevicePtr(obj.dtype, obj.ptr, obj)
        if isinstance(getattr(obj, "ptr", None), DevicePtr):  # a converted kernel argument (execution.CuDeviceArray)
            return obj.ptr
        if hasattr(obj, "data_ptr") and hasattr(obj, "is_cuda"):
            if not obj.is_cuda:
                raise TypeError("expected a CUDA tensor")
            import torch

            table = {torch.float16: np.float16, torch.float32: np.float32}
            if obj.dtype not in table:
                raise TypeError(f"unsupported tensor dtype {obj.dtype}")
            return DevicePtr(table[obj.dtype], obj.data_ptr(), obj)
        raise TypeError(f"cannot take a device pointer of {type(obj).__name__}")


def pointer(obj) -> DevicePtr:
    """``pointer(a_dev)`` of the reference's kernels (examples/wmma/high-level.jl:33)."""
    return DevicePtr.of(obj)


class CuHostArray:
    """Owner of a dense column-major device array."""

    def __init__(self, source, dtype=None, shape=None):
        L = _lib.lib()
        if isinstance(source, np.ndarray):
            host = np.asfortranarray(source if dtype is None else source.astype(dtype))
            self.dtype = host.dtype
            self.shape = host.shape
        else:  # CuHostArray(dtype, shape): uninitialised, like Array{T}(undef, dims)
            host = None
            self.dtype = np.dtype(source if dtype is None else dtype)
            self.shape = tuple(shape)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        status = L.b200_malloc(C.byref(p), self.nbytes)
        if status == _lib.CUDA_ERROR and b"cudaErrorMemoryAllocation" in L.b200_last_error():
            # out of memory: let unreachable arrays release their device memory and try once more,
            # as the reference does (src/array.jl:23-29: Mem.alloc, on OOM GC.gc(), retry)
            import gc

            gc.collect()
            status = L.b200_malloc(C.byref(p), self.nbytes)
        _lib.check(status, "CuHostArray")
        self.ptr = p.value
        if host is not None and self.nbytes:
            _lib.check(L.b200_memcpy_h2d(self.ptr, host.ctypes.data, self.nbytes, None), "upload")
            _lib.check(L.b200_stream_sync(None), "upload")

    def __del__(self):
        try:
            if getattr(self, "ptr", None):
                _lib.lib().b200_free(self.ptr)
                self.ptr = None
        except Exception:
            pass

    @property
    def ld(self) -> int:
        return self.shape[0]

    def to_host(self) -> np.ndarray:
        """``Array(x_dev)``: synchronous download."""
        L = _lib.lib()
        out = np.empty(self.shape, dtype=self.dtype, order="F")
        if self.nbytes:
            _lib.check(L.b200_memcpy_d2h(out.ctypes.data, self.ptr, self.nbytes, None), "download")
            _lib.check(L.b200_stream_sync(None), "download")
        return out


def CuArray(host: np.ndarray) -> CuHostArray:
    return CuHostArray(host)


def Array(dev: CuHostArray) -> np.ndarray:
    return dev.to_host()


def similar(dev: CuHostArray, dtype=None, shape=None) -> CuHostArray:
    return CuHostArray(dev.dtype if dtype is None else dtype, shape=dev.shape if shape is None else shape)
