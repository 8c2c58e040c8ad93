"""Device buffers shared between PROCESSES of one node through CUDA IPC.

``SymmetricBuffer`` (symm.py) serves ranks of one process group that all allocate the same size. The
disaggregated weight push is asymmetric: sampler processes own parameter buffers, trainer processes only need
to store into them. ``IpcBuffer`` is that one-sided form: the owner allocates with the native library
(``csrc/ipc.cu``; plain ``cudaMalloc``, because blocks of PyTorch's caching allocator cannot be exported),
wraps the memory as a tensor and hands out a 64-byte handle; any other process on the node turns the handle
into a device pointer (``open_handle``) that its kernels may store through over NVLink.
"""
from __future__ import annotations

import ctypes

import torch

_ITEM = {torch.bfloat16: ("<u2", torch.uint16), torch.float16: ("<u2", torch.uint16), torch.float32: ("<f4", torch.float32),
         torch.uint8: ("|u1", torch.uint8), torch.int32: ("<i4", torch.int32)}


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can alias memory it did not allocate."""

    def __init__(self, ptr: int, numel: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


class IpcBuffer:
    """``numel`` elements of ``dtype`` on ``device``, exportable to other processes of the node."""

    def __init__(self, numel: int, dtype: torch.dtype, device):
        from ..ops import _common as C
        self.device = torch.device(device)
        self.numel, self.dtype = int(numel), dtype
        typestr, carrier = _ITEM[dtype]
        nbytes = self.numel * torch.empty(0, dtype=dtype).element_size()
        nbytes = (nbytes + 255) // 256 * 256
        out = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            rc = C.lib().axb_ipc_alloc(ctypes.c_longlong(nbytes), ctypes.byref(out))
        if rc != 0 or not out.value:
            raise RuntimeError(f"axb_ipc_alloc({nbytes} bytes) failed with {rc}")
        self.ptr = int(out.value)
        self._keep = _RawCuda(self.ptr, self.numel, typestr)
        base = torch.as_tensor(self._keep, device=self.device)
        self.tensor = base.view(dtype) if carrier != dtype else base
        self._lib = C.lib()

    def handle(self) -> bytes:
        buf = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            rc = self._lib.axb_ipc_export(ctypes.c_void_p(self.ptr), buf)
        if rc != 0:
            raise RuntimeError(f"axb_ipc_export failed with {rc}")
        return bytes(buf)

    def free(self) -> None:
        """Release the allocation. Every tensor that aliases it must be dead, and every process that opened the
        handle must have closed it."""
        if self.ptr:
            self.tensor = None
            self._lib.axb_ipc_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


def open_handle(handle: bytes, device) -> int:
    """Device pointer, valid in THIS process, of an allocation another process exported. ``device`` is the GPU
    whose kernels will use the pointer (peer access to the owner is enabled by the driver on first use)."""
    from ..ops import _common as C
    assert len(handle) == 64
    out = ctypes.c_void_p()
    arr = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
    with torch.cuda.device(torch.device(device)):
        rc = C.lib().axb_ipc_open(arr, ctypes.byref(out))
    if rc != 0 or not out.value:
        raise RuntimeError(f"axb_ipc_open failed with {rc} (is the owning GPU a peer of {device}?)")
    return int(out.value)


def close_handle(ptr: int) -> None:
    from ..ops import _common as C
    if ptr:
        C.lib().axb_ipc_close(ctypes.c_void_p(ptr))
