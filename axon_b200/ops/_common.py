"""Shared plumbing for the native op wrappers: pointers, streams, status words, launch checks."""
from __future__ import annotations

import ctypes

import torch

from .. import _native

_STATUS: dict[int, torch.Tensor] = {}
LAUNCH_COUNT = 0  # number of native kernels launched by this process (bench.py reports it)

_ERR = {
    1: "a consumer waited for a TMA stage that never landed",
    2: "a producer waited for a stage that was never released",
    3: "an epilogue waited for an accumulator that never completed",
    4: "the MMA warp waited for an accumulator that was never drained",
    5: "a flag owned by another rank was never set (peer wait ran out)",
    6: "bad argument detected on the device",
}
_RC = {
    -1: "bad argument (shape, alignment or mode)",
    -2: "CUDA driver entry point unavailable",
    -3: "TMA tensor-map encoding failed",
    -4: "CUDA launch error",
    -5: "size beyond the supported maximum",
}


class NativeKernelError(RuntimeError):
    """A native kernel refused its arguments, failed to launch, or reported a device-side status."""


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors run the hand-written kernels; CPU tensors run the PyTorch reference."""
    return t.is_cuda


def lib():
    return _native.lib()


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _STATUS.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = buf
    return buf


def launched(rc: int, name: str, n: int = 1) -> None:
    global LAUNCH_COUNT
    if rc != 0:
        raise NativeKernelError(f"{name}: launcher returned {rc}: {_RC.get(rc, 'unknown')}")
    LAUNCH_COUNT += n


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on the device recorded an error (bounded wait ran out)."""
    if _native.debug_requested():
        rec = (ctypes.c_int * 4)()
        src = ctypes.create_string_buffer(256)
        if lib().axb_debug_status(rec, src, 256) != 0:
            raise NativeKernelError(f"debug build: index check failed at {src.value.decode()}:{rec[1]} "
                                    f"(value {rec[2]}, limit {rec[3]})")
    devs = [device.index] if device is not None and device.index is not None else list(_STATUS)
    for idx in devs:
        buf = _STATUS.get(idx)
        if buf is None:
            continue
        code = int(buf[0].item())
        if code != 0:
            buf.zero_()
            raise NativeKernelError(f"device {idx}: kernel status {code}: {_ERR.get(code, 'unknown')}")


_WORKSPACE: dict[tuple, torch.Tensor] = {}


def workspace(device: torch.device, nbytes: int, tag: str = "default") -> torch.Tensor:
    """A cached, grow-only uint8 scratch buffer per (device, tag).

    Kernels launched on one stream run in order, so consecutive ops may share a tag; ops that
    may overlap on different streams must use different tags.
    """
    key = (device.index, tag)
    buf = _WORKSPACE.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACE[key] = buf
    return buf
