"""Grow-only, per-device scratch owned by the Python shim (the C ABI allocates nothing).

One buffer per (device, purpose).  A buffer only ever grows, is zero-filled when created (the
attention kernel's arrival counters must start at zero and reset themselves after every call), and
is shared by all calls on that device: calls that may overlap on different streams must pass their
own workspace tensors instead.
"""
from __future__ import annotations

import contextlib

import torch

_buffers: dict = {}
_status: dict = {}


def get(device: torch.device, purpose: str, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), purpose)
    buf = _buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        grow = max(nbytes, 2 * buf.numel() if buf is not None else 0)
        buf = torch.zeros(grow, dtype=torch.uint8, device=device)
        _buffers[key] = buf
    return buf


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word kernels OR their DSA_STATUS_* bits into."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    word = _status.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = word
    return word


_NO_GUARD = contextlib.nullcontext()
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def device_guard(device: torch.device):
    """Context that makes `device` current for a launch; free when it already is."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def stream_handle(device: torch.device) -> int:
    """cudaStream_t of torch's current stream on `device` (the stream the C ABI enqueues on)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


STATUS_BITS = {
    0x1: "a bounded device-side wait timed out",
    0x2: "block_table entry outside [0, num_pages)",
    0x4: "sparse index outside [0, num_slots)",
    0x8: "top-k selection wrote an unexpected number of ids",
}


def check_status(device=None, clear: bool = True) -> int:
    """Synchronise and raise RuntimeError if any kernel on `device` reported a fault."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(device)
    value = int(word.item())
    if clear and value:
        word.zero_()
    if value:
        what = "; ".join(text for bit, text in STATUS_BITS.items() if value & bit)
        raise RuntimeError(f"dsa_b200 device status 0x{value:x}: {what}")
    return value


def release():
    _buffers.clear()
    _status.clear()
