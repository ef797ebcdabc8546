"""Per-stream scratch arenas.

The reference keeps one ``RNSWorkspace`` per (rows, channels, stream) in a dict
that never shrinks (``layers/rns_linear.py:206-223``,
``backends/cuda_backend.py:366-380``) because a workspace shared by two streams
would race.  Here each CUDA stream owns ONE growable byte buffer; every call
carves its temporaries from the start of it.  Work on a stream executes in
order, so the next call on the same stream may reuse the same bytes, and two
streams never share a buffer.

Nothing is allocated while a CUDA graph is being captured: a buffer that would
have to grow then raises, so warm the shape up once before capturing.
"""
from __future__ import annotations

import threading

import torch

_ALIGN = 256


class ArenaFrame:
    """Bump allocator over one stream's buffer for the duration of one call."""

    __slots__ = ("_arena", "_key", "_offset", "_wanted")

    def __init__(self, arena: "StreamArena", key: tuple[int, int]) -> None:
        self._arena = arena
        self._key = key
        self._offset = 0
        self._wanted: list[tuple[int, torch.dtype, tuple[int, ...]]] = []

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        if isinstance(shape, int):
            shape = (shape,)
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * dtype.itemsize
        start = self._offset
        self._offset = (start + nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        buf = self._arena._buffer(self._key, self._offset)
        return buf[start:start + nbytes].view(dtype).view(*shape)


class StreamArena:
    """Scratch buffers keyed by (device index, stream handle)."""

    def __init__(self, initial_bytes: int = 1 << 20) -> None:
        self._initial = int(initial_bytes)
        self._buffers: dict[tuple[int, int], torch.Tensor] = {}
        self._lock = threading.Lock()

    def frame(self, device: torch.device) -> ArenaFrame:
        index = device.index if device.index is not None else torch.cuda.current_device()
        stream = torch.cuda.current_stream(index)
        return ArenaFrame(self, (index, int(stream.cuda_stream)))

    def block(self, device: torch.device, nbytes: int) -> tuple[int, int]:
        """(device pointer, stream handle) of at least ``nbytes`` of the current
        stream's scratch: the allocation-light form of ``frame`` for callers that
        only need addresses (one dictionary lookup instead of tensor views)."""
        index = device.index if device.index is not None else torch.cuda.current_device()
        stream = int(torch.cuda.current_stream(index).cuda_stream)
        return self._buffer((index, stream), int(nbytes)).data_ptr(), stream

    def _buffer(self, key: tuple[int, int], need: int) -> torch.Tensor:
        buf = self._buffers.get(key)
        if buf is not None and buf.numel() >= need:
            return buf
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                "RNS scratch arena must grow during CUDA graph capture; run the same "
                "shapes once on this stream before capturing"
            )
        size = max(self._initial, 1 << (int(need) - 1).bit_length())
        with self._lock:
            new = torch.empty(size, dtype=torch.uint8, device=torch.device("cuda", key[0]))
            # Earlier slices of the old buffer handed out in this frame stay valid:
            # tensors keep their storage alive, and the caching allocator only
            # reuses it after the work queued on this stream has run.
            self._buffers[key] = new
        return new

    def bytes_reserved(self) -> int:
        return sum(int(b.numel()) for b in self._buffers.values())

    def streams(self) -> list[tuple[int, int]]:
        return list(self._buffers)

    def release(self) -> None:
        self._buffers.clear()
