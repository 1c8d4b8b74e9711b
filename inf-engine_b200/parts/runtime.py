"""What every part shares at run time: the device, the activation dtype, named
work buffers, and pinned staging for the per-step host-to-device copy."""

from __future__ import annotations

import numpy as np
import torch


class Workspace:
    """Named device buffers that persist between steps.

    ``take(name, shape, dtype)`` returns a view of a buffer that is at least that
    large; the same name gives the same memory, so layers reuse each other's
    scratch and a captured CUDA graph sees fixed addresses.  ``frozen`` forbids
    growth (set while graphs that point into the buffers are alive).
    """

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}     # (name, shape, dtype) -> the view handed out last time
        self.frozen = False
        self.moves = 0      # how often a buffer was replaced by a larger one (what pointed at the old one is stale)

    def take(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        view = self._take(name, shape, dtype)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[key] = view
        return view

    def _take(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * dtype.itemsize
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < nbytes:
            if self.frozen and buf is not None:
                raise RuntimeError(f"workspace buffer {name!r} would grow from {buf.numel()} to {nbytes} bytes "
                                   "while CUDA graphs point into it")
            # round up so that slowly growing steps do not reallocate every time
            cap = max(nbytes, 256)
            cap = 1 << (cap - 1).bit_length() if cap < (1 << 20) else -(-cap // (1 << 20)) * (1 << 20)
            if buf is not None:
                self.moves += 1
            buf = torch.zeros(cap, dtype=torch.uint8, device=self.device)   # some kernels keep counters that start at zero
            self._buffers[name] = buf
            self._views = {k: v for k, v in self._views.items() if k[0] != name}   # views of the buffer it replaces
        return buf[:nbytes].view(dtype).view(shape)

    def reserved_bytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())


class Staging:
    """Pinned host buffers for one int32 copy per step, used in rotation; a buffer
    is reused only after the copy that last read it has finished."""

    def __init__(self, device: torch.device, depth: int = 4):
        self.device = device
        self.depth = depth
        self._bufs: list[torch.Tensor | None] = [None] * depth
        self._events: list[torch.cuda.Event | None] = [None] * depth
        self._next = 0

    def upload(self, host: np.ndarray, into: torch.Tensor | None = None) -> torch.Tensor:
        """Copy an int32 array to the device (into ``into`` when given) on the current stream."""
        i = self._next
        self._next = (i + 1) % self.depth
        if self._events[i] is not None:
            self._events[i].synchronize()
        n = int(host.size)
        buf = self._bufs[i]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(1024, 1 << max(0, (n - 1)).bit_length()), dtype=torch.int32, pin_memory=True)
            self._bufs[i] = buf
        buf[:n].numpy()[:] = host
        if into is None:
            into = torch.empty(n, dtype=torch.int32, device=self.device)
        into[:n].copy_(buf[:n], non_blocking=True)
        ev = self._events[i] or torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return into[:n]


class Runtime:
    def __init__(self, device: str | torch.device, act_dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        if act_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"activation dtype must be float32 or bfloat16, got {act_dtype}")
        self.act_dtype = act_dtype
        self.ws = Workspace(self.device)
        self.staging = Staging(self.device)
        self.shared: dict = {}      # tables that several parts share (rotary tables, for instance)

    @property
    def exact(self) -> bool:
        """True on the 32-bit path: no tensor cores, no reduced precision anywhere."""
        return self.act_dtype is torch.float32
