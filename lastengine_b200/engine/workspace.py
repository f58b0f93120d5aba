"""Scratch tensors of a step, kept between steps.

Parts ask for a buffer by name and shape; the same storage comes back every time, so a decode
step uses fixed addresses (a captured CUDA graph stays valid) and steady-state steps allocate
nothing.  A request larger than what the name holds replaces the storage and bumps
`generation`, which invalidates captured graphs.
"""
from __future__ import annotations

import torch


_ELEMENT_SIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1}


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}    # (name, shape, dtype) -> the view handed out last time
        self.generation = 0
        self.frozen = False

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view                 # the same request as before: the same tensor, at no cost
        n = 1
        for s in shape:
            n *= int(s)
        esize = _ELEMENT_SIZE.get(dtype) or torch.empty((), dtype=dtype).element_size()
        nbytes = max(n * esize, 16)
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < nbytes:
            if self.frozen:
                raise RuntimeError(f"workspace '{name}' would grow to {nbytes} bytes while a graph is captured")
            # headroom: prompts of slightly different lengths reuse the buffer
            buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=self.device)
            self._bufs[name] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name]:   # views of the storage that was replaced
                del self._views[k]
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n * esize].view(dtype).view(*shape)
        self._views[key] = view
        return view

    def nbytes(self) -> int:
        return sum(b.numel() for b in self._bufs.values())
