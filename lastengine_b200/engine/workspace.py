"""Scratch tensors of a step, kept between steps.

Parts ask for a buffer by name and shape; the same storage comes back every time, so a decode
step uses fixed addresses (a captured CUDA graph stays valid) and steady-state steps allocate
nothing.  A request larger than what the name holds replaces the storage and bumps
`generation`, which invalidates captured graphs.
"""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self.generation = 0
        self.frozen = False

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 16)
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < nbytes:
            if self.frozen:
                raise RuntimeError(f"workspace '{name}' would grow to {nbytes} bytes while a graph is captured")
            # headroom: prompts of slightly different lengths reuse the buffer
            buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=self.device)
            self._bufs[name] = buf
            self.generation += 1
        return buf[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def nbytes(self) -> int:
        return sum(b.numel() for b in self._bufs.values())
