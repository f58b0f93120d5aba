"""Rotary position encoding: the table of inverse frequencies and the pairing style.

angle(pos, i) = pos * theta^(-2i/rope_dim), i < rope_dim/2; pairs (i, i + rope_dim/2) in the
split-half ("neox") style the reference uses for this architecture, or (2i, 2i+1) in the
adjacent style of its other dense architecture (src/dense.rs:103-111, :77).  The rotation
itself happens in the mixer's kernel, in float.
"""
from __future__ import annotations

import torch

from ..registry import POSITION_ENCODINGS
from .base import BuildEnv, Part


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(Part):
    def __init__(self, rope_dim: int, theta: float, style: str = "neox"):
        if rope_dim % 2 != 0 or rope_dim < 2:
            raise ValueError(f"rope_dim must be even and positive, got {rope_dim}")
        if style not in ("neox", "adjacent"):
            raise ValueError(f"unknown rotary pairing '{style}' (neox, adjacent)")
        self.rope_dim = int(rope_dim)
        self.theta = float(theta)
        self.neox = style == "neox"
        self.inv_freq: torch.Tensor | None = None

    def load(self, tensors, env: BuildEnv) -> None:
        i = torch.arange(self.rope_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rope_dim)
        self.inv_freq = inv.to(torch.float32).to(env.device)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(Part):
    """For mixers that take positions from nowhere (the short convolution is causal by itself)."""
    rope_dim = 0
    neox = True
    inv_freq = None

    def __init__(self):
        pass
