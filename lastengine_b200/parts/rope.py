"""Rotary position encoding: the table of inverse frequencies and the pairing style.

angle(pos, i) = pos * theta^(-2i/rope_dim) / factor[i], i < rope_dim/2; pairs (i, i + rope_dim/2)
in the split-half ("neox") style the reference uses for this architecture, or (2i, 2i+1) in the
adjacent style of its other dense architecture (src/dense.rs:103-111, :77).  The factors are the
model's optional `rope_freqs.weight`, which the reference applies on layers without a window only
(src/dense.rs:106,125); without the tensor they are 1.  The rotation itself happens in the
mixer's kernel, in float: this part hands it the table.
"""
from __future__ import annotations

import torch

from ..registry import POSITION_ENCODINGS
from .base import VECTOR, BuildEnv, PositionEncoding, TensorSpec

FREQ_FACTORS = "rope_freqs.weight"     # one tensor for the whole model


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, rope_dim: int, theta: float, style: str = "neox", freq_factors: bool = False):
        if rope_dim % 2 != 0 or rope_dim < 2:
            raise ValueError(f"rope_dim must be even and positive, got {rope_dim}")
        if style not in ("neox", "adjacent"):
            raise ValueError(f"unknown rotary pairing '{style}' (neox, adjacent)")
        self.rope_dim = int(rope_dim)
        self.theta = float(theta)
        self.neox = style == "neox"
        self.freq_factors = bool(freq_factors)     # takes the model's frequency factors when the checkpoint has them
        self.inv_freq: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        if not self.freq_factors:
            return {}
        return {FREQ_FACTORS: TensorSpec((self.rope_dim // 2,), VECTOR, optional=True, shared_name=FREQ_FACTORS)}

    def load(self, tensors, env: BuildEnv) -> None:
        i = torch.arange(self.rope_dim // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rope_dim)
        ff = tensors.get(FREQ_FACTORS) if self.freq_factors else None
        if ff is not None:
            inv = inv / ff.detach().to("cpu", torch.float64).reshape(-1)
        self.inv_freq = inv.to(torch.float32).to(env.device)

    def fused_rotary(self):
        return self.inv_freq, self.rope_dim, self.neox


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """For mixers that take positions from nowhere (a causal mask alone orders the keys)."""

    def __init__(self):
        pass

    def fused_rotary(self):
        return None, 0, True
