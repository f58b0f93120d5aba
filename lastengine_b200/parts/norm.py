"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w  (src/dense.rs:27-30)."""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import NORMS
from .base import NORM, BuildEnv, Part, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    # y = x * r * w with one factor r per row: a block may leave bfloat16(x * w) to the product
    # before it and r to the product after it (a norm with a mean or a bias could not be split so)
    splittable = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), NORM)}

    def load(self, tensors: dict[str, torch.Tensor], env: BuildEnv) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor | None = None,
                add: bool = False) -> None:
        """out = norm(x[rows]) (or out += norm(x) with add); x is the float residual or a float buffer."""
        kernels.rmsnorm(out, x, self.weight, self.eps, rows=rows, add=add)
