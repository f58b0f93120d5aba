"""Token embedding and output head.

x = embed[token] (src/dense.rs:172-177); logits = W_out . norm(x) with W_out the head's own
matrix, or the embedding when the model ties them (src/dense.rs:195-196).  Logits are float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import EMBEDDINGS, HEADS
from .base import EMBEDDING, MATRIX, BuildEnv, Part, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.V, self.D = int(vocab_size), int(hidden_size)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.V, self.D), EMBEDDING)}

    def load(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, tokens: torch.Tensor) -> None:
        kernels.embed(x, self.weight, tokens)


@HEADS.register("linear_head")
class LinearHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.V, self.D, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: torch.Tensor | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {} if self.tied else {"weight": TensorSpec((self.V, self.D), MATRIX)}

    def load(self, tensors, env: BuildEnv) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.weight

    def flops_per_row(self) -> int:
        return 2 * self.V * self.D

    def forward(self, logits: torch.Tensor, xn: torch.Tensor) -> None:
        kernels.linear(logits, xn, self.weight)
