"""Chooses next tokens on the device from a step's logits."""
from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from .params import PENALTY_WINDOW, SamplingParams


class Sampler:
    def __init__(self, params: SamplingParams, device: torch.device):
        self.params = params
        self.device = device

    def needs_uniform(self) -> bool:
        return not self.params.greedy

    def apply_penalties(self, logits: torch.Tensor, histories: list[list[int]]) -> None:
        """Penalises, in place, the tokens of each sequence's last 256 (src/local.rs:60-63)."""
        p = self.params
        if not p.has_penalties:
            return
        n = logits.shape[0]
        h = np.zeros((n, PENALTY_WINDOW), dtype=np.int32)
        ln = np.zeros(n, dtype=np.int32)
        for i, hist in enumerate(histories):
            tail = hist[-PENALTY_WINDOW:]
            h[i, :len(tail)] = tail
            ln[i] = len(tail)
        hd = torch.from_numpy(h).to(self.device)
        ld = torch.from_numpy(ln).to(self.device)
        kernels.penalties(logits, hd, ld, p.repeat_penalty, p.presence_penalty)

    def sample(self, out: torch.Tensor, logits: torch.Tensor, u01: torch.Tensor | None) -> None:
        """out[i] = the chosen token of row i of `logits` (float [n, vocab])."""
        p = self.params
        if p.greedy:
            kernels.argmax(out, logits)
        else:
            kernels.sample(out, logits, u01, p.top_k, p.temperature, p.top_p, p.min_p)
