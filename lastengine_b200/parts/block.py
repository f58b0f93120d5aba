"""Arrangement of a layer's parts.

pre_norm_residual (src/dense.rs:178-194):
    x += [post_norm](Mixer(norm(x)));  x += [post_norm](FeedForward(norm(x)))
The norms after the mixer and after the feed-forward are the reference's own lfm3 layout and
are present only when the layer names them.  The residual x is float and is added to in float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import BLOCKS


@BLOCKS.register("pre_norm_residual")
class PreNormResidualBlock:
    def __init__(self, mixer, ffn, mixer_norm, ffn_norm, post_mixer_norm=None, post_ffn_norm=None):
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.post_mixer_norm, self.post_ffn_norm = post_mixer_norm, post_ffn_norm

    def parts(self) -> dict[str, object]:
        p = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}
        if self.post_mixer_norm is not None:
            p["post_mixer_norm"] = self.post_mixer_norm
        if self.post_ffn_norm is not None:
            p["post_ffn_norm"] = self.post_ffn_norm
        return p

    def forward(self, x: torch.Tensor, batch, cache, env) -> None:
        M, D = x.shape
        ws = env.workspace
        h = ws.get("block.h", (M, D), env.dtype)
        self.mixer_norm.forward(h, x)
        if self.post_mixer_norm is None:
            self.mixer.forward(h, x, True, batch, cache, env)
        else:
            t = ws.get("block.t", (M, D), torch.float32)
            self.mixer.forward(h, t, False, batch, cache, env)
            self.post_mixer_norm.forward(x, t, add=True)
        h = ws.get("block.h", (M, D), env.dtype)
        self.ffn_norm.forward(h, x)
        if self.post_ffn_norm is None:
            self.ffn.forward(h, x, True, batch, env)
        else:
            t = ws.get("block.t", (M, D), torch.float32)
            self.ffn.forward(h, t, False, batch, env)
            self.post_ffn_norm.forward(x, t, add=True)
