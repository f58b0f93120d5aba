"""Arrangement of a layer's parts.

pre_norm_residual (src/dense.rs:178-194):
    x += [post_norm](Mixer(norm(x)));  x += [post_norm](FeedForward(norm(x)))
The norms after the mixer and after the feed-forward are the reference's own lfm3 layout and
are present only when the layer names them.  The residual x is float and is added to in float.

In a decode step of a few bfloat16 rows a norm kernel costs more in launch latency than in work,
so there the block splits a norm between the product that wrote x last and the product that
reads norm(x) first (ops.kernels.SplitNorm), when both parts say they can (`split_norm`); in
every other case the norm runs as a kernel of its own.
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

    def first_reader(self):
        """(norm, part) that read the residual when this block starts: the block before may split that norm."""
        return self.mixer_norm, self.mixer

    def _offer(self, producer, norm, consumer, x, env, which: int):
        """Before `producer` adds into x: if `norm` (the next reader of x) can be split between it
        and `consumer`, asks the producer to leave its half.  Returns the split or None."""
        M, D = x.shape
        if not (getattr(norm, "splittable", False) and getattr(producer, "split_norm", False)
                and getattr(consumer, "split_norm", False)):
            return None
        reader = getattr(consumer, "split_reader_weight", None)
        if not kernels.split_norm_ok(M, env.dtype, reader() if callable(reader) else None):
            return None      # the product that would read the split's values could not scale its rows
        ws = env.workspace
        sp = kernels.SplitNorm(ws.get(f"block.split.values{which}", (M, D), torch.bfloat16),
                               ws.get(f"block.split.ssq{which}", (M, -(-D // 16)), torch.float32),
                               norm.weight, norm.eps)
        env.split_out = sp
        return sp

    def _normed(self, norm, x, pending, env):
        """norm(x) as the next part's input: the split's values (the part scales its first product),
        or the norm kernel's result."""
        env.split_in = env.split_out = None   # nothing is left over from a part that did not take its offer (or raised)
        if pending is not None and pending.filled and pending.weight is norm.weight:
            env.split_in = pending
            return pending.values
        M, D = x.shape
        h = env.workspace.get("block.h", (M, D), env.dtype)
        norm.forward(h, x)
        return h

    def forward(self, x: torch.Tensor, batch, cache, env, pending=None):
        """Runs the layer on the residual x.  `pending`: the split of this block's first norm that
        the block before left, if it did; returns the split of the next block's first norm
        (`env.next_block_norm`) if this block's feed-forward left one."""
        M, D = x.shape
        ws = env.workspace
        h = self._normed(self.mixer_norm, x, pending, env)
        if self.post_mixer_norm is None:
            mid = self._offer(self.mixer, self.ffn_norm, self.ffn, x, env, 0)
            self.mixer.forward(h, x, True, batch, cache, env)
        else:
            mid = None
            t = ws.get("block.t", (M, D), torch.float32)
            self.mixer.forward(h, t, False, batch, cache, env)
            self.post_mixer_norm.forward(x, t, add=True)
        env.split_in = None
        h = self._normed(self.ffn_norm, x, mid, env)
        if self.post_ffn_norm is None:
            nxt = env.next_block_norm
            last = None
            if nxt is not None:
                norm, consumer = nxt
                last = self._offer(self.ffn, norm, consumer, x, env, 1)
            self.ffn.forward(h, x, True, batch, env)
        else:
            last = None
            t = ws.get("block.t", (M, D), torch.float32)
            self.ffn.forward(h, t, False, batch, env)
            self.post_ffn_norm.forward(x, t, add=True)
        env.split_in = env.split_out = None
        return last if last is not None and last.filled else None
