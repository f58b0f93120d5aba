"""Gated short-convolution mixer.

(B, C, x) = in_proj(h) split in this order; bx = B*x; causal depthwise convolution of length
L over time with the last L-1 values of bx per channel carried as state; y = C * conv;
out = out_proj(y).  No activation.  (src/dense.rs:153-170.)  The reference's convolution has no
bias; with `bias` the depthwise convolution adds its own per-channel term before the gate C
(the architecture's `conv_bias` key; tensor `conv.bias` [D]).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import MIXERS
from .base import BIAS, MATRIX, VECTOR, BuildEnv, Mixer, StateSpec, TensorSpec


@MIXERS.register("shortconv")
class ShortConvMixer(Mixer):
    split_norm = True

    def __init__(self, hidden_size: int, L_cache: int, bias: bool = False):
        if not 2 <= L_cache <= 17:
            raise ValueError(f"conv_L_cache {L_cache} outside what the kernel takes (2..17)")
        self.D, self.Lc = int(hidden_size), int(L_cache)
        self.bias = bool(bias)
        self.w_in = self.w_conv = self.w_out = self.b_conv = None

    def tensors(self) -> dict[str, TensorSpec]:
        D, Lc = self.D, self.Lc
        t = {"in_proj.weight": TensorSpec((3 * D, D), MATRIX),
             "conv.weight": TensorSpec((D, 1, Lc), VECTOR),
             "out_proj.weight": TensorSpec((D, D), MATRIX)}
        if self.bias:
            t["conv.bias"] = TensorSpec((D,), BIAS)
        return t

    def cache_spec(self):
        return StateSpec((self.D, self.Lc - 1), torch.float32)

    def load(self, tensors, env: BuildEnv) -> None:
        self.w_in = tensors["in_proj.weight"].contiguous()
        self.w_conv = tensors["conv.weight"].reshape(self.D, self.Lc).contiguous()
        self.w_out = tensors["out_proj.weight"].contiguous()
        self.b_conv = tensors["conv.bias"].contiguous() if self.bias else None

    def split_reader_weight(self):
        return self.w_in

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        M = h.shape[0]
        ws = env.workspace
        scale, emit = env.take_split_in(), env.take_split_out()
        y = ws.get("conv.y", (M, self.D), env.dtype)
        # a decode step of a few sequences: projection and convolution in one launch
        if not kernels.shortconv_decode_fused(y, h, self.w_in, self.w_conv, self.b_conv, cache.state, batch, self.Lc, scale=scale):
            bcx = ws.get("conv.bcx", (M, 3 * self.D), env.dtype)
            kernels.linear(bcx, h, self.w_in, scale=scale)
            kernels.shortconv(y, bcx, self.w_conv, self.b_conv, cache.state, batch, self.Lc)
        kernels.linear(out, y, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE,
                       emit=emit if accumulate else None)
