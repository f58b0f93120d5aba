"""Feed-forward parts: dense SwiGLU, and sigmoid-routed top-k experts of the same shape.

Dense (src/dense.rs:188-191): f = W2 (silu(W1 h) * W3 h).  Gate and up weights are one
matrix, as in the reference's GPU path (src/gpu/dense.rs:67-74).  In bfloat16 their rows are
interleaved in blocks of 16 so that the matrix product's epilogue holds a gate value and its
up value together and applies SwiGLU before anything is written; gate and up are never
rounded.

Experts: z = Wr h (float), s = sigmoid(z); the k experts with the largest s + bias (ties to
the lower index; the bias chooses, it does not weigh); weight s_e, divided by the sum over the
chosen when norm_topk, times the scaling factor; f = sum_e weight_e * expert_e(h).  The
reference's own lfm3 has no experts (src/dense.rs:187-191); its other architecture routes by
softmax and adds a shared expert (src/cpu_ref.rs:239-263), which this is not.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import FEED_FORWARDS
from .base import BIAS, MATRIX, VECTOR, BuildEnv, FeedForward, TensorSpec


def fuse_gate_up(w1: torch.Tensor, w3: torch.Tensor, interleave: bool) -> torch.Tensor:
    """[F, D] x 2 -> [2F, D]: gate rows then up rows, or blocks of 16 gate / 16 up alternating."""
    F_, D = w1.shape
    if not interleave:
        return torch.cat([w1, w3], dim=0).contiguous()
    g = w1.reshape(F_ // 16, 16, D)
    u = w3.reshape(F_ // 16, 16, D)
    return torch.stack([g, u], dim=1).reshape(2 * F_, D).contiguous()


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    split_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.D, self.F = int(hidden_size), int(intermediate_size)
        self.w13 = self.w2 = None
        self.fused = False

    def tensors(self) -> dict[str, TensorSpec]:
        return {"w1.weight": TensorSpec((self.F, self.D), MATRIX),
                "w3.weight": TensorSpec((self.F, self.D), MATRIX),
                "w2.weight": TensorSpec((self.D, self.F), MATRIX)}

    def load(self, tensors, env: BuildEnv) -> None:
        self.fused = (not env.is_float32) and self.F % 16 == 0
        self.w13 = fuse_gate_up(tensors["w1.weight"], tensors["w3.weight"], self.fused)
        self.w2 = tensors["w2.weight"].contiguous()

    def split_reader_weight(self):
        return self.w13

    def forward(self, h, out, accumulate, batch, env) -> None:
        M = h.shape[0]
        ws = env.workspace
        scale, emit = env.take_split_in(), env.take_split_out()
        a = ws.get("ffn.a", (M, self.F), env.dtype)
        if self.fused:
            kernels.linear(a, h, self.w13, kernels.SWIGLU, scale=scale)
        else:
            gu = ws.get("ffn.gu", (M, 2 * self.F), torch.float32)
            kernels.linear(gu, h, self.w13, scale=scale)
            kernels.swiglu(a, gu)
        kernels.linear(out, a, self.w2, kernels.ACCUMULATE if accumulate else kernels.STORE,
                       emit=emit if accumulate else None)


@FEED_FORWARDS.register("sigmoid_topk_moe")
class SigmoidTopKMoE(FeedForward):
    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_size: int,
                 norm_topk: bool = True, use_bias: bool = True, scaling: float = 1.0,
                 bias_std: float = 0.1):
        if not 1 <= top_k <= min(num_experts, 16):
            raise ValueError(f"top-{top_k} of {num_experts} experts: the router takes 1..min(experts, 16)")
        if num_experts > 256:
            raise ValueError(f"{num_experts} experts: the router takes at most 256")
        self.D, self.E, self.k, self.Fe = int(hidden_size), int(num_experts), int(top_k), int(expert_size)
        self.norm_topk, self.use_bias, self.scaling = bool(norm_topk), bool(use_bias), float(scaling)
        self.bias_std = float(bias_std)
        self.router_w = self.router_b = self.w13 = self.w2 = None
        self.fused = False

    def tensors(self) -> dict[str, TensorSpec]:
        t = {"gate.weight": TensorSpec((self.E, self.D), VECTOR)}
        if self.use_bias:
            t["expert_bias"] = TensorSpec((self.E,), BIAS, std=self.bias_std)
        for e in range(self.E):
            t[f"experts.{e}.w1.weight"] = TensorSpec((self.Fe, self.D), MATRIX)
            t[f"experts.{e}.w3.weight"] = TensorSpec((self.Fe, self.D), MATRIX)
            t[f"experts.{e}.w2.weight"] = TensorSpec((self.D, self.Fe), MATRIX)
        return t

    def load(self, tensors, env: BuildEnv) -> None:
        self.fused = (not env.is_float32) and self.Fe % 16 == 0
        self.router_w = tensors["gate.weight"].contiguous()
        self.router_b = tensors["expert_bias"].contiguous() if self.use_bias else None
        self.w13 = torch.stack([fuse_gate_up(tensors[f"experts.{e}.w1.weight"], tensors[f"experts.{e}.w3.weight"],
                                             self.fused) for e in range(self.E)]).contiguous()
        self.w2 = torch.stack([tensors[f"experts.{e}.w2.weight"] for e in range(self.E)]).contiguous()

    def flops_per_row(self) -> int:
        return 2 * self.D * self.E + self.k * 6 * self.D * self.Fe       # the router, and k experts of three matrices

    def unread_weight_bytes(self, rows: int) -> float:
        """With uniform routing an expert is chosen by none of `rows` rows with probability (1 - k/E)^rows."""
        if self.w13 is None:
            return 0.0
        per_expert = (self.w13[0].numel() + self.w2[0].numel()) * self.w13.element_size()
        return self.E * per_expert * (1.0 - self.k / self.E) ** rows

    def forward(self, h, out, accumulate, batch, env) -> None:
        M = h.shape[0]
        P = M * self.k
        ws = env.workspace
        ids = ws.get("moe.ids", (M, self.k), torch.int32)
        wts = ws.get("moe.w", (M, self.k), torch.float32)
        kernels.moe_router(ids, wts, h, self.router_w, self.router_b, self.norm_topk, self.scaling)
        offsets = ws.get("moe.offsets", (self.E + 1,), torch.int32)
        sorted_pair = ws.get("moe.sorted", (P,), torch.int32)
        pair_row = ws.get("moe.rows", (P,), torch.int32)
        kernels.moe_align(offsets, sorted_pair, pair_row, ids, self.E)
        xs = ws.get("moe.xs", (P, self.D), env.dtype)
        kernels.gather_rows(xs, h, sorted_pair, div=self.k)
        a = ws.get("moe.a", (P, self.Fe), env.dtype)
        if self.fused:
            kernels.linear(a, xs, self.w13, kernels.SWIGLU, group_offsets=offsets, rows_hint=P)
        else:
            gu = ws.get("moe.gu", (P, 2 * self.Fe), torch.float32)
            kernels.linear(gu, xs, self.w13, group_offsets=offsets, rows_hint=P)
            kernels.swiglu(a, gu)
        ys = ws.get("moe.ys", (P, self.D), torch.float32)
        kernels.linear(ys, a, self.w2, group_offsets=offsets, rows_hint=P)
        kernels.moe_combine(out, ys, pair_row, wts, accumulate)
