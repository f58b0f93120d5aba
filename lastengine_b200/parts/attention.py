"""Grouped-query attention mixer over the paged cache.

q = Wq h, k = Wk h, v = Wv h; optional per-head RMSNorm on q and k (shared [head_dim] weights,
the model's eps) before the rotation; k and v appended to the cache at the token's position;
causal softmax attention with scale 1/sqrt(head_dim), optionally inside a window; optional
sigmoid gate per head from its own projection; out = Wo o.  (src/dense.rs:113-152.)
The three projections (and the gate) are one matrix product over fused weights, as the
reference fuses gate and up (src/gpu/dense.rs:67-74).
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, NORM, BuildEnv, KVSpec, Mixer, PartSpec, TensorSpec


@MIXERS.register("attention")
class AttentionMixer(Mixer):
    split_norm = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 norm_eps: float, qk_norm: bool = True, position: PartSpec | None = None,
                 window: int = 0, output_gate: bool = False, own_kv: bool = True,
                 scale: float | None = None):
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is larger than the attention kernels take (256)")
        self.D, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.eps = float(norm_eps)
        self.qk_norm = bool(qk_norm)
        self.window = int(window)
        self.output_gate = bool(output_gate)
        self.own_kv = bool(own_kv)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        pos = position or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos.kind)(**pos.params)
        self.w_in = self.w_out = self.q_norm_w = self.k_norm_w = None

    def tensors(self) -> dict[str, TensorSpec]:
        D, nh, nkv, hd = self.D, self.nh, self.nkv, self.hd
        t = {"q_proj.weight": TensorSpec((nh * hd, D), MATRIX),
             "out_proj.weight": TensorSpec((D, nh * hd), MATRIX)}
        if self.own_kv:
            t["k_proj.weight"] = TensorSpec((nkv * hd, D), MATRIX)
            t["v_proj.weight"] = TensorSpec((nkv * hd, D), MATRIX)
        if self.qk_norm:
            t["q_layernorm.weight"] = TensorSpec((hd,), NORM)
            if self.own_kv:
                t["k_layernorm.weight"] = TensorSpec((hd,), NORM)
        if self.output_gate:
            t["gate_proj.weight"] = TensorSpec((nh, D), MATRIX)
        for name, spec in self.position.tensors().items():
            t[f"position.{name}"] = spec
        return t

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window)

    def load(self, tensors, env: BuildEnv) -> None:
        parts = [tensors["q_proj.weight"]]
        if self.own_kv:
            parts += [tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if self.output_gate:
            parts.append(tensors["gate_proj.weight"])
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        self.w_out = tensors["out_proj.weight"].contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors["q_layernorm.weight"].contiguous()
            self.k_norm_w = tensors["k_layernorm.weight"].contiguous() if self.own_kv else None
        self.position.load({n[len("position."):]: v for n, v in tensors.items() if n.startswith("position.")}, env)

    def split_reader_weight(self):
        return self.w_in

    def flops_per_query_key(self) -> int:
        return 4 * self.nh * self.hd        # a score and a weighted value, a multiply-add each, per head and dimension

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        M = h.shape[0]
        ws = env.workspace
        scale, emit = env.take_split_in(), env.take_split_out()
        writes = self.own_kv and cache.writable
        if self.own_kv and not cache.writable:
            w_in = self.w_in[: nh * hd] if not self.output_gate else None
        else:
            w_in = self.w_in
        if w_in is None:  # q and gate rows are not adjacent once k, v are skipped: two products
            raise NotImplementedError("a gated attention layer reading another layer's cache")
        proj = ws.get("attn.proj", (M, w_in.shape[0]), env.dtype)
        kernels.linear(proj, h, w_in, scale=scale)
        q_in = proj[:, : nh * hd]
        k_in = v_in = gate = None
        col = nh * hd
        if writes:
            k_in = proj[:, col: col + nkv * hd]
            v_in = proj[:, col + nkv * hd: col + 2 * nkv * hd]
            col += 2 * nkv * hd
        if self.output_gate:
            gate = proj[:, col: col + nh]
        q = ws.get("attn.q", (M, nh * hd), env.dtype)
        kp, vp = (cache.k, cache.v) if writes else (None, None)
        rotary = self.position.fused_rotary()
        raw = None
        if rotary is not None and kernels.decode_attention_takes_raw(env.dtype, batch, M, nh, nkv, hd, cache.page_size, *rotary):
            # a decode step: the attention kernel norms and rotates q and k and stores k and v itself
            raw = kernels.RawQKV(q_in, k_in, v_in, self.q_norm_w, self.k_norm_w if writes else None, self.eps, *rotary)
        elif rotary is not None:
            # per-head norm, rotation and the cache write in one launch
            kernels.qk_rope_store(q, q_in, k_in, v_in, kp, vp, cache.block_table, batch, self.q_norm_w,
                                  self.k_norm_w if writes else None, self.eps, *rotary, nh, nkv, hd, cache.page_size)
        else:
            # an encoding of the part's own: norm, then the part on the normed q and k, then the store
            qn = ws.get("attn.qn", (M, nh * hd), env.dtype)
            kernels.qk_rope_store(qn, q_in, None, None, None, None, cache.block_table, batch, self.q_norm_w, None,
                                  self.eps, None, 0, True, nh, nkv, hd, cache.page_size)
            kn = vn = None
            if writes:
                kn = ws.get("attn.kn", (M, nkv * hd), env.dtype)
                kernels.qk_rope_store(kn, k_in, None, None, None, None, cache.block_table, batch, self.k_norm_w, None,
                                      self.eps, None, 0, True, nkv, nkv, hd, cache.page_size)
                vn = ws.get("attn.vn", (M, nkv * hd), env.dtype)      # the values beside them, rows as wide as kn's
                kernels.qk_rope_store(vn, v_in, None, None, None, None, cache.block_table, batch, None, None,
                                      self.eps, None, 0, True, nkv, nkv, hd, cache.page_size)
            self.position.apply(qn.view(M, nh, hd), kn.view(M, nkv, hd) if writes else None, batch.row_pos)
            kernels.qk_rope_store(q, qn, kn, vn, kp, vp, cache.block_table, batch, None, None, self.eps,
                                  None, 0, True, nh, nkv, hd, cache.page_size)
        o = ws.get("attn.o", (M, nh * hd), env.dtype)
        n_splits = kernels.attention_splits(batch, nkv, nh // nkv, hd=hd)
        scratch = None
        if n_splits > 1:
            scratch = ws.get("attn.part", (M * nh * n_splits * (hd + 2),), torch.float32)
        kernels.attention(o, None if raw is not None else q, cache.k, cache.v, cache.block_table, batch, nh, nkv, hd,
                          cache.page_size, self.window, self.scale, gate=gate, n_splits=n_splits, scratch=scratch, raw=raw)
        kernels.linear(out, o, self.w_out, kernels.ACCUMULATE if accumulate else kernels.STORE,
                       emit=emit if accumulate else None)
