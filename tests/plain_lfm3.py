"""A plain, slow implementation of the LFM3 hybrid decoder, for tests only.

Whole sequences, no cache, no batching, one function per part, ordinary tensor arithmetic
on the CPU.  It shares no code with the library: it reads config.json and the safetensors
file itself.  Every function is written from the reference's formulas and cites them
(file:line inside TheSyrianDev/LastEngine).

It rests on those formulas, not on a run of the reference: the reference is Rust and this
environment has no Rust toolchain, and its only loader reads quantized GGUF files, so its
model code can neither be compiled nor fed here.  The one piece of the reference that does
compile here (the bodies of its short-convolution kernels, plain C under a small shim) anchors
`short_conv` through tests/golden/.

`rnd` is a rounding hook: the identity for the 32-bit path, rounding to bfloat16 for the
bfloat16 path.  It is applied exactly where the library's bfloat16 path stores a value in
bfloat16 (activations that feed matrix products, and the cached keys and values); norms,
softmax, rotation, router and the residual stay unrounded, as in the library.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np
import torch

_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2), "F64": (np.float64, 8)}


def read_safetensors(path: str, dtype=torch.float64) -> dict[str, torch.Tensor]:
    """name -> tensor (converted to `dtype`), names without a leading 'model.'."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        np_dt, _ = _ST_DTYPES[e["dtype"]]
        b, t = e["data_offsets"]
        arr = np.frombuffer(data[b:t], dtype=np_dt).reshape(e["shape"])
        if e["dtype"] == "BF16":
            arr32 = (arr.astype(np.uint32) << 16).view(np.float32)
            ten = torch.from_numpy(arr32.copy())
        else:
            ten = torch.from_numpy(arr.astype(np.float64))
        key = name[len("model."):] if name.startswith("model.") else name
        out[key] = ten.to(dtype)
    return out


def identity(t: torch.Tensor) -> torch.Tensor:
    return t


def round_bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


# ---- parts -----------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """src/dense.rs:27-30: r = 1/sqrt(sum(x^2)/n + eps); y = x*r*w."""
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return x * r * w


def silu(x: torch.Tensor) -> torch.Tensor:
    """src/dense.rs:31: x / (1 + exp(-x))."""
    return x / (1.0 + torch.exp(-x))


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    """src/dense.rs:32."""
    return 1.0 / (1.0 + torch.exp(-x))


def rope(v: torch.Tensor, positions: torch.Tensor, rope_dim: int, theta: float, neox: bool = True,
         freq_factors: torch.Tensor | None = None) -> torch.Tensor:
    """src/dense.rs:103-111.  v: [T, heads, head_dim]; pairs (i, i+half) when neox, else (2i, 2i+1);
    angle = pos * theta^(-2i/rope_dim) / freq_factors[i] (:106; no factors: 1); a' = a cos - b sin,
    b' = a sin + b cos."""
    half = rope_dim // 2
    i = torch.arange(half, dtype=v.dtype, device=v.device)
    th = positions.to(v.dtype)[:, None] * torch.pow(torch.tensor(theta, dtype=v.dtype, device=v.device),
                                                    -(2.0 * i) / rope_dim)[None, :]
    if freq_factors is not None:
        th = th / freq_factors.to(v.dtype)[None, :]
    s, c = torch.sin(th)[:, None, :], torch.cos(th)[:, None, :]
    out = v.clone()
    if neox:
        a, b = v[..., :half], v[..., half:2 * half]
        out[..., :half] = a * c - b * s
        out[..., half:2 * half] = a * s + b * c
    else:
        a, b = v[..., 0:2 * half:2], v[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = a * c - b * s
        out[..., 1:2 * half:2] = a * s + b * c
    return out


def attention(h, p, T, *, nh, nkv, hd, eps, theta, rope_dim, window=0, gate=False, rnd=identity, pos0=0,
              freq_factors=None):
    """src/dense.rs:113-152.  h: [T, D]; p: the layer's tensors by short name.  `freq_factors`: the
    model's `rope_freqs.weight`, which the caller hands over for layers without a window only (:125)."""
    q = rnd(h @ p["q_proj.weight"].T).view(T, nh, hd)
    k = rnd(h @ p["k_proj.weight"].T).view(T, nkv, hd)
    v = rnd(h @ p["v_proj.weight"].T).view(T, nkv, hd)
    q = rms_norm(q, p["q_layernorm.weight"], eps)          # :119-123, per head over head_dim, before rope
    k = rms_norm(k, p["k_layernorm.weight"], eps)
    pos = torch.arange(pos0, pos0 + T, device=h.device)
    q = rnd(rope(q, pos, rope_dim, theta, freq_factors=freq_factors))
    k = rnd(rope(k, pos, rope_dim, theta, freq_factors=freq_factors))   # :126-128: the cache holds rotated keys
    G = nh // nkv
    out = torch.zeros(T, nh, hd, dtype=h.dtype, device=h.device)
    for hh in range(nh):
        kvh = hh // G                                       # :133
        sc = (q[:, hh, :] @ k[:, kvh, :].T) / math.sqrt(hd)  # :136
        t = torch.arange(T, device=h.device)
        allowed = t[None, :] <= t[:, None]                  # keys up to the query's own position
        if window > 0:                                      # :130: t0 = n - window when n > window, n = pos+1
            allowed &= t[None, :] > t[:, None] - window
        sc = sc.masked_fill(~allowed, float("-inf"))
        m = sc.max(-1, keepdim=True).values                 # :138-140
        e = torch.exp(sc - m)
        w = e / e.sum(-1, keepdim=True)
        out[:, hh, :] = w @ v[:, kvh, :]                    # :141-145
    if gate:                                                # :147-150
        g = rnd(h @ p["gate_proj.weight"].T)
        out = out * sigmoid(g)[:, :, None]
    o = rnd(out.reshape(T, nh * hd))
    return o @ p["out_proj.weight"].T                       # :151


def short_conv(h, p, T, *, D, Lc, rnd=identity, state=None):
    """src/dense.rs:153-170.  bcx = in_proj h; B = bcx[:D], C = bcx[D:2D], x = bcx[2D:];
    bx = B*x; acc_t = sum_k s[k] w[ch,k] + bx_t w[ch,Lc-1] with s the previous Lc-1 values of bx
    (zeros at the start); y = C*acc; out = out_proj y.  The reference has no bias; where the
    checkpoint has `conv.bias` [D] (config key conv_bias) it is the depthwise convolution's own:
    acc_t = bias[ch] + the taps' sum."""
    bcx = rnd(h @ p["in_proj.weight"].T)
    B, C, xg = bcx[:, :D], bcx[:, D:2 * D], bcx[:, 2 * D:]
    bx = B * xg
    w = p["conv.weight"].reshape(D, Lc)
    hist = torch.zeros(Lc - 1, D, dtype=h.dtype, device=h.device) if state is None else state
    padded = torch.cat([hist, bx], dim=0)                   # row t+Lc-1 is token t
    acc = torch.zeros(T, D, dtype=h.dtype, device=h.device)
    if "conv.bias" in p:
        acc = acc + p["conv.bias"][None, :]
    for j in range(Lc):
        acc = acc + padded[j:j + T, :] * w[:, j][None, :]   # tap Lc-1 meets the current token (:163)
    y = rnd(C * acc)
    return y @ p["out_proj.weight"].T, padded[T:, :]


def swiglu_ffn(h, w1, w3, w2, rnd=identity):
    """src/dense.rs:188-191: down(silu(gate h) * (up h))."""
    a = rnd(silu(h @ w1.T) * (h @ w3.T))
    return a @ w2.T


def moe_route(h, wr, bias, k, norm_topk, scaling):
    """Sigmoid router: s = sigmoid(Wr h); choose the k largest s + bias, ties to the lower index
    (the reference's router for its other architecture breaks ties the same way,
    src/cuda/kernels.cu:450); weight s_e / sum of chosen s when norm_topk; times scaling."""
    s = sigmoid(h @ wr.T)
    c = s + (bias if bias is not None else 0.0)
    order = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :k]
    w = torch.gather(s, 1, order)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True)
    return order, w * scaling, c


def moe_ffn(h, p, *, E, k, norm_topk, use_bias, scaling, rnd=identity):
    ids, wts, _ = moe_route(h, p["gate.weight"], p.get("expert_bias") if use_bias else None, k, norm_topk, scaling)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(k):
            e = int(ids[t, j])
            f = swiglu_ffn(h[t:t + 1], p[f"experts.{e}.w1.weight"], p[f"experts.{e}.w3.weight"],
                           p[f"experts.{e}.w2.weight"], rnd)
            out[t] = out[t] + wts[t, j] * f[0]
    return out


# ---- the model ---------------------------------------------------------------------------------
def _sub(tensors, prefix):
    n = len(prefix) + 1
    return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}


def layer_kinds(cfg: dict) -> list[str]:
    if "layer_types" in cfg:
        return ["conv" if t == "conv" else ("sliding" if t == "sliding_attention" else "attention")
                for t in cfg["layer_types"]]
    idx = set(cfg["full_attn_idxs"])
    return ["attention" if i in idx else "conv" for i in range(cfg["num_hidden_layers"])]


def ffn_width(cfg: dict) -> int:
    f = cfg.get("intermediate_size", cfg.get("block_ff_dim"))
    if cfg.get("block_auto_adjust_ff_dim", False):
        f = int(2 * f / 3)
        if cfg.get("block_ffn_dim_multiplier") is not None:
            f = int(cfg["block_ffn_dim_multiplier"] * f)
        mo = cfg.get("block_multiple_of", 1)
        f = mo * ((f + mo - 1) // mo)
    return f


def forward(cfg: dict, tensors: dict[str, torch.Tensor], tokens, rnd=identity, upto_layer=None,
            logit_positions=None):
    """Logits [T, vocab] of one whole sequence (src/dense.rs:171-197, all positions at once), or of
    `logit_positions` only (the output matrix is applied to those rows alone).  Runs where the
    tensors live."""
    D = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim", D // nh)
    eps = cfg.get("norm_eps", 1e-5)
    theta = cfg.get("rope_theta", 10000.0)
    T = len(tokens)
    dev = tensors["embed_tokens.weight"].device
    x = tensors["embed_tokens.weight"][torch.as_tensor(tokens, dtype=torch.long, device=dev)].clone()
    ff_global = tensors.get("rope_freqs.weight")
    sandwich = cfg.get("sandwich_norms", False)
    E = cfg.get("num_experts", 0)
    for l, kind in enumerate(layer_kinds(cfg)):
        if upto_layer is not None and l >= upto_layer:
            break
        p = _sub(tensors, f"layers.{l}")
        h = rnd(rms_norm(x, p["operator_norm.weight"], eps))                      # :180
        if kind == "conv":
            m, _ = short_conv(h, _sub(p, "conv"), T, D=D, Lc=cfg["conv_L_cache"], rnd=rnd)
        else:
            sliding = kind == "sliding"
            m = attention(h, _sub(p, "self_attn"), T, nh=nh, nkv=nkv, hd=hd, eps=eps,
                          theta=cfg.get("rope_theta_swa", 10000.0) if sliding else theta,
                          rope_dim=cfg.get("rope_dim", hd),
                          window=cfg.get("sliding_window", 0) if sliding else 0,
                          gate=cfg.get("attn_output_gate", False), rnd=rnd,
                          freq_factors=None if sliding else ff_global)                # :125
        if sandwich:
            m = rms_norm(m, p["post_mixer_norm.weight"], eps)                     # :185
        x = x + m                                                                 # :186
        h2 = rnd(rms_norm(x, p["ffn_norm.weight"], eps))                          # :187
        ff = _sub(p, "feed_forward")
        if E > 0 and l >= cfg.get("num_dense_layers", 0):
            f = moe_ffn(h2, ff, E=E, k=cfg["num_experts_per_tok"], norm_topk=cfg.get("norm_topk_prob", True),
                        use_bias=cfg.get("use_expert_bias", True), scaling=cfg.get("routed_scaling_factor", 1.0),
                        rnd=rnd)
        else:
            f = swiglu_ffn(h2, ff["w1.weight"], ff["w3.weight"], ff["w2.weight"], rnd)
        if sandwich:
            f = rms_norm(f, p["post_ffn_norm.weight"], eps)                       # :192
        x = x + f                                                                 # :193
    if upto_layer is not None:
        return x
    if logit_positions is not None:
        x = x[torch.as_tensor(logit_positions, dtype=torch.long, device=dev)]
    xn = rnd(rms_norm(x, tensors["embedding_norm.weight"], eps))                  # :195
    tied = cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True))
    wout = tensors["embed_tokens.weight"] if tied else tensors["lm_head.weight"]  # :196
    return xn @ wout.T


# ---- sampling (src/local.rs:57-80) ---------------------------------------------------------------
class XorShift64:
    """src/local.rs:57: s ^= s<<13; s ^= s>>7; s ^= s<<17; (s>>40) / 2^24."""

    def __init__(self, seed=None):
        m = (1 << 64) - 1
        self.s = 0x9E3779B97F4A7C15 if seed is None else ((seed * 0x9E3779B97F4A7C15) & m) | 1   # :244

    def next(self) -> float:
        m = (1 << 64) - 1
        s = self.s
        s ^= (s << 13) & m
        s ^= s >> 7
        s ^= (s << 17) & m
        self.s = s
        return float(np.float32(s >> 40) / np.float32(1 << 24))


def sample(logits: np.ndarray, temperature, top_k, top_p, min_p, u: float) -> int:
    """src/local.rs:59-80 without the penalties; equal logits ordered by lower id first."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature <= 0:
        return int(np.argmax(logits))
    k = 64 if top_k == 0 else min(top_k, 256)
    k = min(k, logits.size)
    order = np.lexsort((np.arange(logits.size), -logits.astype(np.float64)))[:k]
    t = (logits[order] / np.float32(temperature)).astype(np.float32)
    p = np.exp(t - t[0]).astype(np.float32)
    z = np.float32(0)
    for v in p:
        z = np.float32(z + v)
    p = (p / z).astype(np.float32)
    keep, cum = k, np.float32(0)
    for i, v in enumerate(p):
        cum = np.float32(cum + v)
        if 0.0 < top_p < 1.0 and cum >= np.float32(top_p):
            keep = i + 1
            break
    if min_p > 0:
        thr = np.float32(p[0] * np.float32(min_p))
        below = np.nonzero(p < thr)[0]
        keep = max(1, min(keep, int(below[0]) if below.size else k))
    zk = np.float32(0)
    for v in p[:keep]:
        zk = np.float32(zk + v)
    r = np.float32(np.float32(u) * zk)
    for i in range(keep):
        r = np.float32(r - p[i])
        if r <= 0:
            return int(order[i])
    return int(order[keep - 1])
