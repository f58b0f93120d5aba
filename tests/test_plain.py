"""The plain implementation checked against itself and against hand-made cases (no GPU)."""
import math

import numpy as np
import torch

import harness as H
import plain_lfm3 as P
from tiny_configs import TINY_A, TINY_B


def test_rms_norm_and_silu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.5)
    r = 1 / math.sqrt((9 + 16) / 2 + 0.5)
    assert torch.allclose(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))
    assert abs(float(P.silu(torch.tensor(1.0))) - 1 / (1 + math.exp(-1))) < 1e-7


def test_rope_pairs_and_angles():
    v = torch.arange(8, dtype=torch.float64).view(1, 1, 8) + 1
    out = P.rope(v, torch.tensor([3]), 4, 100.0)           # rotates dims (0,2) and (1,3); 4..7 untouched
    th0, th1 = 3.0, 3.0 * 100.0 ** (-0.5)
    assert torch.allclose(out[0, 0, 0], torch.tensor(1 * math.cos(th0) - 3 * math.sin(th0), dtype=torch.float64))
    assert torch.allclose(out[0, 0, 2], torch.tensor(1 * math.sin(th0) + 3 * math.cos(th0), dtype=torch.float64))
    assert torch.allclose(out[0, 0, 3], torch.tensor(2 * math.sin(th1) + 4 * math.cos(th1), dtype=torch.float64))
    assert torch.equal(out[0, 0, 4:], v[0, 0, 4:])
    adj = P.rope(v, torch.tensor([3]), 4, 100.0, neox=False)   # pairs (0,1) and (2,3)
    assert torch.allclose(adj[0, 0, 1], torch.tensor(1 * math.sin(th0) + 2 * math.cos(th0), dtype=torch.float64))


def test_short_conv_equals_token_by_token_recurrence():
    """The whole-sequence convolution against the reference's one-token update (src/dense.rs:153-170)."""
    D, Lc, T = 6, 4, 9
    g = torch.Generator().manual_seed(0)
    p = {"in_proj.weight": torch.randn(3 * D, D, generator=g, dtype=torch.float64),
         "conv.weight": torch.randn(D, 1, Lc, generator=g, dtype=torch.float64),
         "out_proj.weight": torch.randn(D, D, generator=g, dtype=torch.float64)}
    h = torch.randn(T, D, generator=g, dtype=torch.float64)
    whole, _ = P.short_conv(h, p, T, D=D, Lc=Lc)
    w = p["conv.weight"].reshape(D, Lc)
    s = torch.zeros(D, Lc - 1, dtype=torch.float64)
    rows = []
    for t in range(T):
        bcx = p["in_proj.weight"] @ h[t]
        y = torch.zeros(D, dtype=torch.float64)
        for ch in range(D):
            bx = bcx[ch] * bcx[2 * D + ch]
            acc = bx * w[ch, Lc - 1]
            for k in range(Lc - 1):
                acc = acc + s[ch, k] * w[ch, k]
            for k in range(Lc - 2):
                s[ch, k] = s[ch, k + 1]
            s[ch, Lc - 2] = bx
            y[ch] = bcx[D + ch] * acc
        rows.append(p["out_proj.weight"] @ y)
    assert torch.allclose(whole, torch.stack(rows), atol=1e-12)
    # and carried state: two halves equal the whole
    a, st = P.short_conv(h[:4], p, 4, D=D, Lc=Lc)
    b, _ = P.short_conv(h[4:], p, T - 4, D=D, Lc=Lc, state=st)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)


def test_attention_equals_token_by_token_with_growing_keys():
    """Whole-sequence attention against the reference's one-token form with an appended cache."""
    nh, nkv, hd, D, T = 4, 2, 8, 12, 7
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)   # noqa: E731
    p = {"q_proj.weight": r(nh * hd, D), "k_proj.weight": r(nkv * hd, D), "v_proj.weight": r(nkv * hd, D),
         "out_proj.weight": r(D, nh * hd), "q_layernorm.weight": r(hd), "k_layernorm.weight": r(hd)}
    h = r(T, D)
    for window in (0, 3):
        whole = P.attention(h, p, T, nh=nh, nkv=nkv, hd=hd, eps=1e-5, theta=100.0, rope_dim=hd, window=window)
        kc, vc, rows = [], [], []
        for pos in range(T):
            q = P.rms_norm((p["q_proj.weight"] @ h[pos]).view(nh, hd), p["q_layernorm.weight"], 1e-5)
            k = P.rms_norm((p["k_proj.weight"] @ h[pos]).view(nkv, hd), p["k_layernorm.weight"], 1e-5)
            q = P.rope(q[None], torch.tensor([pos]), hd, 100.0)[0]
            kc.append(P.rope(k[None], torch.tensor([pos]), hd, 100.0)[0])
            vc.append((p["v_proj.weight"] @ h[pos]).view(nkv, hd))
            n = pos + 1
            t0 = n - window if window and n > window else 0
            o = torch.zeros(nh, hd, dtype=torch.float64)
            for hh in range(nh):
                sc = torch.stack([kc[t][hh // 2] @ q[hh] / math.sqrt(hd) for t in range(t0, n)])
                w = torch.softmax(sc, 0)
                o[hh] = sum(w[i] * vc[t][hh // 2] for i, t in enumerate(range(t0, n)))
            rows.append(p["out_proj.weight"] @ o.reshape(-1))
        assert torch.allclose(whole, torch.stack(rows), atol=1e-10)


def test_router_choice_weights_and_ties():
    h = torch.eye(3, dtype=torch.float64)
    wr = torch.tensor([[1.0, 0, 0], [1.0, 0, 0], [0, 2.0, 0], [0, 0, -1.0]], dtype=torch.float64)
    ids, w, _ = P.moe_route(h, wr, None, 2, True, 1.0)
    assert ids[0].tolist() == [0, 1]                 # a tie: lower index first
    assert torch.allclose(w[0], torch.tensor([0.5, 0.5], dtype=torch.float64))
    assert ids[1].tolist()[0] == 2
    bias = torch.tensor([0.0, 0.0, 0.0, 10.0], dtype=torch.float64)
    ids, w, _ = P.moe_route(h, wr, bias, 1, False, 2.0)
    assert ids[:, 0].tolist() == [3, 3, 3]           # the bias chooses ...
    s = 1 / (1 + math.exp(1.0))
    assert abs(float(w[2, 0]) - 2.0 * s) < 1e-12     # ... but does not weigh


def test_forward_shapes_prefix_property_and_bf16_distance(tmp_path):
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1)):
        d = H.make_model_dir(cfg, seed, str(tmp_path / f"m{seed}"))
        toks = H.requests_for(cfg, [30], 3)[0]
        full = H.plain_logits(cfg, d, toks, False)
        assert full.shape == (30, cfg["vocab_size"]) and torch.isfinite(full).all()
        part = H.plain_logits(cfg, d, toks[:13], False)
        assert torch.allclose(part, full[:13], atol=1e-10)      # causal: a prefix gives the same logits
        bf = H.plain_logits(cfg, d, toks, True)
        assert 1e-5 < H.rel_err(bf, full) < 3e-2


def test_sampler_by_hand():
    lg = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    assert P.sample(lg, 0.0, 40, 0.95, 0.0, 0.9) == 0
    assert [P.sample(lg, 1.0, 40, 1.0, 0.0, u) for u in (0.1, 0.6, 0.9, 0.99)] == [0, 1, 2, 3]
    assert [P.sample(lg, 1.0, 2, 1.0, 0.0, u) for u in (0.1, 0.7)] == [0, 1]            # top-2: 0.625 / 0.375
    assert P.sample(lg, 1.0, 40, 0.7, 0.0, 0.99) == 1                                   # top-p keeps {0,1}
    assert P.sample(lg, 1.0, 40, 1.0, 0.4, 0.99) == 1                                   # min-p 0.4*0.5 cuts 0.15


def test_short_conv_against_the_references_own_kernels():
    """tests/golden/shortconv_golden.npz holds inputs and outputs of the reference's two
    short-convolution kernels (made by tests/golden/make_shortconv_golden.py from the reference
    checkout).  With identity projections the plain convolution must reproduce them: the B/C/x
    split order, the tap order, and the state layout (oldest value first)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "shortconv_golden.npz"))
    for case in range(3):
        bcx, w = torch.from_numpy(g[f"bcx{case}"]).double(), torch.from_numpy(g[f"w{case}"]).double()
        T, n = bcx.shape[0], w.shape[0]
        lc = w.shape[1]
        # in_proj: the plain function computes bcx = h @ in_proj^T; feed bcx itself through a selector
        p = {"in_proj.weight": torch.eye(3 * n, dtype=torch.float64), "conv.weight": w.reshape(n, 1, lc),
             "out_proj.weight": torch.eye(n, dtype=torch.float64)}
        # the reference's state is [channel][oldest..newest]; the plain function carries rows of time
        st_in = torch.from_numpy(g[f"state_in{case}"]).double().T.contiguous()
        # identity projections: the 3n-wide input rows are (B, C, x) themselves
        out, st = P.short_conv(bcx, p, T, D=n, Lc=lc, state=st_in)
        assert torch.allclose(out, torch.from_numpy(g[f"y{case}"]).double(), atol=1e-5)
        assert torch.allclose(st.T, torch.from_numpy(g[f"state_out{case}"]).double(), atol=1e-6)


def test_norm_swiglu_rotation_and_attention_against_the_references_own_kernels():
    """tests/golden/dense_kernels_golden.npz holds inputs and outputs of the reference's `rmsnorm`,
    `swiglu_gu`, `dn_prep` and `dn_attn` kernels, run unchanged on a GPU by
    tests/golden/make_dense_kernels_golden.py.  The plain functions must reproduce them: eps inside
    the root; silu(gate) * up over [gate | up] rows; the per-head norm before the rotation, both
    pairings, a rotation over part of the head, frequency factors; in attention the kv head of a
    query head, the scale, the window's first key, the head gate.  The reference keeps cached keys
    and values in 16-bit floats and uses the fast exponential, hence 2e-3 for the attention chain."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dense_kernels_golden.npz"))
    t64 = lambda name: torch.from_numpy(g[name]).double()
    rel = lambda got, want: float((got - want).abs().max() / want.abs().max())
    for case in range(3):
        y = P.rms_norm(t64(f"norm_x{case}"), t64(f"norm_w{case}"), float(g[f"norm_eps{case}"]))
        assert rel(y, t64(f"norm_y{case}")) < 1e-5
    gu = t64("swiglu_gu")
    ffn = gu.shape[1] // 2
    assert rel(P.silu(gu[:, :ffn]) * gu[:, ffn:], t64("swiglu_y")) < 1e-5
    n_prep = sum(1 for k in g.files if k.startswith("prep_x"))
    assert n_prep == 5
    for case in range(n_prep):
        heads, hd, rd, neox, pos0, T = (int(v) for v in g[f"prep_meta{case}"])
        x = t64(f"prep_x{case}")
        if f"prep_nw{case}" in g.files:
            x = P.rms_norm(x, t64(f"prep_nw{case}"), 1e-5)                  # the norm comes first
        ff = t64(f"prep_ff{case}") if f"prep_ff{case}" in g.files else None
        y = P.rope(x, torch.arange(pos0, pos0 + T), rd, float(g[f"prep_base{case}"]), neox=bool(neox), freq_factors=ff)
        assert rel(y, t64(f"prep_y{case}")) < 2e-5, case     # float angles: positions up to 40 times base^0
    n_attn = sum(1 for k in g.files if k.startswith("attn_o"))
    assert n_attn == 5
    for case in range(n_attn):
        nh, nkv, hd, rd, win, T = (int(v) for v in g[f"attn_meta{case}"])
        q, k, v = (t64(f"attn_{n}{case}").reshape(T, -1) for n in "qkv")
        gate = t64(f"attn_gate{case}") if f"attn_gate{case}" in g.files else None
        cols = [q, k, v] + ([gate] if gate is not None else [])
        h = torch.cat(cols, dim=1)                                        # the projections only pick columns
        D, o0 = h.shape[1], 0
        p = {}
        for name, width in (("q_proj", nh * hd), ("k_proj", nkv * hd), ("v_proj", nkv * hd), ("gate_proj", nh if gate is not None else 0)):
            if width:
                w = torch.zeros(width, D, dtype=torch.float64)
                w[torch.arange(width), o0 + torch.arange(width)] = 1.0
                p[f"{name}.weight"] = w
                o0 += width
        p["q_layernorm.weight"], p["k_layernorm.weight"] = t64(f"attn_qn{case}"), t64(f"attn_kn{case}")
        p["out_proj.weight"] = torch.eye(nh * hd, dtype=torch.float64)
        ff = t64(f"attn_ff{case}") if f"attn_ff{case}" in g.files else None
        o = P.attention(h, p, T, nh=nh, nkv=nkv, hd=hd, eps=1e-5, theta=float(g[f"attn_base{case}"]), rope_dim=rd,
                        window=win, gate=gate is not None, freq_factors=ff)
        assert rel(o, t64(f"attn_o{case}").reshape(T, nh * hd)) < 2e-3, case
