"""Helpers shared by the tests: tiny model folders, request sets, replay through the engine,
and the error measure."""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

import plain_lfm3 as P  # noqa: E402

# tolerances: max |engine - plain| over max |plain|, per request.  Fixed; never widened to pass.
TOL_F32 = 2e-5
TOL_BF16 = 1.5e-2


def make_model_dir(cfg: dict, seed: int, path: str, router_scale: float = 1.0, freq_factors: bool = False,
                   expert_bias_scale: float = 1.0) -> str:
    """Random model folder; norm weights random around 1 (all-ones would hide a swapped norm);
    router rows scaled so that the experts' scores are well apart (a near-tie would make the
    choice of expert, not the arithmetic, decide the comparison), the experts' selection biases
    scaled to the same end; convolution biases (written as
    zeros) made random; with `freq_factors` the model's optional rotary factors are added."""
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile, save_file
    write_model_dir(cfg, path, seed=seed, dtype="bfloat16", norm_init="random")
    if router_scale != 1.0 or expert_bias_scale != 1.0 or freq_factors or cfg.get("conv_bias", False):
        f = os.path.join(path, "model.safetensors")
        sf = SafetensorsFile(f)
        t = {n: sf.tensor(n).clone() for n in sf.names()}
        g = torch.Generator().manual_seed(1000 + seed)
        for n in sorted(t):
            if n.endswith("feed_forward.gate.weight"):
                t[n] = (t[n].float() * router_scale).to(t[n].dtype)
            if n.endswith("feed_forward.expert_bias"):
                t[n] = t[n] * expert_bias_scale
            if n.endswith("conv.conv.bias"):
                t[n] = (0.004 * torch.randn(t[n].shape, generator=g)).to(t[n].dtype)
        if freq_factors:
            hd = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
            half = cfg.get("rope_dim", hd) // 2
            t["model.rope_freqs.weight"] = 1.0 + 7.0 * torch.rand(half, generator=g)      # 32-bit, as a norm weight would be
        del sf
        save_file(t, f)
    return path


def requests_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


_tensors_on: dict = {}


def plain_tensors(model_dir: str, device: str = "cpu") -> dict:
    """The folder's tensors in double precision as the plain implementation reads them, kept per
    (folder, device).  `device` other than the CPU only moves the same arithmetic to where a model
    of real layer sizes takes seconds instead of minutes."""
    key = (model_dir, device)
    if key not in _tensors_on:
        t = P.read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.float64)
        _tensors_on[key] = t if device == "cpu" else {k: v.to(device) for k, v in t.items()}
    return _tensors_on[key]


def plain_logits(cfg: dict, model_dir: str, tokens, bf16: bool, device: str | None = None) -> torch.Tensor:
    t = plain_tensors(model_dir, device) if device else \
        P.read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.float64)
    return P.forward(cfg, t, tokens, rnd=P.round_bf16 if bf16 else P.identity)


# A router near-tie is a discontinuity: when the chosen and the first rejected expert score
# closer than bfloat16 rounding moves them, rounding decides which expert runs, and the logits
# of that position jump.  Such positions (found by the plain implementation alone) are left
# out of bfloat16 comparisons; in 32-bit every position is compared.
ROUTER_GAP_BF16 = 1e-3
ROUTER_GAP_F32 = 1e-5


def router_gap(bf16: bool, hidden_size: int = 96) -> float:
    """The gap below which a routing decision counts as a near-tie.  A router score is a sum over
    the hidden size of terms that each carry bfloat16 rounding noise, so its noise grows with the
    root of the width: the gap set at a width of 96 is scaled accordingly for wider models."""
    if not bf16:
        return ROUTER_GAP_F32
    return ROUTER_GAP_BF16 * max(1.0, (hidden_size / 96) ** 0.5)


def plain_logits_and_margins(cfg: dict, model_dir: str, tokens, bf16: bool, device: str | None = None):
    """Plain logits [T, V] and, per position, the smallest gap between the last chosen and the
    first rejected expert score over the model's routed layers (inf without experts)."""
    margins = []
    orig = P.moe_route

    def spy(h, wr, bias, k, norm_topk, scaling):
        ids, w, c = orig(h, wr, bias, k, norm_topk, scaling)
        cs = torch.sort(c, dim=-1, descending=True).values
        margins.append(cs[:, k - 1] - cs[:, k] if cs.shape[1] > k
                       else torch.full((cs.shape[0],), float("inf"), dtype=cs.dtype, device=cs.device))
        return ids, w, c
    P.moe_route = spy
    try:
        lg = plain_logits(cfg, model_dir, tokens, bf16, device)
    finally:
        P.moe_route = orig
    m = torch.stack(margins).amin(0) if margins else \
        torch.full((len(tokens),), float("inf"), dtype=torch.float64, device=lg.device)
    return lg, m


def decided(margins: torch.Tensor, bf16: bool, hidden_size: int = 96) -> torch.Tensor:
    """Positions whose routing does not hang on rounding."""
    return margins > router_gap(bf16, hidden_size)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want|, computed where `want` lives."""
    got, want = got.to(want.device).double(), want.double()
    return float((got - want).abs().max() / want.abs().max())


def first_bad_position(got: torch.Tensor, want: torch.Tensor, tol: float) -> int | None:
    got, want = got.to(want.device).double(), want.double()
    e = (got - want).abs().amax(dim=-1) / want.abs().max()
    bad = torch.nonzero(e > tol)
    return int(bad[0]) if bad.numel() else None


# ---- replay through the engine -----------------------------------------------------------------
def to_host(t: torch.Tensor) -> torch.Tensor:
    return t.float().cpu().clone()


def on_device(t: torch.Tensor) -> torch.Tensor:
    """Keeps a step's logits where they are (large vocabularies); the step's buffer is reused."""
    return t.float().clone()


def run_whole(eng, tokens, keep=to_host) -> torch.Tensor:
    s = eng.new_sequence()
    try:
        return keep(eng.step([s], [tokens], [list(range(len(tokens)))]))
    finally:
        eng.release(s)


def run_tail(eng, tokens, tail: int = 32, keep=to_host) -> torch.Tensor:
    """The prompt whole, then the last `tail` tokens one by one."""
    n = len(tokens)
    head = max(1, n - tail)
    s = eng.new_sequence()
    try:
        out = [keep(eng.step([s], [tokens[:head]], [list(range(head))]))]
        for i in range(head, n):
            out.append(keep(eng.step([s], [[tokens[i]]], [[0]])))
        return torch.cat(out, dim=0)
    finally:
        eng.release(s)


def run_batch(eng, requests, prompt_lens, keep=to_host) -> list[torch.Tensor]:
    """All requests start together with prompts of unequal lengths, then one token each per
    step; a request leaves when its tokens are used up.  Returns logits [len, vocab] per request."""
    seqs = [eng.new_sequence() for _ in requests]
    got = [[] for _ in requests]
    live = list(range(len(requests)))
    try:
        lg = keep(eng.step([seqs[i] for i in live], [requests[i][:prompt_lens[i]] for i in live],
                           [list(range(prompt_lens[i])) for i in live]))
        r0 = 0
        for i in live:
            got[i].append(lg[r0:r0 + prompt_lens[i]])
            r0 += prompt_lens[i]
        fed = list(prompt_lens)
        while True:
            done = [i for i in live if fed[i] >= len(requests[i])]
            for i in done:
                eng.release(seqs[i])
                seqs[i] = None
            live = [i for i in live if i not in done]
            if not live:
                break
            lg = keep(eng.step([seqs[i] for i in live], [[requests[i][fed[i]]] for i in live],
                               [[0] for _ in live]))
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                fed[i] += 1
        return [torch.cat(g, dim=0) for g in got]
    finally:
        for s in seqs:
            if s is not None:
                eng.release(s)
