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


def make_model_dir(cfg: dict, seed: int, path: str, router_scale: float = 1.0) -> str:
    """Random model folder; norm weights random around 1 (all-ones would hide a swapped norm);
    router rows scaled so that the experts' scores are well apart (a near-tie would make the
    choice of expert, not the arithmetic, decide the comparison)."""
    from lastengine_b200.weights import write_model_dir
    from lastengine_b200.weights.safetensors_io import SafetensorsFile, save_file
    write_model_dir(cfg, path, seed=seed, dtype="bfloat16", norm_init="random")
    if router_scale != 1.0:
        f = os.path.join(path, "model.safetensors")
        sf = SafetensorsFile(f)
        t = {n: sf.tensor(n).clone() for n in sf.names()}
        for n in t:
            if n.endswith("feed_forward.gate.weight"):
                t[n] = (t[n].float() * router_scale).to(t[n].dtype)
        del sf
        save_file(t, f)
    return path


def requests_for(cfg: dict, lengths, seed: int) -> list[list[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


def plain_logits(cfg: dict, model_dir: str, tokens, bf16: bool) -> torch.Tensor:
    t = P.read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.float64)
    return P.forward(cfg, t, tokens, rnd=P.round_bf16 if bf16 else P.identity)


# A router near-tie is a discontinuity: when the chosen and the first rejected expert score
# closer than bfloat16 rounding moves them, rounding decides which expert runs, and the logits
# of that position jump.  Such positions (found by the plain implementation alone) are left
# out of bfloat16 comparisons; in 32-bit every position is compared.
ROUTER_GAP_BF16 = 1e-3
ROUTER_GAP_F32 = 1e-5


def plain_logits_and_margins(cfg: dict, model_dir: str, tokens, bf16: bool):
    """Plain logits [T, V] and, per position, the smallest gap between the last chosen and the
    first rejected expert score over the model's routed layers (inf without experts)."""
    margins = []
    orig = P.moe_route

    def spy(h, wr, bias, k, norm_topk, scaling):
        ids, w, c = orig(h, wr, bias, k, norm_topk, scaling)
        cs = torch.sort(c, dim=-1, descending=True).values
        margins.append(cs[:, k - 1] - cs[:, k] if cs.shape[1] > k else torch.full((cs.shape[0],), float("inf")))
        return ids, w, c
    P.moe_route = spy
    try:
        lg = plain_logits(cfg, model_dir, tokens, bf16)
    finally:
        P.moe_route = orig
    m = torch.stack(margins).amin(0) if margins else torch.full((len(tokens),), float("inf"), dtype=torch.float64)
    return lg, m


def decided(margins: torch.Tensor, bf16: bool) -> torch.Tensor:
    """Positions whose routing does not hang on rounding."""
    return margins > (ROUTER_GAP_BF16 if bf16 else ROUTER_GAP_F32)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max())


def first_bad_position(got: torch.Tensor, want: torch.Tensor, tol: float) -> int | None:
    got, want = got.double().cpu(), want.double().cpu()
    e = (got - want).abs().amax(dim=-1) / want.abs().max()
    bad = torch.nonzero(e > tol)
    return int(bad[0]) if bad.numel() else None


# ---- replay through the engine -----------------------------------------------------------------
def run_whole(eng, tokens) -> torch.Tensor:
    s = eng.new_sequence()
    try:
        return eng.step([s], [tokens], [list(range(len(tokens)))]).float().cpu().clone()
    finally:
        eng.release(s)


def run_tail(eng, tokens, tail: int = 32) -> torch.Tensor:
    """The prompt whole, then the last `tail` tokens one by one."""
    n = len(tokens)
    head = max(1, n - tail)
    s = eng.new_sequence()
    try:
        out = [eng.step([s], [tokens[:head]], [list(range(head))]).float().cpu().clone()]
        for i in range(head, n):
            out.append(eng.step([s], [[tokens[i]]], [[0]]).float().cpu().clone())
        return torch.cat(out, dim=0)
    finally:
        eng.release(s)


def run_batch(eng, requests, prompt_lens) -> list[torch.Tensor]:
    """All requests start together with prompts of unequal lengths, then one token each per
    step; a request leaves when its tokens are used up.  Returns logits [len, vocab] per request."""
    seqs = [eng.new_sequence() for _ in requests]
    got = [[] for _ in requests]
    live = list(range(len(requests)))
    try:
        lg = eng.step([seqs[i] for i in live], [requests[i][:prompt_lens[i]] for i in live],
                      [list(range(prompt_lens[i])) for i in live]).float().cpu().clone()
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
            lg = eng.step([seqs[i] for i in live], [[requests[i][fed[i]]] for i in live],
                          [[0] for _ in live]).float().cpu().clone()
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                fed[i] += 1
        return [torch.cat(g, dim=0) for g in got]
    finally:
        for s in seqs:
            if s is not None:
                eng.release(s)
