"""Generation through the Python entry point and the replay program, on the GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import harness as H
import plain_lfm3 as P
from tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {"A": H.make_model_dir(TINY_A, 0, str(tmp_path_factory.mktemp("genA"))),
            "B": H.make_model_dir(TINY_B, 1, str(tmp_path_factory.mktemp("genB")))}


def plain_greedy(cfg, model_dir, prompt, n, bf16):
    """Greedy continuation by the plain implementation, with the margin between the two best
    logits at every step (0 where the step's routing hangs on rounding)."""
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        lg, rm = H.plain_logits_and_margins(cfg, model_dir, toks, bf16)
        lg = lg[-1]
        top = torch.topk(lg, 2).values
        margins.append(float((top[0] - top[1]) / lg.abs().max()) if H.decided(rm, bf16)[-1] else 0.0)
        t = int(torch.argmax(lg))
        out.append(t)
        toks.append(t)
    return out, margins


@pytest.mark.parametrize("name,cfg,lens,steps", [("A", TINY_A, [5, 11, 17], 8), ("B", TINY_B, [1, 7, 23, 40], 12)])
@pytest.mark.parametrize("dtype,bf16,gap", [("float32", False, H.TOL_F32), ("bfloat16", True, H.TOL_BF16)])
def test_greedy_generation_matches_plain(name, cfg, lens, steps, dtype, bf16, gap, dirs):
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024)
    prompts = H.requests_for(cfg, lens, 21)
    res = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=steps, stop_token_ids=[])
    compared = 0
    for p, got, reason in zip(prompts, res.tokens, res.finish_reasons):
        want, margins = plain_greedy(cfg, dirs[name], p, steps, bf16)
        assert len(got) == steps and reason == "length"
        for i in range(steps):
            if margins[i] < gap:        # the two best logits are closer than the path's tolerance: stop here
                break
            assert got[i] == want[i], f"{name} {dtype}: prompt of {len(p)}, token {i}: {got[i]} != {want[i]}"
            compared += 1
    assert compared >= steps * len(prompts) // 3
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


def test_sampling_is_seeded_and_independent_of_batching(dirs):
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=1024)
    prompts = H.requests_for(TINY_A, [5, 11, 17, 3, 30], 22)
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=1234)
    a = eng.generate(prompts, sp, max_new_tokens=8, stop_token_ids=[])
    b = eng.generate(prompts, sp, max_new_tokens=8, stop_token_ids=[])
    assert a.tokens == b.tokens
    c = eng.generate(prompts, sp, max_new_tokens=8, stop_token_ids=[], max_batch=2)      # three batches, slots reused
    assert c.tokens == a.tokens and c.stats.batches == 3
    d = eng.generate(prompts, SamplingParams(temperature=0.8, seed=99), max_new_tokens=8, stop_token_ids=[])
    assert d.tokens != a.tokens
    # request 0 of a call draws the reference's numbers: alone it must give the same tokens as in the batch
    e = eng.generate(prompts[:1], sp, max_new_tokens=8, stop_token_ids=[])
    assert e.tokens[0] == a.tokens[0]
    # the first draw follows the plain sampler fed with the plain logits
    tensors = P.read_safetensors(os.path.join(dirs["A"], "model.safetensors"), torch.float64)
    lg = P.forward(TINY_A, tensors, prompts[0])[-1].float().numpy()
    u = P.XorShift64(1234).next()
    assert a.tokens[0][0] == P.sample(lg, 0.8, 40, 0.95, 0.0, u)


def test_stop_tokens_end_requests_early(dirs):
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=1024)
    prompts = H.requests_for(TINY_A, [5, 11, 17, 9], 23)
    free = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=10, stop_token_ids=[])
    stop = free.tokens[1][3]                     # request 1 will hit this at its 4th token
    res = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=10, stop_token_ids=[stop])
    for f, r, reason in zip(free.tokens, res.tokens, res.finish_reasons):
        cut = f.index(stop) if stop in f else len(f)
        assert r == f[:cut]                      # the stop token is not part of the output
        assert reason == ("stop" if stop in f else "length")
    assert eng.cache.slots.n_held == 0
    eng.cache.check()
    # steps launched ahead of the host (graphs) and steps run one by one give the same tokens
    slow = eng.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=10, stop_token_ids=[stop], use_graphs=False)
    assert slow.tokens == res.tokens and slow.finish_reasons == res.finish_reasons
    sp = SamplingParams(temperature=0.9, seed=5)
    assert eng.generate(prompts, sp, max_new_tokens=10, stop_token_ids=[stop]).tokens == \
        eng.generate(prompts, sp, max_new_tokens=10, stop_token_ids=[stop], use_graphs=False).tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_with_a_window_and_early_stops(dtype, tmp_path):
    """The configuration with a sliding window (its pages come and go, so every decode step is staged
    in full), head gate and sandwich norms: generation with steps launched ahead of the host gives
    the tokens of generation step by step, with requests that stop at different times, and with
    a batch limit that makes slots come round again."""
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(H.make_model_dir(TINY_C, 2, str(tmp_path)), dtype=dtype, max_tokens=2048)
    prompts = H.requests_for(TINY_C, [3, 19, 40, 7, 90], 31)
    greedy = SamplingParams(temperature=0.0)
    free = eng.generate(prompts, greedy, max_new_tokens=24, stop_token_ids=[], use_graphs=False)
    stops = [free.tokens[1][5], free.tokens[3][11]]
    for sp in (greedy, SamplingParams(temperature=0.9, top_k=20, seed=4)):
        slow = eng.generate(prompts, sp, max_new_tokens=24, stop_token_ids=stops, use_graphs=False)
        fast = eng.generate(prompts, sp, max_new_tokens=24, stop_token_ids=stops)
        assert fast.tokens == slow.tokens and fast.finish_reasons == slow.finish_reasons
        assert "stop" in fast.finish_reasons and len({len(t) for t in fast.tokens}) > 1     # they end at different times
        two = eng.generate(prompts, sp, max_new_tokens=24, stop_token_ids=stops, max_batch=2)
        assert two.tokens == slow.tokens and two.stats.batches == 3
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


def test_penalties_on_the_device_match_the_step_by_step_path(dirs):
    """Repeat and presence penalties in captured decode steps (rings of recent tokens on the device,
    fed by the steps themselves) against the path that builds every step's history on the host; long
    enough for the 256-token rings to wrap, prompts longer and shorter than the window."""
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=4096)
    prompts = H.requests_for(TINY_A, [5, 300, 17], 41)
    for sp in (SamplingParams(temperature=0.0, repeat_penalty=1.3, presence_penalty=0.4),
               SamplingParams(temperature=0.8, top_k=30, seed=9, repeat_penalty=1.15)):
        slow = eng.generate(prompts, sp, max_new_tokens=290, stop_token_ids=[], use_graphs=False)
        fast = eng.generate(prompts, sp, max_new_tokens=290, stop_token_ids=[])
        assert fast.tokens == slow.tokens
        plain = eng.generate(prompts, SamplingParams(temperature=sp.temperature, top_k=sp.top_k, seed=sp.seed),
                             max_new_tokens=40, stop_token_ids=[])
        assert plain.tokens[0] != fast.tokens[0][:40]           # the penalties do change what is chosen
    assert eng.cache.slots.n_held == 0


def run_trace(model_dir, dtype, steps, out_dir, max_tokens=1024):
    exe = os.path.join(H.ROOT, "bin", "trace_run")
    p = subprocess.run([sys.executable, exe, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens)],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype,bf16,tol", [("float32", False, H.TOL_F32), ("bfloat16", True, H.TOL_BF16)])
def test_trace_run_program(dtype, bf16, tol, dirs, tmp_path):
    """The replay program on a trace with a whole request, a request decoded at its end, and two
    unequal batches one after another; logits compared with the plain implementation."""
    cfg = TINY_B
    reqs = dict(zip("abcdefg", H.requests_for(cfg, [40, 50, 7, 23, 1, 30, 12], 24)))
    steps, n = [], 0
    expect = []   # (step, [(request, positions)])

    def add(entries, end=()):
        nonlocal n
        steps.append({"step": n, "entries": [{"id": r, "tokens": reqs[r][lo:hi], "want": list(range(hi - lo)) if w else []}
                                             for r, lo, hi, w in entries], "end": list(end)})
        if any(w for *_, w in entries):
            expect.append((n, [(r, list(range(lo, hi))) for r, lo, hi, w in entries if w]))
        n += 1
    add([("a", 0, 40, True)], end=["a"])
    add([("b", 0, 18, False)])                                   # nothing wanted: no file
    for i in range(18, 50):
        add([("b", i, i + 1, True)], end=["b"] if i == 49 else [])
    fed = {"c": 5, "d": 20, "e": 1}
    add([(r, 0, fed[r], True) for r in "cde"], end=["e"])
    live = ["c", "d"]
    while live:
        ent = [(r, fed[r], fed[r] + 1, True) for r in live]
        for r in live:
            fed[r] += 1
        ended = [r for r in live if fed[r] >= len(reqs[r])]
        add(ent, end=ended)
        live = [r for r in live if r not in ended]
    add([("f", 0, 30, True), ("g", 0, 12, True)], end=["f", "g"])   # the next batch reuses slots and pages
    out = str(tmp_path / "out")
    run_trace(dirs["B"], dtype, steps, out, max_tokens=256)
    assert not os.path.exists(os.path.join(out, "1.f32"))
    V = cfg["vocab_size"]
    plain = {r: H.plain_logits_and_margins(cfg, dirs["B"], t, bf16) for r, t in reqs.items()}
    n_cmp = n_all = 0
    for step, parts in expect:
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, V))
        want = torch.cat([plain[r][0][pos] for r, pos in parts])
        keep = torch.cat([H.decided(plain[r][1][pos], bf16) for r, pos in parts])
        assert got.shape == want.shape
        n_cmp, n_all = n_cmp + int(keep.sum()), n_all + keep.numel()
        if keep.any():
            assert H.rel_err(got[keep], want[keep]) <= tol, f"step {step}: {H.rel_err(got[keep], want[keep]):.3e}"
    assert n_cmp >= 0.9 * n_all
