"""The step function's edges on the GPU: steps that cannot run, steps cut into pieces, a kernel
that gave up on a bounded wait, a step launched ahead that finds no cache room, and decode
graphs whose page tables follow the live sequences instead of the cache's capacity."""
import numpy as np
import pytest
import torch

import harness as H
from tiny_configs import TINY_A, TINY_B

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {"A": H.make_model_dir(TINY_A, 0, str(tmp_path_factory.mktemp("engA"))),
            "B": H.make_model_dir(TINY_B, 1, str(tmp_path_factory.mktemp("engB")))}


def test_steps_that_cannot_run_raise_and_change_nothing(dirs):
    from lastengine_b200 import Engine, StepError
    from lastengine_b200.cache import CacheFull
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=256, max_seqs=4)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([a], [[1, 2, 3]], None)
    gone = eng.new_sequence()
    eng.release(gone)
    cases = [
        (([a, b], [[1]]), "as many token lists as sequences"),
        (([], []), "at least one"),
        (([a, a], [[1], [2]]), "appears twice"),
        (([a, b], [[1], []]), "brings no tokens"),
        (([gone], [[1]]), "not live"),
        (([a], [[1, 256]]), "token id 256"),
        (([a], [[-1]]), "token id -1"),
    ]
    for (seqs, toks), needle in cases:
        with pytest.raises(StepError, match=needle):
            eng.step(seqs, toks)
    with pytest.raises(StepError, match="one list of places per sequence"):
        eng.step([a, b], [[1], [2]], [[0]])
    with pytest.raises(StepError, match="wanted place 2"):
        eng.step([a, b], [[1], [2, 3]], [[0], [2]])
    with pytest.raises(CacheFull):                                # 4 pages of 64: a and b cannot hold 200 + 100
        eng.step([a, b], [[5] * 200, [6] * 100])
    assert eng.length(a) == 3 and eng.length(b) == 0              # nothing ran, nothing was reserved
    eng.cache.check()
    assert sum(len(p) for g in eng.cache.kv_groups for p in g.seq_pages.values()) == len(eng.cache.kv_groups)
    # places may be asked for in any order and come back in that order
    toks = H.requests_for(TINY_A, [20], 3)[0]
    up = eng.step([b], [toks], [[3, 7, 19]]).clone()
    eng.release([a, b])
    c = eng.new_sequence()
    down = eng.step([c], [toks], [[19, 3, 7]]).clone()
    eng.release(c)
    assert torch.equal(down, up[[2, 0, 1]])
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("name,dtype,bf16,tol", [("B", "float32", False, H.TOL_F32), ("A", "float32", False, H.TOL_F32),
                                                ("A", "bfloat16", True, H.TOL_BF16)])
def test_a_step_longer_than_max_batch_tokens_runs_in_pieces(name, dtype, bf16, tol, dirs):
    """Three prompts of 130, 7 and 65 tokens with at most 50 rows per pass: five pieces, two of
    them cutting a sequence; all logits as from one pass, and as the plain implementation's.
    The model with experts is compared in 32-bit only: in bfloat16 pieces of 50 rows and a pass of
    202 rows round at different places (the split norms of steps of up to 128 rows), a router
    near-tie at an early position then falls the other way in one of the two, and the keys of that
    position carry the difference to every later one."""
    from lastengine_b200 import Engine, EngineOptions, SamplingParams
    cfg = {"A": TINY_A, "B": TINY_B}[name]
    reqs = H.requests_for(cfg, [130, 7, 65], 61)
    small = Engine.from_pretrained(dirs[name], EngineOptions(dtype=dtype, max_tokens=1024, max_batch_tokens=50))
    large = Engine.from_pretrained(dirs[name], dtype=dtype, max_tokens=1024)
    got = {}
    for which, eng in (("pieces", small), ("whole", large)):
        seqs = [eng.new_sequence() for _ in reqs]
        lg = eng.step(seqs, reqs, [list(range(len(r))) for r in reqs], check=True).float().cpu().clone()
        last = eng.step(seqs, [[1], [2], [3]], "last").float().cpu().clone()       # the cache is what one pass leaves
        eng.release(seqs)
        got[which] = (lg, last)
    r0 = 0
    for r in reqs:
        want, m = H.plain_logits_and_margins(cfg, dirs[name], r, bf16)
        assert H.decided(m, bf16).all()
        assert H.rel_err(got["pieces"][0][r0:r0 + len(r)], want) <= tol
        r0 += len(r)
    if not bf16:
        # 32-bit: the pieces change no result beyond rounding (the sums run in the same order)
        assert H.rel_err(got["pieces"][0], got["whole"][0]) <= 2e-6
        assert H.rel_err(got["pieces"][1], got["whole"][1]) <= 2e-6
    # generation starts its prompts through the same pieces
    greedy = SamplingParams(temperature=0.0)
    a = small.generate(reqs, greedy, max_new_tokens=6, stop_token_ids=[])
    b = large.generate(reqs, greedy, max_new_tokens=6, stop_token_ids=[])
    if not bf16:
        assert a.tokens == b.tokens
    assert small.cache.slots.n_held == 0 and large.cache.slots.n_held == 0
    small.cache.check()


def test_a_kernel_that_gave_up_is_reported_where_the_tokens_are_read(dirs):
    """A block waits with the products' own bounded wait on a barrier nobody arrives on: it gives up
    after 2,000 polls, sets the status word and returns (no fault, the context stays usable).  The
    engine reports that at the next place where it reads a step's result, and goes on afterwards."""
    from lastengine_b200 import Engine, SamplingParams
    from lastengine_b200.ops import kernels
    eng = Engine.from_pretrained(dirs["A"], dtype="bfloat16", max_tokens=1024)
    prompts = H.requests_for(TINY_A, [9, 30], 62)
    greedy = SamplingParams(temperature=0.0)
    want = eng.generate(prompts, greedy, max_new_tokens=8, stop_token_ids=[]).tokens
    eng.check_status()
    # 1. the step function with check=True
    kernels.selftest_bounded_wait(eng.device, limit=2000, role=9)
    s = eng.new_sequence()
    with pytest.raises(kernels.KernelError, match="gave up waiting \\(role 9\\)"):
        eng.step([s], [prompts[0]], "last", check=True)
    eng.release(s)
    eng.check_status()                                  # the word was cleared when it was reported
    # 2. generation with captured steps launched ahead, and step by step
    for use_graphs in (True, False):
        kernels.selftest_bounded_wait(eng.device, limit=2000, role=7)
        with pytest.raises(kernels.KernelError, match="role 7"):
            eng.generate(prompts, greedy, max_new_tokens=8, stop_token_ids=[], use_graphs=use_graphs)
        assert eng.cache.slots.n_held == 0              # the failed call left no sequence behind
        eng.cache.check()
        assert eng.generate(prompts, greedy, max_new_tokens=8, stop_token_ids=[], use_graphs=use_graphs).tokens == want
    with pytest.raises(kernels.KernelError, match="limit"):
        kernels.selftest_bounded_wait(eng.device, limit=1 << 20)


def test_a_step_launched_ahead_that_finds_no_cache_room(dirs):
    """Two pages in all, one of them held by another sequence: generation from a 60-token prompt
    wants a second page at its fifth token.  The step launched ahead meets CacheFull and is
    dropped; the step asked for next raises it; the call gives its sequence back.  With the
    other sequence gone the same call runs through, graphs on and off alike."""
    from lastengine_b200 import Engine, SamplingParams
    from lastengine_b200.cache import CacheFull
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=128, max_seqs=2)
    prompt = H.requests_for(TINY_A, [60], 63)
    greedy = SamplingParams(temperature=0.0)
    blocker = eng.new_sequence()
    eng.step([blocker], [[1, 2, 3]], None)
    for use_graphs in (True, False):
        with pytest.raises(CacheFull):
            eng.generate(prompt, greedy, max_new_tokens=12, stop_token_ids=[], use_graphs=use_graphs)
        assert eng.cache.slots.n_held == 1 and eng.length(blocker) == 3
        eng.cache.check()
    eng.release(blocker)
    fast = eng.generate(prompt, greedy, max_new_tokens=12, stop_token_ids=[])
    slow = eng.generate(prompt, greedy, max_new_tokens=12, stop_token_ids=[], use_graphs=False)
    assert fast.tokens == slow.tokens and len(fast.tokens[0]) == 12
    assert eng.cache.slots.n_held == 0


def test_decode_graphs_follow_the_live_lengths_not_the_cache_size(dirs):
    """An engine with room for 65,536 tokens: a sequence of about 100 tokens decodes with page
    tables of 2 pages, so the decode attention is chosen for 128 positions and runs unsplit; as
    the sequence grows past 128 and 256 tokens wider graphs take over, with the tokens of the
    path without graphs."""
    from lastengine_b200 import Engine, SamplingParams
    from lastengine_b200.ops import kernels
    eng = Engine.from_pretrained(dirs["A"], dtype="float32", max_tokens=65536, max_seqs=8)
    greedy = SamplingParams(temperature=0.0)
    prompts = H.requests_for(TINY_A, [100, 40], 64)
    splits = []
    orig = kernels.attention_splits
    kernels.attention_splits = lambda batch, nkv, G, **kw: splits.append((batch.max_kvlen, orig(batch, nkv, G, **kw))) or splits[-1][1]
    try:
        res = eng.generate(prompts, greedy, max_new_tokens=20, stop_token_ids=[])
    finally:
        kernels.attention_splits = orig
    graphs = eng._decode_graphs[greedy]
    widths = sorted(k[1] for k in graphs if isinstance(k, tuple) and isinstance(k[0], int))
    assert widths == [2], widths
    decode_calls = [s for s in splits if s[0] <= 128]
    assert decode_calls and all(n == 1 for _, n in decode_calls), splits
    long = eng.generate(prompts, greedy, max_new_tokens=180, stop_token_ids=[])
    widths = sorted({k[1] for k in graphs if isinstance(k, tuple) and isinstance(k[0], int)})
    assert widths == [2, 4, 8], widths
    slow = eng.generate(prompts, greedy, max_new_tokens=180, stop_token_ids=[], use_graphs=False)
    assert long.tokens == slow.tokens and long.tokens[0][:20] == res.tokens[0]
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_run_as_captured_steps(dtype, dirs):
    """Prompts of a few hundred tokens in all are a captured step too (buckets of rows and of
    sequences, padded with sequences that hold no slot): the same tokens as the uncaptured path,
    the buckets used again by later calls, longer prompts and sampling with penalties uncaptured."""
    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained(dirs["A"], dtype=dtype, max_tokens=8192, max_seqs=16)
    greedy = SamplingParams(temperature=0.0)
    cases = [[5], [31], [3, 40, 17], [1, 1], [9, 2, 2, 7, 30, 1, 12, 25], [200], [300, 100, 60], [129, 64, 64, 1]]
    agree = total = 0
    for k, lens in enumerate(cases):
        prompts = H.requests_for(TINY_A, lens, 70 + k)
        a = eng.generate(prompts, greedy, max_new_tokens=5, stop_token_ids=[], use_graphs=True)
        b = eng.generate(prompts, greedy, max_new_tokens=5, stop_token_ids=[], use_graphs=False)
        agree += sum(x == y for x, y in zip(a.tokens, b.tokens))
        total += len(lens)
        assert eng.cache.slots.n_held == 0
    assert agree == total if dtype == "float32" else agree >= total - 2, (agree, total)
    keys = sorted(k[1:] for k in eng._decode_graphs[greedy] if isinstance(k, tuple) and k[0] == "prompts")
    assert sorted({(r, b) for r, b, w in keys}) == [(32, 1), (32, 2), (64, 4), (128, 8), (256, 1), (512, 4)], keys
    before = len(eng._decode_graphs[greedy])
    eng.generate(H.requests_for(TINY_A, [20, 8], 90), greedy, max_new_tokens=3, stop_token_ids=[])
    assert len(eng._decode_graphs[greedy]) == before            # (32, 2) again: nothing new is captured
    eng.generate(H.requests_for(TINY_A, [400, 200], 91), greedy, max_new_tokens=3, stop_token_ids=[])
    assert not any(isinstance(k, tuple) and k[0] == "prompts" and k[1] > 512 for k in eng._decode_graphs[greedy])
    # sampling with a temperature: the uniform numbers reach the captured prompt step as they reach the plain one
    warm = SamplingParams(temperature=0.8, top_k=20, seed=3)
    u = eng.generate(H.requests_for(TINY_A, [20, 8, 33], 93), warm, max_new_tokens=6, stop_token_ids=[], use_graphs=True)
    v = eng.generate(H.requests_for(TINY_A, [20, 8, 33], 93), warm, max_new_tokens=6, stop_token_ids=[], use_graphs=False)
    assert u.tokens == v.tokens or dtype == "bfloat16"
    assert any(isinstance(k, tuple) and k[0] == "prompts" for k in eng._decode_graphs[warm])
    pen = SamplingParams(temperature=0.0, repeat_penalty=1.3)
    x = eng.generate(H.requests_for(TINY_A, [20, 8], 92), pen, max_new_tokens=4, stop_token_ids=[], use_graphs=True)
    y = eng.generate(H.requests_for(TINY_A, [20, 8], 92), pen, max_new_tokens=4, stop_token_ids=[], use_graphs=False)
    assert x.tokens == y.tokens or dtype == "bfloat16"
    assert not any(isinstance(k, tuple) and k[0] == "prompts" for k in eng._decode_graphs.get(pen, {}))
    eng.cache.check()


def test_split_norm_is_offered_only_where_the_reader_can_scale_its_rows():
    """A feed-forward so wide (gate and up together 38,016 rows) that the sliced product of 17-128
    rows does not take it: a decode step of 32 sequences must then run that layer's norm as a
    kernel (it used to hand the product a half norm it could not apply).  Compared with the
    plain implementation."""
    import tempfile
    from lastengine_b200 import Engine
    from lastengine_b200.ops import kernels
    cfg = dict(TINY_A, intermediate_size=19008, num_hidden_layers=2, layer_types=["conv", "attention"])
    w = torch.empty(38016, 64, dtype=torch.bfloat16, device="cuda")
    assert kernels.split_norm_ok(16, torch.bfloat16, w) and not kernels.split_norm_ok(32, torch.bfloat16, w)
    assert kernels.split_norm_ok(32, torch.bfloat16, w[:11264]) and not kernels.split_norm_ok(32, torch.bfloat16, None)
    assert not kernels.split_norm_ok(32, torch.float32, w[:11264].float())
    with tempfile.TemporaryDirectory() as d:
        H.make_model_dir(cfg, 5, d)
        eng = Engine.from_pretrained(d, dtype="bfloat16", max_tokens=4096)
        reqs = H.requests_for(cfg, [12] * 32, 65)
        got = H.run_batch(eng, reqs, [8] * 32)
        for r, g in zip(reqs[:6], got[:6]):
            assert H.rel_err(g, H.plain_logits(cfg, d, r, True)) <= H.TOL_BF16
        eng.check_status()
