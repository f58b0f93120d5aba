"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way
of cutting the work: each request alone and whole; with its last 32 tokens one by one; in
batches of unequal lengths whose shorter requests end earlier, one batch after another so
that slots and pages are used again; long decoding; the first tokens of a sequence."""
import numpy as np
import pytest
import torch

import harness as H
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}
LENGTHS = {"A": [5, 11, 17, 64, 100], "B": [1, 7, 23, 40, 65, 130], "C": [3, 33, 70, 90], "D": [2, 41, 66, 120]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {k: H.make_model_dir(cfg, seed, str(tmp_path_factory.mktemp(f"tiny{k}")), freq_factors=k == "D")
            for k, (cfg, seed) in CONFIGS.items()}


@pytest.fixture(scope="module")
def engines(model_dirs):
    from lastengine_b200 import Engine
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = Engine.from_pretrained(model_dirs[name], dtype=dtype, max_tokens=2048)
        return cache[(name, dtype)]
    return get


_plain = {}


def plain(name, model_dirs, tokens, bf16):
    """(logits, positions to compare): see harness.ROUTER_GAP_BF16."""
    key = (name, tuple(tokens), bf16)
    if key not in _plain:
        lg, m = H.plain_logits_and_margins(CONFIGS[name][0], model_dirs[name], tokens, bf16)
        keep = H.decided(m, bf16)
        assert keep.all() or bf16, "a router near-tie at 32-bit level: choose other tokens"
        assert keep.double().mean() >= 0.7, "too many router near-ties to test anything"
        _plain[key] = (lg, keep)
    return _plain[key]


def check(got, plain_result, tol, what):
    want, keep = plain_result
    got, want = got[keep], want[keep]
    e = H.rel_err(got, want)
    bad = H.first_bad_position(got, want, tol)
    assert e <= tol, f"{what}: error {e:.3e} > {tol:.1e}; first wrong position {bad} of {want.shape[0]} compared"


DTYPES = [("float32", False, H.TOL_F32), ("bfloat16", True, H.TOL_BF16)]


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_whole(name, dtype, bf16, tol, model_dirs, engines):
    eng = engines(name, dtype)
    for toks in H.requests_for(CONFIGS[name][0], LENGTHS[name], 11):
        check(H.run_whole(eng, toks), plain(name, model_dirs, toks, bf16), tol, f"{name} {dtype} whole len {len(toks)}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_last_32_one_by_one(name, dtype, bf16, tol, model_dirs, engines):
    eng = engines(name, dtype)
    for toks in H.requests_for(CONFIGS[name][0], LENGTHS[name], 11):
        check(H.run_tail(eng, toks, 32), plain(name, model_dirs, toks, bf16), tol, f"{name} {dtype} tail len {len(toks)}")
    eng.cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_unequal_batches_reuse_slots(name, dtype, bf16, tol, model_dirs, engines):
    eng = engines(name, dtype)
    cfg = CONFIGS[name][0]
    reqs = H.requests_for(cfg, LENGTHS[name] + [9, 2, 77], 12)
    # prompts of unequal lengths; the rest of each request is decoded, so requests end at different steps
    prompt_lens = [max(1, len(r) - d) for r, d in zip(reqs, [3, 9, 0, 30, 12, 5, 1, 40, 20])]
    for lo in range(0, len(reqs), 3):        # one batch after another: slots and pages come back and are reused
        part, pl = reqs[lo:lo + 3], prompt_lens[lo:lo + 3]
        got = H.run_batch(eng, part, pl)
        for r, g in zip(part, got):
            check(g, plain(name, model_dirs, r, bf16), tol, f"{name} {dtype} batch from {lo}, len {len(r)}")
        eng.cache.check()
        assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_batch_of_200_requests(name, dtype, bf16, tol, model_dirs):
    """More sequences in a step than the decode products for up to 128 rows take: the prompts are one
    step of some 1,500 rows, the decode steps have 200, then fewer and fewer rows (requests end at
    different steps), so the products pass from the tiled kernels to the sliced and the streaming ones.
    Then the same requests through generate(), captured steps (a bucket of 256) against plain ones."""
    from lastengine_b200 import Engine, SamplingParams
    cfg = CONFIGS[name][0]
    rng = np.random.default_rng(21)
    lengths = rng.integers(4, 22, size=200).tolist()
    reqs = H.requests_for(cfg, lengths, 22)
    prompt_lens = [max(1, n - int(d)) for n, d in zip(lengths, rng.integers(1, 13, size=200))]
    eng = Engine.from_pretrained(model_dirs[name], dtype=dtype, max_tokens=200 * 64 + 1024)
    got = H.run_batch(eng, reqs, prompt_lens)
    for i in range(0, 200, 7):
        check(got[i], plain(name, model_dirs, reqs[i], bf16), tol, f"{name} {dtype} request {i} of 200, len {lengths[i]}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
    prompts = [r[:p] for r, p in zip(reqs, prompt_lens)]
    sp = SamplingParams(temperature=0.0)
    a = eng.generate(prompts, sp, max_new_tokens=6, max_batch=200, use_graphs=True)
    b = eng.generate(prompts, sp, max_new_tokens=6, max_batch=200, use_graphs=False)
    same = sum(x == y for x, y in zip(a.tokens, b.tokens))
    assert same >= (200 if not bf16 else 190), f"{same} of 200 requests agree between captured and plain steps"
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_long_decode(name, dtype, bf16, tol, model_dirs, engines):
    """A short prompt and 200 single-token steps: crosses cache pages at 64, 128 and 192."""
    eng = engines(name, dtype)
    toks = H.requests_for(CONFIGS[name][0], [203], 13)[0]
    check(H.run_tail(eng, toks, 200), plain(name, model_dirs, toks, bf16), tol, f"{name} {dtype} long decode")


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_first_tokens(name, dtype, bf16, tol, model_dirs, engines):
    """A one-token prompt, then single tokens: fewer rows than the convolution reaches back."""
    eng = engines(name, dtype)
    toks = H.requests_for(CONFIGS[name][0], [6], 14)[0]
    check(H.run_tail(eng, toks, 5), plain(name, model_dirs, toks, bf16), tol, f"{name} {dtype} first tokens")


@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_chunked_prompt(dtype, bf16, tol, model_dirs, engines):
    """A prompt fed in three pieces (the step function takes any number of tokens per sequence)."""
    eng = engines("B", dtype)
    toks = H.requests_for(TINY_B, [150], 15)[0]
    s = eng.new_sequence()
    out = []
    for lo, hi in ((0, 70), (70, 71), (71, 150)):
        out.append(eng.step([s], [toks[lo:hi]], [list(range(hi - lo))]).float().cpu().clone())
    eng.release(s)
    check(torch.cat(out), plain("B", model_dirs, toks, bf16), tol, f"B {dtype} chunked prompt")


@pytest.mark.parametrize("name", ["B", "C"])
@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_sequence_exported_and_imported_goes_on(name, dtype, bf16, tol, model_dirs, engines):
    """A sequence written out as bytes after 90 tokens, released, and read back into other pages
    and another slot (a second sequence took its old ones) goes on as if nothing had happened:
    keys, values (a window's too) and the convolution state all came back."""
    eng = engines(name, dtype)
    cfg = CONFIGS[name][0]
    toks, filler = H.requests_for(cfg, [130, 75], 19)
    s = eng.new_sequence()
    out = [eng.step([s], [toks[:90]], [list(range(90))]).float().cpu().clone()]
    data = eng.export_sequence(s)
    eng.release(s)
    f = eng.new_sequence()
    eng.step([f], [filler], "last")
    t = eng.import_sequence(data)
    assert f == s and t != s and eng.length(t) == 90
    out.append(eng.step([t], [toks[90:100]], [list(range(10))]).float().cpu().clone())
    for i in range(100, 130):
        out.append(eng.step([t], [[toks[i]]], [[0]]).float().cpu().clone())
    eng.release([f, t])
    check(torch.cat(out), plain(name, model_dirs, toks, bf16), tol, f"{name} {dtype} exported and imported")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


def test_padding_changes_nothing(model_dirs, engines):
    """Padding sequences (slot -1) in a step leave the real rows' logits bit-identical."""
    eng = engines("A", "float32")
    toks = H.requests_for(TINY_A, [20, 9], 16)
    seqs = [eng.new_sequence() for _ in toks]
    a = eng.step(seqs, toks, "last").clone()
    eng.release(seqs)
    seqs = [eng.new_sequence() for _ in toks]
    b = eng.step([seqs[0], -1, seqs[1], -1], [toks[0], [0, 0, 0], toks[1], [5]], [[19], [], [8], []]).clone()
    eng.release(seqs)
    assert torch.equal(a, b)
