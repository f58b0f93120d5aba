"""The engine against the plain implementation at the layer sizes the benchmark runs.

The tiny configurations reach none of the kernels a model of real width runs: head size 64
attention on tcgen05, the paired 256 x 256 matrix product from 1,024 rows, the sliced product of
17-128 rows with its split norms, the output matrix over 65,536 words with the multi-block
argmax behind it, page tables over many pages.  Here the layers have the sizes of the 1.2B-shaped
configuration (hidden 2048, 32 query and 8 kv heads of 64, feed-forward 8192 adjusted to 5632,
vocabulary 65536, convolution length 3, tied output) with 5 of its 16 layers, and once the sizes of
the 8B-A1B-shaped configuration's expert layers (32 experts of 1792, 4 per token) with 2 of its 24
layers.  Same three ways of cutting the work as for the tiny models, same fixed tolerances, in
32-bit and in bfloat16; the plain implementation runs in double precision on the device's
library routines here (its arithmetic is the same; on the CPU it would take minutes).
"""
import numpy as np
import pytest
import torch

import harness as H

pytestmark = pytest.mark.gpu

REAL_DENSE = {   # 5 of the 16 layers of the 1.2B-shaped configuration
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 5,
    "layer_types": ["conv", "conv", "attention", "conv", "attention"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 8192, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "norm_eps": 1e-5, "tie_embedding": True,
}

REAL_MOE = {     # 2 of the 24 layers of the 8B-A1B-shaped configuration: one dense, one with experts
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 8192, "hidden_size": 2048, "num_hidden_layers": 2,
    "layer_types": ["conv", "attention"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 7168, "num_experts": 32, "num_experts_per_tok": 4, "moe_intermediate_size": 1792,
    "num_dense_layers": 1, "norm_topk_prob": True, "use_expert_bias": True,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "norm_eps": 1e-5, "tie_embedding": True,
}

DEV = "cuda:0"
DTYPES = [("float32", False, H.TOL_F32), ("bfloat16", True, H.TOL_BF16)]


@pytest.fixture(scope="module")
def dense_dir(tmp_path_factory):
    return H.make_model_dir(REAL_DENSE, 7, str(tmp_path_factory.mktemp("real_dense")))


@pytest.fixture(scope="module")
def moe_dir(tmp_path_factory):
    # 32 scores lie closer together than 8: the selection biases are spread so that most positions
    # have a clear fourth expert
    return H.make_model_dir(REAL_MOE, 8, str(tmp_path_factory.mktemp("real_moe")), expert_bias_scale=5.0)


@pytest.fixture(scope="module")
def engines(dense_dir):
    from lastengine_b200 import Engine
    made = {}

    def get(dtype):
        if dtype not in made:
            made[dtype] = Engine.from_pretrained(dense_dir, dtype=dtype, max_tokens=16384)
        return made[dtype]
    yield get
    made.clear()
    torch.cuda.empty_cache()


_plain: dict = {}


def plain(cfg, model_dir, tokens, bf16):
    key = (model_dir, tuple(tokens), bf16)
    if key not in _plain:
        lg, m = H.plain_logits_and_margins(cfg, model_dir, tokens, bf16, device=DEV)
        keep = H.decided(m, bf16, cfg["hidden_size"])
        assert keep.double().mean() >= 0.7, "too many router near-ties to test anything"
        _plain[key] = (lg, keep)
    return _plain[key]


def check(got, plain_result, tol, what):
    want, keep = plain_result
    got, want = got.to(want.device)[keep], want[keep]
    e = H.rel_err(got, want)
    assert e <= tol, (f"{what}: error {e:.3e} > {tol:.1e}; first wrong position "
                      f"{H.first_bad_position(got, want, tol)} of {want.shape[0]} compared")
    return e


def status_clear():
    """No tensor-core kernel gave up on a bounded wait while the test ran."""
    from lastengine_b200.ops import kernels
    kernels.check_device_status()


@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_whole_prompts(dtype, bf16, tol, dense_dir, engines):
    """1,150 tokens in one step (the paired product, 18 pages of tcgen05 attention, the output
    matrix over 1,150 rows) and 300 tokens."""
    eng = engines(dtype)
    for toks in H.requests_for(REAL_DENSE, [1150, 300], 51):
        check(H.run_whole(eng, toks, keep=H.on_device), plain(REAL_DENSE, dense_dir, toks, bf16), tol,
              f"dense {dtype} whole len {len(toks)}")
    status_clear()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_last_32_one_by_one(dtype, bf16, tol, dense_dir, engines):
    """The same requests with their last 32 tokens as single steps: the weight-streaming product,
    the fused convolution step, split decode attention over 18 and 5 pages, a page boundary
    crossed at 1,152 / 320 while decoding."""
    eng = engines(dtype)
    for toks in H.requests_for(REAL_DENSE, [1170, 340], 51):
        check(H.run_tail(eng, toks, 32, keep=H.on_device), plain(REAL_DENSE, dense_dir, toks, bf16), tol,
              f"dense {dtype} tail len {len(toks)}")
    status_clear()


@pytest.mark.parametrize("dtype,bf16,tol", DTYPES)
def test_unequal_batches_of_many_requests(dtype, bf16, tol, dense_dir, engines):
    """48 requests of unequal lengths start together; their decode steps have 48 rows at first
    (the sliced tcgen05 product of 17-128 rows and both halves of its split norms) and fewer and
    fewer as the shorter ones end, down to the weight stream of up to 16 rows; then a batch of 5
    and one of 20 take over the slots and pages that came back."""
    eng = engines(dtype)
    rng = np.random.default_rng(52)
    for n_req in (48, 5, 20):
        lens = rng.integers(40, 200, size=n_req).tolist()
        reqs = H.requests_for(REAL_DENSE, lens, 53 + n_req)
        prompt_lens = [max(1, n - int(d)) for n, d in zip(lens, rng.integers(0, 34, size=n_req))]
        got = H.run_batch(eng, reqs, prompt_lens, keep=H.on_device)
        worst = 0.0
        for r, g in zip(reqs, got):
            worst = max(worst, check(g, plain(REAL_DENSE, dense_dir, r, bf16), tol,
                                     f"dense {dtype} batch of {n_req}, len {len(r)}"))
        eng.cache.check()
        assert eng.cache.slots.n_held == 0
        _plain.clear()
    status_clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_of_64_requests_graphs_on_and_off(dtype, dense_dir, engines):
    """64 requests through the entry point with captured decode steps launched ahead (buckets 64,
    32, 16, ... as requests stop) and step by step without graphs: the same tokens.  Where the two
    part ways, the two best logits of that step must be a near-tie (the two paths sum the
    attention splits in a different order)."""
    from lastengine_b200 import SamplingParams
    eng = engines(dtype)
    prompts = H.requests_for(REAL_DENSE, np.random.default_rng(54).integers(8, 120, size=64).tolist(), 55)
    greedy = SamplingParams(temperature=0.0)
    free = eng.generate(prompts, greedy, max_new_tokens=24, stop_token_ids=[], use_graphs=False)
    stops = [free.tokens[i][4 + i % 16] for i in range(0, 64, 3)]       # a third of the requests stop early
    slow = eng.generate(prompts, greedy, max_new_tokens=24, stop_token_ids=stops, use_graphs=False)
    fast = eng.generate(prompts, greedy, max_new_tokens=24, stop_token_ids=stops)
    assert len({len(t) for t in fast.tokens}) > 3
    for i, (a, b) in enumerate(zip(fast.tokens, slow.tokens)):
        if a == b:
            continue
        j = next(k for k in range(min(len(a), len(b)) + 1) if a[k:k + 1] != b[k:k + 1])
        s = eng.new_sequence()
        lg = eng.step([s], [prompts[i] + b[:j]], "last")[0].double()
        eng.release(s)
        top = torch.topk(lg, 2).values
        gap = float((top[0] - top[1]) / lg.abs().max())
        assert gap < (H.TOL_BF16 if dtype == "bfloat16" else H.TOL_F32), \
            f"{dtype}: request {i} differs at token {j} ({a[j:j + 1]} vs {b[j:j + 1]}) with a clear best logit (gap {gap:.2e})"
    assert sum(a == b for a, b in zip(fast.tokens, slow.tokens)) >= 60
    status_clear()
    assert eng.cache.slots.n_held == 0
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompts_as_captured_steps_at_real_sizes(dtype, dense_dir, engines):
    """Prompts of a few hundred rows in all through the entry point: with graphs they are one
    captured step (a bucket of rows and sequences, padded), without them a plain step; the same
    tokens, and where the two part ways the two best logits there are a near-tie."""
    from lastengine_b200 import SamplingParams
    eng = engines(dtype)
    greedy = SamplingParams(temperature=0.0)
    for lens in ([40, 100, 200], [7], [250, 3]):
        prompts = H.requests_for(REAL_DENSE, lens, 56 + len(lens))
        fast = eng.generate(prompts, greedy, max_new_tokens=8, stop_token_ids=[])
        slow = eng.generate(prompts, greedy, max_new_tokens=8, stop_token_ids=[], use_graphs=False)
        for i, (a, b) in enumerate(zip(fast.tokens, slow.tokens)):
            if a == b:
                continue
            j = next(k for k in range(min(len(a), len(b)) + 1) if a[k:k + 1] != b[k:k + 1])
            s = eng.new_sequence()
            lg = eng.step([s], [prompts[i] + b[:j]], "last")[0].double()
            eng.release(s)
            top = torch.topk(lg, 2).values
            gap = float((top[0] - top[1]) / lg.abs().max())
            assert gap < (H.TOL_BF16 if dtype == "bfloat16" else H.TOL_F32), \
                f"{dtype}: prompts {lens}, request {i} differs at token {j} with a clear best logit (gap {gap:.2e})"
    assert any(isinstance(k, tuple) and k[0] == "prompts" for k in eng._decode_graphs[greedy])
    status_clear()
    assert eng.cache.slots.n_held == 0


def test_expert_layers_of_real_size(moe_dir):
    """The 8B-A1B shape's expert layer (32 experts of 1792, 4 per token) in bfloat16: a prompt of
    700 tokens (the grouped tcgen05 product), its last 32 tokens one by one (the grouped weight
    stream), and a batch of 24 unequal requests."""
    from lastengine_b200 import Engine
    eng = Engine.from_pretrained(moe_dir, dtype="bfloat16", max_tokens=8192)
    toks = H.requests_for(REAL_MOE, [700], 56)[0]
    check(H.run_whole(eng, toks, keep=H.on_device), plain(REAL_MOE, moe_dir, toks, True), H.TOL_BF16, "experts whole")
    check(H.run_tail(eng, toks, 32, keep=H.on_device), plain(REAL_MOE, moe_dir, toks, True), H.TOL_BF16, "experts tail")
    lens = np.random.default_rng(57).integers(20, 90, size=24).tolist()
    reqs = H.requests_for(REAL_MOE, lens, 58)
    got = H.run_batch(eng, reqs, [max(1, n - 12) for n in lens], keep=H.on_device)
    for r, g in zip(reqs, got):
        check(g, plain(REAL_MOE, moe_dir, r, True), H.TOL_BF16, f"experts batch, len {len(r)}")
    status_clear()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
    _plain.clear()
    H._tensors_on.clear()
