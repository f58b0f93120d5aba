"""Each part alone against its plain counterpart, and the library's openness: a mixer with
state of its own, another position encoding and another layer order are registered, built
and stepped from the test, without a change to the library's files."""
import numpy as np
import pytest
import torch

import harness as H
import plain_lfm3 as P
from tiny_configs import TINY_A

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def env_for(dtype):
    from lastengine_b200.engine.workspace import Workspace
    from lastengine_b200.parts.base import BuildEnv
    return BuildEnv(device=DEV, dtype=dtype, workspace=Workspace(DEV))


def gen(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return scale * torch.randn(*shape, generator=g)


def err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / (want.abs().max() + 1e-30))


def load_part(part, env, seed, std=0.2):
    """Random bfloat16-representable weights; returns them as float64 by short name."""
    from lastengine_b200.weights.loader import kept_dtype
    from lastengine_b200.parts.base import NORM
    vals, dev = {}, {}
    for i, (name, spec) in enumerate(part.tensors().items()):
        t = gen(*spec.shape, seed=seed + i, scale=spec.std or std)
        if spec.role == NORM:
            t = 1 + 0.1 * t
        t = t.to(torch.bfloat16)
        vals[name] = t.double()
        dev[name] = t.to(device=DEV, dtype=kept_dtype(spec, t.dtype, env.dtype))
    part.load(dev, env)
    return vals


def one_sequence_batch(n, pos0=0, slot=0, table=None):
    from lastengine_b200.engine.batch import BatchBuilder
    return BatchBuilder(DEV).build([slot], [[0] * n], [pos0], [], {0: table} if table is not None else {})


CASES = [(torch.float32, P.identity, 2e-5), (torch.bfloat16, P.round_bf16, 1.5e-2)]


@pytest.mark.parametrize("dtype,rnd,tol", CASES)
def test_swiglu_part(dtype, rnd, tol):
    from lastengine_b200.parts.ffn import SwiGLU
    env = env_for(dtype)
    part = SwiGLU(hidden_size=72, intermediate_size=112)
    w = load_part(part, env, 100)
    h = rnd(gen(50, 72, seed=1).double())
    out = gen(50, 72, seed=2).to(DEV)
    base = out.cpu().double()
    part.forward(h.to(device=DEV, dtype=dtype), out, True, one_sequence_batch(50), env)
    want = base + P.swiglu_ffn(h, w["w1.weight"], w["w3.weight"], w["w2.weight"], rnd)
    assert err(out, want) < tol


@pytest.mark.parametrize("dtype,rnd,tol", CASES)
def test_moe_part(dtype, rnd, tol):
    from lastengine_b200.parts.ffn import SigmoidTopKMoE
    env = env_for(dtype)
    part = SigmoidTopKMoE(hidden_size=72, num_experts=6, top_k=3, expert_size=32, norm_topk=True,
                          use_bias=True, scaling=1.25)
    w = load_part(part, env, 200)
    h = rnd(gen(41, 72, seed=3).double())
    out = torch.zeros(41, 72, device=DEV)
    part.forward(h.to(device=DEV, dtype=dtype), out, False, one_sequence_batch(41), env)
    want = P.moe_ffn(h, w, E=6, k=3, norm_topk=True, use_bias=True, scaling=1.25, rnd=rnd)
    assert err(out, want) < tol


@pytest.mark.parametrize("dtype,rnd,tol", CASES)
def test_shortconv_part(dtype, rnd, tol):
    from lastengine_b200.parts.shortconv import ShortConvMixer
    from lastengine_b200.cache import CacheView
    env = env_for(dtype)
    part = ShortConvMixer(hidden_size=72, L_cache=4)
    w = load_part(part, env, 300)
    h = rnd(gen(30, 72, seed=4).double())
    state = torch.zeros(3, 72, 3, device=DEV)
    view = CacheView(writable=True, state=state)
    out = torch.zeros(30, 72, device=DEV)
    hd = h.to(device=DEV, dtype=dtype)
    part.forward(hd[:19], out[:19], False, one_sequence_batch(19, 0, slot=1), view, env)
    part.forward(hd[19:], out[19:], False, one_sequence_batch(11, 19, slot=1), view, env)
    want, _ = P.short_conv(h, w, 30, D=72, Lc=4, rnd=rnd)
    assert err(out, want) < tol


@pytest.mark.parametrize("dtype,rnd,tol", CASES)
@pytest.mark.parametrize("window,gate", [(0, False), (20, True)])
def test_attention_part(dtype, rnd, tol, window, gate):
    from lastengine_b200.parts.attention import AttentionMixer
    from lastengine_b200.parts.base import PartSpec
    from lastengine_b200.cache import CacheView
    env = env_for(dtype)
    nh, nkv, hd, D = 6, 3, 48, 72
    part = AttentionMixer(hidden_size=D, num_heads=nh, num_kv_heads=nkv, head_dim=hd, norm_eps=1e-4,
                          position=PartSpec("rope", {"rope_dim": 32, "theta": 5e4}), window=window,
                          output_gate=gate)
    w = load_part(part, env, 400)
    T = 100
    h = rnd(gen(T, D, seed=5).double())
    pool = torch.zeros(2, 4, nkv, 64, hd, device=DEV, dtype=dtype)
    table = np.array([[2, 0]], dtype=np.int32)
    out = torch.zeros(T, D, device=DEV)
    hdv = h.to(device=DEV, dtype=dtype)
    for lo, hi in ((0, 70), (70, 71), (71, 100)):       # a prompt, one token, another chunk
        b = one_sequence_batch(hi - lo, lo, table=table)
        view = CacheView(writable=True, k=pool[0], v=pool[1].view(4, nkv, hd, 64), block_table=b.tables[0])
        part.forward(hdv[lo:hi], out[lo:hi], False, b, view, env)
    want = P.attention(h, w, T, nh=nh, nkv=nkv, hd=hd, eps=1e-4, theta=5e4, rope_dim=32, window=window,
                       gate=gate, rnd=rnd)
    assert err(out, want) < tol


# ---- openness ----------------------------------------------------------------------------------------
def test_toy_parts_register_build_and_step():
    """A toy architecture made here: a mixer that keeps an exponential moving average of its input
    per sequence (fixed-size state in the cache), a feed-forward that routes each token to one of
    two matrices by the sign of a feature, a layer named twice in the schedule, and an attention
    layer with a learned-position-free rotary variant (adjacent pairs).  Written with tensor
    operations; registered, built, stepped token by token and as a whole prompt."""
    from lastengine_b200 import Engine
    from lastengine_b200.parts.base import (MATRIX, FeedForward, LayerSpec, Mixer, ModelPlan, PartSpec,
                                            ScheduleEntry, StateSpec, TensorSpec)
    from lastengine_b200.registry import ARCHITECTURES, FEED_FORWARDS, MIXERS
    from lastengine_b200.weights import load_random

    @MIXERS.register("toy_ema", replace=True)
    class EmaMixer(Mixer):
        def __init__(self, hidden_size, decay):
            self.D, self.decay = hidden_size, decay

        def tensors(self):
            return {"proj.weight": TensorSpec((self.D, self.D), MATRIX)}

        def load(self, tensors, env):
            self.w = tensors["proj.weight"].float()

        def cache_spec(self):
            return StateSpec((self.D,), torch.float32)

        def forward(self, h, out, accumulate, batch, cache, env):
            slots = batch.row_slot.long()
            y = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            for m in range(h.shape[0]):                     # rows of a sequence are in order
                s = int(slots[m])
                if s < 0:
                    y[m] = 0
                    continue
                cache.state[s] = self.decay * cache.state[s] + (1 - self.decay) * h[m].float()
                y[m] = cache.state[s]
            y = y @ self.w.T
            out.add_(y) if accumulate else out.copy_(y)

    @FEED_FORWARDS.register("toy_sign_router", replace=True)
    class SignRouter(FeedForward):
        def __init__(self, hidden_size):
            self.D = hidden_size

        def tensors(self):
            return {"a.weight": TensorSpec((self.D, self.D), MATRIX), "b.weight": TensorSpec((self.D, self.D), MATRIX)}

        def load(self, tensors, env):
            self.a, self.b = tensors["a.weight"].float(), tensors["b.weight"].float()

        def forward(self, h, out, accumulate, batch, env):
            hf = h.float()
            y = torch.where(hf[:, :1] > 0, hf @ self.a.T, hf @ self.b.T)
            out.add_(y) if accumulate else out.copy_(y)

    @ARCHITECTURES.register("ToyForCausalLM", replace=True)
    def toy_plan(raw):
        D, V = raw["hidden_size"], raw["vocab_size"]
        norm = PartSpec("rmsnorm", {"size": D, "eps": 1e-5})
        ema = LayerSpec("layers.0", PartSpec("toy_ema", {"hidden_size": D, "decay": raw["decay"]}),
                        PartSpec("toy_sign_router", {"hidden_size": D}), norm, norm,
                        names={"mixer": "ema", "ffn": "router", "mixer_norm": "n1", "ffn_norm": "n2"})
        att = LayerSpec("layers.1", PartSpec("attention", {
            "hidden_size": D, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "norm_eps": 1e-5, "qk_norm": False,
            "position": PartSpec("rope", {"rope_dim": 16, "theta": 100.0, "style": "adjacent"})}),
            PartSpec("swiglu", {"hidden_size": D, "intermediate_size": 48}), norm, norm,
            names={"mixer": "attn", "ffn": "mlp", "mixer_norm": "n1", "ffn_norm": "n2"})
        return ModelPlan("ToyForCausalLM", D, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": D}),
                         norm, PartSpec("linear_head", {"vocab_size": V, "hidden_size": D, "tied": True}),
                         layers=[ema, att],
                         schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)],   # layer 0 runs twice
                         names={"embedding": "emb", "final_norm": "norm_f", "head": "head"})

    try:
        cfg = {"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 50, "decay": 0.75}
        for dtype, tol in (("float32", 1e-5), ("bfloat16", 3e-2)):
            eng = Engine.from_config(cfg, seed=3, dtype=dtype, max_tokens=512, norm_init="random")
            specs = eng.model.cache_specs()
            assert isinstance(specs[0], StateSpec) and isinstance(specs[2], StateSpec)      # two states for one layer
            assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].data.shape[0] == 2
            toks = H.requests_for(cfg, [40], 5)[0]
            whole = H.run_whole(eng, toks)
            stepwise = H.run_tail(eng, toks, 39)
            assert torch.isfinite(whole).all()
            assert err(stepwise, whole) < tol
            # a second sequence in a reused slot starts from a zero state
            again = H.run_whole(eng, toks)
            assert torch.equal(again, whole)
    finally:
        MIXERS.unregister("toy_ema")
        FEED_FORWARDS.unregister("toy_sign_router")
        ARCHITECTURES.unregister("ToyForCausalLM")


def test_toy_position_encoding_defined_here():
    """A position encoding that is no rotation, defined in this test and registered: it adds a
    feature of the position, log(1 + pos) / 8, to the first element of every normed query and key
    head.  The attention mixer is built with it by name and knows nothing of it; a prompt in three
    pieces must give the plain computation with the same encoding."""
    from lastengine_b200.cache import CacheView
    from lastengine_b200.parts.attention import AttentionMixer
    from lastengine_b200.parts.base import PartSpec, PositionEncoding
    from lastengine_b200.registry import POSITION_ENCODINGS

    @POSITION_ENCODINGS.register("toy_log_position", replace=True)
    class LogPosition(PositionEncoding):
        def __init__(self, strength):
            self.strength = strength

        def apply(self, q, k, row_pos):
            f = (torch.log1p(row_pos.float()) * self.strength).to(q.dtype)[:, None]
            q[:, :, 0] += f
            if k is not None:
                k[:, :, 0] += f

    def plain_encoding(v, positions, rope_dim, theta, neox=True, freq_factors=None):
        out = v.clone()
        out[:, :, 0] += torch.log1p(positions.to(v.dtype))[:, None] * 0.125
        return out

    try:
        for dtype, rnd, tol in CASES:
            env = env_for(dtype)
            nh, nkv, hd, D = 4, 2, 32, 64
            part = AttentionMixer(hidden_size=D, num_heads=nh, num_kv_heads=nkv, head_dim=hd, norm_eps=1e-5,
                                  position=PartSpec("toy_log_position", {"strength": 0.125}))
            assert part.position.fused_rotary() is None
            w = load_part(part, env, 410)
            T = 90
            h = rnd(gen(T, D, seed=6).double())
            pool = torch.zeros(2, 4, nkv, 64, hd, device=DEV, dtype=dtype)
            table = np.array([[1, 3]], dtype=np.int32)
            out = torch.zeros(T, D, device=DEV)
            hdv = h.to(device=DEV, dtype=dtype)
            for lo, hi in ((0, 50), (50, 51), (51, 90)):
                b = one_sequence_batch(hi - lo, lo, table=table)
                view = CacheView(writable=True, k=pool[0], v=pool[1].view(4, nkv, hd, 64), block_table=b.tables[0])
                part.forward(hdv[lo:hi], out[lo:hi], False, b, view, env)
            orig = P.rope
            P.rope = plain_encoding
            try:
                want = P.attention(h, w, T, nh=nh, nkv=nkv, hd=hd, eps=1e-5, theta=0.0, rope_dim=hd, rnd=rnd)
            finally:
                P.rope = orig
            assert err(out, want) < tol
    finally:
        POSITION_ENCODINGS.unregister("toy_log_position")


def test_toy_part_takes_part_in_split_norms():
    """A feed-forward defined here that says `split_norm = True` and passes the two halves on to its
    products: in decode steps the block then splits the norms around it (no norm kernel between
    the conv mixer and it, nor between it and the next layer's mixer).  The same model with the
    part saying False runs the norm kernels; both agree with each other and, token by token, with
    the whole prompt."""
    from lastengine_b200 import Engine
    from lastengine_b200.ops import kernels
    from lastengine_b200.parts.base import MATRIX, FeedForward, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, TensorSpec
    from lastengine_b200.registry import ARCHITECTURES, FEED_FORWARDS

    calls = {"scaled": 0, "emitted": 0}

    class TwoMatrices(FeedForward):
        def __init__(self, hidden_size, inner):
            self.D, self.F = hidden_size, inner

        def tensors(self):
            return {"a.weight": TensorSpec((self.F, self.D), MATRIX), "b.weight": TensorSpec((self.D, self.F), MATRIX)}

        def load(self, tensors, env):
            self.a, self.b = tensors["a.weight"].contiguous(), tensors["b.weight"].contiguous()

        def forward(self, h, out, accumulate, batch, env):
            scale, emit = env.take_split_in(), env.take_split_out()
            calls["scaled"] += scale is not None
            calls["emitted"] += emit is not None
            t = env.workspace.get("toy.t", (h.shape[0], self.F), env.dtype)
            kernels.linear(t, h, self.a, scale=scale)
            kernels.linear(out, t, self.b, kernels.ACCUMULATE if accumulate else kernels.STORE,
                           emit=emit if accumulate else None)

    def plan_of(kind):
        def plan(raw):
            D, V = raw["hidden_size"], raw["vocab_size"]
            norm = PartSpec("rmsnorm", {"size": D, "eps": 1e-5})
            layer = lambda i: LayerSpec(f"layers.{i}", PartSpec("shortconv", {"hidden_size": D, "L_cache": 3}),
                                        PartSpec(kind, {"hidden_size": D, "inner": 80}), norm, norm,
                                        names={"mixer": "conv", "ffn": "mlp", "mixer_norm": "n1", "ffn_norm": "n2"})
            return ModelPlan("Toy2ForCausalLM", D, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": D}),
                             norm, PartSpec("linear_head", {"vocab_size": V, "hidden_size": D, "tied": True}),
                             layers=[layer(0), layer(1)], schedule=[ScheduleEntry(0), ScheduleEntry(1)],
                             names={"embedding": "emb", "final_norm": "norm_f", "head": "head"})
        return plan

    cfg = {"architectures": ["Toy2ForCausalLM"], "hidden_size": 48, "vocab_size": 60}
    toks = H.requests_for(cfg, [50], 8)[0]
    got = {}
    try:
        for split in (True, False):
            part = type("TwoMatricesSplit" if split else "TwoMatricesPlain", (TwoMatrices,), {"split_norm": split})
            FEED_FORWARDS.register("toy_two_matrices", replace=True)(part)
            ARCHITECTURES.register("Toy2ForCausalLM", replace=True)(plan_of("toy_two_matrices"))
            eng = Engine.from_config(cfg, seed=4, dtype="bfloat16", max_tokens=512, norm_init="random")
            calls["scaled"] = calls["emitted"] = 0
            got[split] = (H.run_whole(eng, toks), H.run_tail(eng, toks, 30))
            if split:
                assert calls["scaled"] > 0 and calls["emitted"] > 0      # the block did hand it the halves
            else:
                assert calls["scaled"] == 0 and calls["emitted"] == 0
            assert err(got[split][1], got[split][0]) < 3e-2
        assert err(got[True][0], got[False][0]) < 3e-2 and err(got[True][1], got[False][1]) < 3e-2
    finally:
        FEED_FORWARDS.unregister("toy_two_matrices")
        ARCHITECTURES.unregister("Toy2ForCausalLM")


def test_layer_reads_another_layers_cache(tmp_path):
    """A schedule in which the second attention layer keeps no keys of its own and attends over the
    first one's: it must equal the plain computation with the first layer's keys and values."""
    from lastengine_b200 import Engine
    from lastengine_b200.arch.lfm3 import lfm3_plan
    from lastengine_b200.config import Lfm3Config
    from lastengine_b200.parts.base import ScheduleEntry
    import dataclasses
    cfg = Lfm3Config.from_dict(TINY_A)
    plan = lfm3_plan(cfg)
    lay = list(plan.layers)
    shared = dataclasses.replace(lay[3], mixer=dataclasses.replace(lay[3].mixer, params={**lay[3].mixer.params, "own_kv": False}))
    lay[3] = shared
    plan = dataclasses.replace(plan, layers=lay, schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2),
                                                          ScheduleEntry(3, cache=1, writes_cache=False)])
    eng = Engine(plan, dtype="float32", max_tokens=512)
    from lastengine_b200.weights import load_random
    load_random(eng.model, seed=9, norm_init="random")
    eng.loaded = True
    assert "layers.3.self_attn.k_proj.weight" not in eng.model.tensor_specs()
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].k_pool.shape[0] == 1
    toks = H.requests_for(TINY_A, [90], 6)[0]
    whole = H.run_whole(eng, toks)
    stepwise = H.run_tail(eng, toks, 40)
    assert err(stepwise, whole) < 2e-5
