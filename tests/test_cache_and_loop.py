"""The cache's bookkeeping and the generation loop's decisions (no GPU)."""
import random

import pytest
import torch

import harness as H  # noqa: F401
from lastengine_b200.cache import Cache, CacheError, CacheFull, IdPool
from lastengine_b200.engine.generate import GenerationLoop, plan_batches
from lastengine_b200.parts.base import KVSpec, StateSpec
from lastengine_b200.sampling.params import SamplingParams, XorShift64


def test_id_pool_never_loses_or_doubles():
    p = IdPool(5, "slot")
    got = [p.alloc() for _ in range(5)]
    assert sorted(got) == list(range(5))
    with pytest.raises(CacheFull):
        p.alloc()
    p.free(3)
    with pytest.raises(CacheError):
        p.free(3)                       # freed twice
    with pytest.raises(CacheError):
        p.free(17)                      # never given out
    assert p.alloc() == 3               # reused
    with pytest.raises(CacheFull):
        p.alloc_many(2)
    p.check()


def make_cache(max_tokens=640, max_seqs=6):
    specs = {0: StateSpec((8, 2)), 1: KVSpec(2, 16), 2: StateSpec((8, 2)), 3: KVSpec(2, 16),
             4: KVSpec(2, 16, window=100, v_head_dim=24), 5: StateSpec((4,))}
    return Cache(specs, max_tokens=max_tokens, max_seqs=max_seqs, dtype=torch.float32, device="cpu")


def test_groups_have_storage_of_their_own():
    c = make_cache()
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 2
    full = c.kv_groups[c.group_of(1)[1]]
    win = c.kv_groups[c.group_of(4)[1]]
    assert full.k_pool.shape == (2, 10, 2, 64, 16) and full.v_pool.shape == (2, 10, 2, 16, 64)
    assert win.k_pool.shape == (1, 10, 2, 64, 16) and win.v_pool.shape == (1, 10, 2, 24, 64)      # values wider than keys
    assert c.state_groups[c.group_of(0)[1]].data.shape == (2, 6, 8, 2)
    assert c.group_of(1) == c.group_of(3) != c.group_of(4)


def test_random_alloc_free_keeps_invariants():
    rnd = random.Random(0)
    c = make_cache(max_tokens=64 * 12, max_seqs=5)
    live = {}
    for _ in range(600):
        r = rnd.random()
        if r < 0.3 and len(live) < 5:
            s = c.alloc_seq()
            assert s not in live
            live[s] = 0
        elif r < 0.8 and live:
            s = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 5, 70, 200])
            try:
                c.reserve({s: n})
                c.commit({s: n})
                live[s] += n
            except CacheFull:
                pass                      # nothing may have changed
        elif live:
            s = rnd.choice(list(live))
            c.free_seq(s)
            del live[s]
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            full = c.kv_groups[0].seq_pages.get(s, [])
            assert len(full) == -(-n // 64) and all(p >= 0 for p in full)
    for s in list(live):
        c.free_seq(s)
    c.check()
    assert all(g.pages.n_held == 0 for g in c.kv_groups) and c.slots.n_held == 0


def test_cache_full_changes_nothing_and_names_the_need():
    c = make_cache(max_tokens=128, max_seqs=4)
    a, b = c.alloc_seq(), c.alloc_seq()
    c.reserve({a: 64})
    c.commit({a: 64})
    before = {g: dict((k, list(v)) for k, v in g.seq_pages.items()) for g in c.kv_groups}
    with pytest.raises(CacheFull, match="2 more cache pages"):
        c.reserve({a: 1, b: 1})
    assert all(before[g] == g.seq_pages for g in c.kv_groups)
    c.check()
    with pytest.raises(CacheError):
        c.free_seq(3)
    c.free_seq(a)
    with pytest.raises(CacheError):
        c.free_seq(a)
    with pytest.raises(CacheError):
        c.length(a)


def test_window_group_gives_pages_back_and_slot_state_is_zeroed():
    c = make_cache()
    s = c.alloc_seq()
    c.state_groups[0].data[:, s] = 5.0
    c.reserve({s: 300})
    win = c.kv_groups[c.group_of(4)[1]]
    assert len(win.seq_pages[s]) == 5 and all(p >= 0 for p in win.seq_pages[s])   # all there during the step
    c.commit({s: 300})
    # the next query is at 300 and reaches back to 201: pages 0..2 (positions < 192) are gone
    assert [p >= 0 for p in win.seq_pages[s]] == [False, False, False, True, True]
    assert all(p >= 0 for p in c.kv_groups[c.group_of(1)[1]].seq_pages[s])
    t = win.table([s, -1], 6)
    assert t.shape == (2, 6) and list(t[0, :3]) == [-1, -1, -1] and t[0, 3] >= 0 and list(t[1]) == [-1] * 6
    c.check()
    c.free_seq(s)
    s2 = c.alloc_seq()
    assert s2 == s and float(c.state_groups[0].data[:, s2].abs().max()) == 0.0     # reused, and clean


def test_a_sequence_goes_out_as_bytes_and_comes_back_in_other_pages():
    c = make_cache(max_tokens=1280, max_seqs=6)
    g = torch.Generator().manual_seed(3)
    for grp in c.kv_groups:
        grp.k_pool.copy_(torch.randn(grp.k_pool.shape, generator=g))
        grp.v_pool.copy_(torch.randn(grp.v_pool.shape, generator=g))
    other = c.alloc_seq()
    c.reserve({other: 70}); c.commit({other: 70})          # so that the copy lands in other pages
    s = c.alloc_seq()
    for grp in c.state_groups:
        grp.data[:, s] = torch.randn(grp.data[:, s].shape, generator=g)
    c.reserve({s: 150}); c.commit({s: 150})
    data = c.export_seq(s)
    kv = 2 * 150 * 2 * 16 * 4
    kv_win = 150 * 2 * (16 + 24) * 4                        # the windowed entry's values are 24 wide
    assert len(data) == 8 + 2 * kv + kv_win + (16 + 16 + 4) * 4 and int.from_bytes(data[:8], "little") == 150
    # keys of entry 1 follow the state of entry 0, as [position][kv head][dim]
    full = c.kv_groups[c.group_of(1)[1]]
    k = torch.frombuffer(bytearray(data[8 + 64:8 + 64 + kv // 2]), dtype=torch.float32).view(150, 2, 16)
    assert torch.equal(k[70], full.k_pool[0, full.seq_pages[s][1], :, 6, :])
    win = c.kv_groups[c.group_of(4)[1]]
    v = torch.frombuffer(bytearray(data[-16 - kv_win + 150 * 2 * 16 * 4:-16]), dtype=torch.float32).view(150, 2, 24)
    assert torch.equal(v[130], win.v_pool[0, win.seq_pages[s][2], :, :, 2])
    t = c.import_seq(data)
    assert t != s and c.length(t) == 150 and c.export_seq(t) == data
    assert set(full.seq_pages[t]).isdisjoint(full.seq_pages[s])
    win = c.kv_groups[c.group_of(4)[1]]
    assert [p >= 0 for p in win.seq_pages[t]] == [p >= 0 for p in win.seq_pages[s]] == [True, True, True]
    c.check()
    # bytes of another model, and no room: both leave the cache as it was
    held, free = c.slots.n_held, [grp.pages.n_free for grp in c.kv_groups]
    with pytest.raises(CacheError, match="does not match"):
        c.import_seq(data[:-4])
    with pytest.raises(CacheError, match="too short"):
        c.import_seq(b"abc")
    for _ in range(8):
        try:
            c.import_seq(data)
        except CacheFull:
            break
    else:
        raise AssertionError("the cache never filled")
    c.check()
    with pytest.raises(CacheFull):
        c.import_seq(data)
    assert c.slots.n_held > held and all(grp.pages.n_free <= f for grp, f in zip(c.kv_groups, free))
    c.check()


def test_workspace_keeps_addresses_and_hands_out_the_same_views():
    from lastengine_b200.engine.workspace import Workspace
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    assert ws.get("x", (4, 8), torch.float32) is a                     # the same request: the same tensor
    b = ws.get("x", (2, 8), torch.bfloat16)                             # another shape and type under the name: same storage
    assert b.data_ptr() == a.data_ptr() and b.shape == (2, 8) and b.dtype == torch.bfloat16
    gen = ws.generation
    a.fill_(3.0)
    big = ws.get("x", (64, 8), torch.float32)                           # does not fit: new storage, graphs are told
    assert ws.generation == gen + 1 and big.data_ptr() != a.data_ptr()
    again = ws.get("x", (4, 8), torch.float32)                          # the old view is not handed out again
    assert again is not a and again.data_ptr() == big.data_ptr()
    ws.frozen = True
    assert ws.get("x", (4, 8), torch.float32) is again
    with pytest.raises(RuntimeError, match="would grow"):
        ws.get("x", (1024, 8), torch.float32)


def test_xorshift_matches_the_reference_recurrence():
    g = XorShift64(None)
    assert g.state == 0x9E3779B97F4A7C15
    s = 0x9E3779B97F4A7C15
    m = (1 << 64) - 1
    s ^= (s << 13) & m
    s ^= s >> 7
    s ^= (s << 17) & m
    assert g.next() == (s >> 40) / (1 << 24)
    assert XorShift64(7).state == ((7 * 0x9E3779B97F4A7C15) & m) | 1
    assert XorShift64(7, stream=2).state == XorShift64(9).state
    assert all(0.0 <= XorShift64(3).next() < 1.0 for _ in range(3))


class Scripted:
    """A backend that plays tokens from a script: request r's i-th token is script[r][i]."""

    def __init__(self, script, n_slots=8):
        self.script, self.free, self.owner, self.count = script, list(range(n_slots)), {}, {}
        self.log = []

    def _req(self, prompt):
        return prompt[0]                 # the test puts the request number first in the prompt

    def start(self, prompts, u01, histories):
        slots = [self.free.pop(0) for _ in prompts]
        for s, p in zip(slots, prompts):
            self.owner[s], self.count[s] = self._req(p), 0
        self.log.append(("start", list(slots), [self._req(p) for p in prompts], u01))
        return slots, [self._next(s) for s in slots]

    def _next(self, s):
        t = self.script[self.owner[s]][self.count[s]]
        self.count[s] += 1
        return t

    def decode(self, slots, tokens, u01, histories):
        for i, (s, t) in enumerate(zip(slots, tokens)):
            assert t == self.script[self.owner[s]][self.count[s] - 1]
            assert histories is None or histories[i][-1] == t
        self.log.append(("decode", list(slots), u01))
        return [self._next(s) for s in slots]

    def finish(self, slots):
        for s in slots:
            del self.owner[s]
            self.free.insert(0, s)
        self.log.append(("finish", list(slots)))


def test_loop_stop_tokens_budgets_and_batches():
    script = {0: [5, 6, 99, 7], 1: [99], 2: [1, 2, 3, 4, 5, 6], 3: [8, 8, 8, 8, 8, 8], 4: [9, 99]}
    be = Scripted(script)
    loop = GenerationLoop(be, SamplingParams(temperature=0.0), max_new_tokens=4, stop_token_ids=[99], max_batch=3)
    res = loop.run([[0, 50], [1], [2, 50, 51], [3], [4, 1, 2, 3]])
    assert res.tokens == [[5, 6], [], [1, 2, 3, 4], [8, 8, 8, 8], [9]]
    assert res.finish_reasons == ["stop", "stop", "length", "length", "stop"]
    assert res.stats.batches == 2 and res.stats.prefill_tokens == 2 + 1 + 3 + 1 + 4
    kinds = [e[0] for e in be.log]
    assert kinds.count("start") == 2
    # request 1 ends at once, request 0 after two tokens, request 2 runs to its budget alone
    first = be.log[:kinds.index("start", 1)]
    assert first[1] == ("finish", [1])
    decodes = [e for e in first if e[0] == "decode"]
    assert [len(e[1]) for e in decodes] == [2, 2, 1]
    # the second batch reuses the slots the first gave back
    assert set(be.log[kinds.index("start", 1)][1]) <= {0, 1, 2}
    assert not be.owner and res.stats.decode_tokens == sum(len(e[1]) for e in be.log if e[0] == "decode")
    assert all(e[-1] is None for e in be.log if e[0] in ("start", "decode"))     # greedy draws nothing


def test_loop_context_budget_and_sampling_streams():
    be = Scripted({0: [1] * 10, 1: [2] * 10})
    loop = GenerationLoop(be, SamplingParams(temperature=0.7, seed=11), max_new_tokens=8, max_seq_len=6)
    res = loop.run([[0, 9, 9], [1, 9, 9, 9, 9]])
    # budget = min(8, 6 - 1 - prompt): 2 tokens for the first, none for the second (it is never started)
    assert res.tokens == [[1, 1], []] and res.finish_reasons == ["length", "length"]
    u = be.log[0][3]
    assert u == [XorShift64(11, stream=0).next()]
    with pytest.raises(ValueError, match="empty prompt"):
        loop.run([[]])


def test_loop_builds_histories_only_for_penalties():
    be = Scripted({0: [1, 2, 3]})
    GenerationLoop(be, SamplingParams(temperature=0.0), max_new_tokens=3).run([[0, 5]])
    be2 = Scripted({0: [1, 2, 3]})
    seen = []
    orig = be2.decode
    be2.decode = lambda slots, tokens, u01, histories: (seen.append(histories), orig(slots, tokens, u01, histories))[1]
    GenerationLoop(be2, SamplingParams(temperature=0.0, repeat_penalty=1.2), max_new_tokens=3).run([[0, 5]])
    assert seen and seen[0] == [[0, 5, 1]]


class LookingAhead(Scripted):
    """A scripted backend that takes the loop's look-ahead and checks that the loop keeps it."""
    lookahead = True

    def __init__(self, script):
        super().__init__(script)
        self.promised = None

    def decode(self, slots, tokens, u01, histories, lookahead=None):
        if self.promised is not None:
            next_u, may, given = self.promised
            assert set(slots) <= may                                   # only requests said to go on come back
            assert all(given[s] == t for s, t in zip(slots, tokens))   # and they are fed what was chosen
            if next_u is not None:
                assert [next_u[s] for s in slots] == u01
        res = super().decode(slots, tokens, u01, histories)
        assert lookahead is not None
        nu, goes_on = lookahead
        self.promised = (dict(zip(slots, nu)) if nu is not None else None,
                         {s for s, c in zip(slots, goes_on) if c}, dict(zip(slots, res)))
        return res

    def start(self, prompts, u01, histories):
        self.promised = None
        return super().start(prompts, u01, histories)


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_loop_look_ahead_is_a_promise_it_keeps(temperature):
    script = {0: [5, 6, 99, 7], 1: [99], 2: [1, 2, 3, 4, 5, 6], 3: [8, 8, 8, 8, 8, 8], 4: [9, 99]}
    be = LookingAhead(script)
    loop = GenerationLoop(be, SamplingParams(temperature=temperature, seed=3), max_new_tokens=4, stop_token_ids=[99], max_batch=3)
    res = loop.run([[0, 50], [1], [2, 50, 51], [3], [4, 1, 2, 3]])
    assert res.tokens == [[5, 6], [], [1, 2, 3, 4], [8, 8, 8, 8], [9]]
    plain = Scripted(script)
    res2 = GenerationLoop(plain, SamplingParams(temperature=temperature, seed=3), max_new_tokens=4, stop_token_ids=[99],
                          max_batch=3).run([[0, 50], [1], [2, 50, 51], [3], [4, 1, 2, 3]])
    assert res2.tokens == res.tokens and plain.log == be.log          # the same calls with the same numbers
    g = XorShift64(5)
    a = g.peek()
    assert a == g.next() and g.peek() != a


def test_plan_batches_respects_cache_room():
    assert plan_batches([10, 10, 10], [5, 5, 5], max_batch=2, token_budget=1000, page=64) == [[0, 1], [2]]
    assert plan_batches([60, 60, 60], [10, 10, 10], max_batch=8, token_budget=256, page=64) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="request 1 needs room"):
        plan_batches([10, 300], [5, 5], max_batch=8, token_budget=256, page=64)
