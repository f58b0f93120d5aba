"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early,
and one batch after another until every request is served.

For one request the reference does: prefill the prompt, then repeat { sample; stop token?
-> finish "stop" without emitting or feeding it; emit; budget reached? -> finish "length";
feed the token } with budget = min(max_tokens, context - 1 - prompt length)
(src/local.rs:219,249-264).  Here a batch of requests starts together: all prompts in one
step, then one token per live request per step; a request that finishes leaves the batch
and gives its slot back at once, and the next batch starts when the current one is empty.

The loop's decisions do not touch the device: they run against a `backend` with three calls
(`start`, `decode`, `finish`), so they are tested on the CPU with a scripted backend.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Protocol, Sequence

from ..sampling.params import SamplingParams, XorShift64


@dataclass
class GenerationStats:
    """prefill tok/s = prompt tokens / prefill time; decode tok/s = tokens after each request's
    first / decode time (src/server/mod.rs:270-286)."""
    prefill_tokens: int = 0
    prefill_ms: float = 0.0
    decode_tokens: int = 0
    decode_ms: float = 0.0
    decode_steps: int = 0
    batches: int = 0

    @property
    def prefill_tok_s(self) -> float:
        return self.prefill_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tok_s(self) -> float:
        return self.decode_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


@dataclass
class GenerationResult:
    tokens: list[list[int]]
    finish_reasons: list[str]          # "stop" | "length"
    stats: GenerationStats = field(default_factory=GenerationStats)


class Backend(Protocol):
    def start(self, prompts: list[list[int]], u01: list[float] | None,
              histories: list[list[int]] | None) -> tuple[list[int], list[int]]:
        """Allocates a slot per prompt, runs all prompts in one step; returns (slots, first tokens)."""

    def decode(self, slots: list[int], tokens: list[int], u01: list[float] | None,
               histories: list[list[int]]) -> list[int]:
        """Feeds one token per slot; returns the next token of each.  A backend with a true
        attribute `lookahead` also takes `lookahead=(the following step's uniform numbers or
        None, for each slot whether its request can go on after this step)`, a promise that the
        next call feeds the returned tokens to a subset of those slots; it may run ahead on it."""

    def finish(self, slots: list[int]) -> None:
        """Gives the slots back."""


@dataclass
class _Request:
    index: int
    prompt: list[int]
    budget: int
    rng: XorShift64
    out: list[int] = field(default_factory=list)
    reason: str | None = None
    slot: int = -1

    @property
    def history(self) -> list[int]:
        return self.prompt + self.out


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def plan_batches(prompt_lens: Sequence[int], budgets: Sequence[int], max_batch: int, token_budget: int,
                 page: int) -> list[list[int]]:
    """Splits request indices, in order, into batches that fit the cache: at most `max_batch`
    requests, and the sum over the batch of (prompt + budget) rounded up to whole pages at most
    `token_budget`."""
    batches, cur, used = [], [], 0
    for i, (n, b) in enumerate(zip(prompt_lens, budgets)):
        need = round_up(n + max(b, 0), page)
        if need > token_budget:
            raise ValueError(f"request {i} needs room for {need} tokens; the cache holds {token_budget}")
        if cur and (len(cur) >= max_batch or used + need > token_budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    def __init__(self, backend: Backend, sampling: SamplingParams, max_new_tokens: int,
                 stop_token_ids: Sequence[int] = (), max_batch: int = 64, max_seq_len: int = 1 << 30,
                 token_budget: int = 1 << 30, page: int = 64, clock=time.perf_counter):
        self.backend, self.sampling = backend, sampling
        self.max_new = int(max_new_tokens)
        self.stop = set(int(t) for t in stop_token_ids)
        self.max_batch = max(1, int(max_batch))
        self.max_seq_len, self.token_budget, self.page = int(max_seq_len), int(token_budget), int(page)
        self.clock = clock

    def run(self, prompts: Sequence[Sequence[int]]) -> GenerationResult:
        reqs = []
        for i, p in enumerate(prompts):
            p = [int(t) for t in p]
            if not p:
                raise ValueError(f"request {i} has an empty prompt")
            budget = min(self.max_new, self.max_seq_len - 1 - len(p))      # src/local.rs:219,249
            reqs.append(_Request(i, p, budget, XorShift64(self.sampling.seed, stream=i)))
        stats = GenerationStats()
        live = [r for r in reqs if r.budget > 0]
        for r in reqs:
            if r.budget <= 0:
                r.reason = "length"
        draw = not self.sampling.greedy
        want_hist = self.sampling.has_penalties      # histories are only built for the penalties
        for group in plan_batches([len(r.prompt) for r in live], [r.budget for r in live],
                                  self.max_batch, self.token_budget, self.page):
            batch = [live[i] for i in group]
            stats.batches += 1
            t0 = self.clock()
            u = [r.rng.next() for r in batch] if draw else None
            slots, toks = self.backend.start([r.prompt for r in batch], u,
                                             [r.history for r in batch] if want_hist else None)
            stats.prefill_ms += (self.clock() - t0) * 1e3
            stats.prefill_tokens += sum(len(r.prompt) for r in batch)
            for r, s in zip(batch, slots):
                r.slot = s
            active = batch
            t1 = self.clock()
            try:
                active = self._decode_batch(active, toks, stats, draw, want_hist)
            except BaseException:
                # a step failed (no cache room, a kernel that gave up): nothing of the batch stays behind
                held = [r.slot for r in batch if r.reason is None]
                if held:
                    getattr(self.backend, "abort", self.backend.finish)(held)
                raise
            stats.decode_ms += (self.clock() - t1) * 1e3
        return GenerationResult([r.out for r in reqs], [r.reason or "length" for r in reqs], stats)

    def _decode_batch(self, active, toks, stats, draw, want_hist):
        """One batch from its first tokens until its last request has ended."""
        while True:
            done = []
            for r, t in zip(active, toks):
                t = int(t)
                if t in self.stop:                    # not emitted and not fed (src/local.rs:252)
                    r.reason = "stop"
                else:
                    r.out.append(t)
                    if len(r.out) >= r.budget:        # emitted, not fed (src/local.rs:262)
                        r.reason = "length"
                if r.reason is not None:
                    done.append(r)
            if done:
                self.backend.finish([r.slot for r in done])
                active = [r for r in active if r.reason is None]
            if not active:
                break
            u = [r.rng.next() for r in active] if draw else None
            kw = {}
            if getattr(self.backend, "lookahead", False):
                kw["lookahead"] = ([r.rng.peek() for r in active] if draw else None,
                                   [len(r.out) + 1 < r.budget for r in active])
            toks = self.backend.decode([r.slot for r in active], [r.out[-1] for r in active], u,
                                       [r.history for r in active] if want_hist else None, **kw)
            stats.decode_steps += 1
            stats.decode_tokens += len(active)
        return active


class EngineBackend:
    """Runs the loop's three calls on an Engine: steps on the device, tokens back to the host."""

    def __init__(self, engine, sampling: SamplingParams):
        import torch
        from ..sampling.sampler import Sampler
        self.engine = engine
        self.sampler = Sampler(sampling, engine.device)
        self._torch = torch
        self._host = torch.empty(1025, dtype=torch.int32, pin_memory=True)
        self.d2h_bytes = 0

    def _choose(self, logits, u01_dev, histories) -> list[int]:
        """Chooses a token per row of `logits` and brings the tokens to the host, the device's
        status word with them: a step in which a kernel gave up on a bounded wait raises KernelError
        instead of handing out what it left."""
        from ..ops import kernels
        torch, dev = self._torch, self.engine.device
        n = logits.shape[0]
        if n + 1 > self._host.numel():
            self._host = torch.empty(2 * n + 1, dtype=torch.int32, pin_memory=True)
        if histories is not None:
            self.sampler.apply_penalties(logits, histories)
        if n <= kernels.RESULT_TOKENS:
            self.sampler.sample(kernels.result_tokens(dev), logits, u01_dev)
            self._host[:n + 1].copy_(kernels.status_and_tokens(dev, n), non_blocking=True)
        else:                                      # more rows than the shared buffer holds: two copies
            out = torch.empty(n, dtype=torch.int32, device=dev)
            self.sampler.sample(out, logits, u01_dev)
            self._host[:1].copy_(kernels.status_and_tokens(dev, 0), non_blocking=True)
            self._host[1:n + 1].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes = (n + 1) * 4
        vals = self._host[:n + 1].tolist()
        kernels.raise_on_status(vals[0], dev)
        return vals[1:]

    def _step(self, slots, tokens, u01, histories) -> list[int]:
        import numpy as np
        eng = self.engine
        u = np.asarray(u01, dtype=np.float32) if u01 is not None else None
        limit = eng.options.max_batch_tokens
        if limit and sum(len(t) for t in tokens) > limit:
            # prompts of more rows than one pass takes: the step function cuts them
            logits = eng.step(slots, tokens, "last")
            u_dev = self._torch.from_numpy(u).to(eng.device) if u is not None else None
            return self._choose(logits, u_dev, histories)
        batch, grow = eng.prepare(slots, tokens, "last", u01=u)
        logits = eng.model.forward(batch, eng.cache)
        eng.cache.commit(grow)
        return self._choose(logits, batch.u01, histories)

    def start(self, prompts, u01, histories):
        slots = [self.engine.new_sequence() for _ in prompts]
        try:
            return slots, self._step(slots, prompts, u01, histories)
        except Exception:
            self.engine.release(slots)
            raise

    def decode(self, slots, tokens, u01, histories):
        return self._step(slots, [[t] for t in tokens], u01, histories)

    def finish(self, slots):
        self.engine.release(slots)

    abort = finish
