"""Decode steps as captured CUDA graphs.

A decode step is a fixed sequence of launches whose arguments do not change from token to
token: positions, slots and page tables live in device memory that the host refreshes with
one copy before each replay.  The reference captures its decode layer loop the same way, with
the position in device memory (src/gpu/dense.rs:270-337, :21).  One graph per batch-size
bucket; a batch smaller than its bucket is filled up with padding sequences, which change no
result.  Each bucket has scratch memory of its own, so prompts of any size between two decode
steps cannot move what a graph points at.
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache import CacheFull
from ..ops import kernels
from ..sampling.params import PENALTY_WINDOW, SamplingParams
from ..sampling.sampler import Sampler
from .batch import BatchBuilder
from .generate import EngineBackend
from .workspace import Workspace

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return -(-n // 256) * 256


class DecodeGraph:
    """The captured step of one bucket: forward pass, choice of the next tokens, and (for runs
    that feed themselves) the move to the next position."""

    def __init__(self, engine, sampler: Sampler, bucket: int, table_width: int, self_feeding: bool = False,
                 out: torch.Tensor | None = None, fed: bool = False, history=None, workspace: Workspace | None = None,
                 rows: int | None = None):
        """`table_width`: pages per sequence the step's page tables have; the longest sequence a
        replay can serve, and the length the split of the decode attention is chosen for.  `out`:
        where the chosen tokens go (shared between the graphs of one backend, so that a step of
        one bucket can take its tokens from the step of another).  `fed`: the step begins by
        taking tokens from `out` where the staged step says so.  `history`: (ring of recent
        tokens per cache slot [slots, 256], tokens seen per slot) on the device, for the penalties.
        `workspace`: scratch shared with the other widths of the same bucket.  `rows`: the step is
        one of short prompts, padded to this many rows (`stage_prompts`); `bucket` then counts its
        sequences with the padding ones."""
        self.history = history
        self.rows = rows
        self.engine, self.sampler, self.bucket, self.width = engine, sampler, bucket, table_width
        self.self_feeding, self.fed = self_feeding, fed
        self.ws = workspace if workspace is not None else Workspace(engine.device)
        self.builder = BatchBuilder(engine.device)
        self.out = out if out is not None else torch.zeros(bucket, dtype=torch.int32, device=engine.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.batch = None
        self.staged_slots: list[int] = []
        self.cache_version = -1
        self.launches = 0
        self.ws_generation = -1

    def _run(self, batch) -> None:
        eng = self.engine
        if batch.feed is not None:
            kernels.feed_tokens(batch, self.out)
        logits = eng.model.forward(batch, eng.cache)
        p = self.sampler.params
        if p.has_penalties and self.history is not None:
            kernels.penalties_slots(logits, self.history[0], self.history[1], batch.seq_slot, p.repeat_penalty,
                                    p.presence_penalty)
        self.sampler.sample(self.out[:self.bucket], logits, batch.u01)
        if p.has_penalties and self.history is not None:
            kernels.history_append(self.history[0], self.history[1], batch.seq_slot, self.out, self.bucket)
        if self.self_feeding:
            kernels.advance(batch, self.out)

    def stage(self, slots: list[int], tokens: list[int] | None, u01, feed=None) -> dict[int, int]:
        """Lays the step's inputs out in this bucket's fixed device buffers (one copy).  With
        `feed`, sequence i takes the token the previous step chose at place feed[i]."""
        eng = self.engine
        pad = self.bucket - len(slots)
        seqs = list(slots) + [-1] * pad
        toks = [[t] for t in (tokens if tokens is not None else [0] * len(slots))] + [[0]] * pad
        u = None
        if self.sampler.needs_uniform():
            u = np.zeros(self.bucket, dtype=np.float32)
            u[:len(slots)] = u01
        fd = None
        if self.fed:
            fd = np.full(self.bucket, -1, dtype=np.int32)
            if feed is not None:
                fd[:len(slots)] = feed
        batch, grow = eng.prepare(seqs, toks, "last", u01=u, builder=self.builder, table_width=self.width, feed=fd)
        if self.batch is not None:
            same = (batch.tokens.data_ptr() == self.batch.tokens.data_ptr()
                    and all(batch.tables[k].data_ptr() == self.batch.tables[k].data_ptr() for k in batch.tables))
            if not same:
                self.graph = None      # the staging buffer moved: capture again
        # what is baked into the graph must not depend on how long the sequences are today
        batch.max_kvlen = self.width * eng.cache.page_size
        self.batch = batch
        self.staged_slots = list(slots)
        return grow

    def stage_prompts(self, slots: list[int], prompts: list[list[int]], u01) -> dict[int, int]:
        """Lays a step of whole prompts out in the fixed buffers: the prompts' rows, one row for each
        padding sequence that fills the bucket, and a last padding sequence whose rows fill the
        step up to `rows`.  What the captured kernels take as numbers (rows, sequences, the longest
        prompt, the longest sequence) is the bucket's, not this step's."""
        eng = self.engine
        n = len(slots)
        fill = self.bucket - 1 - n                       # padding sequences of one row
        rest = self.rows - sum(len(p) for p in prompts) - fill
        assert fill >= 0 and rest >= 1, "the bucket was chosen too small for the prompts"
        seqs = list(slots) + [-1] * (fill + 1)
        toks = [list(p) for p in prompts] + [[0]] * fill + [[0] * rest]
        u = None
        if self.sampler.needs_uniform():
            u = np.zeros(self.bucket, dtype=np.float32)
            u[:n] = u01
        batch, grow = eng.prepare(seqs, toks, "last", u01=u, builder=self.builder, table_width=self.width)
        if self.batch is not None:
            same = (batch.tokens.data_ptr() == self.batch.tokens.data_ptr()
                    and all(batch.tables[k].data_ptr() == self.batch.tables[k].data_ptr() for k in batch.tables))
            if not same:
                self.graph = None      # the staging buffer moved: capture again
        assert batch.n_rows == self.rows and batch.n_seqs == self.bucket
        batch.max_kvlen = self.width * eng.cache.page_size
        batch.max_qlen = self.rows
        self.batch = batch
        self.staged_slots = []         # not a step restage() can follow
        return grow

    def restage(self, slots: list[int], tokens: list[int] | None, u01, feed=None) -> dict[int, int] | None:
        """The step after the one staged before, for the same sequences in the same order: only
        the tokens, the positions (+1) and, where a sequence enters a new page, one entry of its
        page table change.  Done in place in the staging buffer, then one copy.  Returns None
        when the step is not of that kind (the caller stages it in full)."""
        eng, bb = self.engine, self.builder
        if self.batch is None or slots != self.staged_slots or eng.cache.state_version != self.cache_version:
            return None
        if any(g.spec.window > 0 for g in eng.cache.kv_groups):
            return None      # windowed groups give pages back as they go: stage those steps in full
        cache = eng.cache
        n = len(slots)
        page = cache.page_size
        pos = bb.host_view("seq_pos0")
        grow = {}
        if bb._copied is not None:
            bb._copied.synchronize()          # the last copy has read the buffer we are about to change
        new_page = [i for i in range(n) if (int(pos[i]) + 1) % page == 0]
        if new_page:
            cache.reserve({slots[i]: 1 for i in new_page})
            for gi, g in enumerate(cache.kv_groups):
                tab = bb.host_view(f"table{gi}").reshape(self.bucket, -1)
                for i in new_page:
                    lst = g.seq_pages[slots[i]]
                    if len(lst) > tab.shape[1]:
                        return None
                    tab[i, len(lst) - 1] = lst[-1]
        if tokens is not None:
            bb.host_view("tokens")[:n] = tokens
        if "feed" in bb.layout:
            bb.host_view("feed")[:n] = feed if feed is not None else -1
        pos[:n] += 1
        bb.host_view("row_pos")[:n] += 1
        if u01 is not None and "u01" in bb.layout:
            bb.host_view("u01")[:n] = np.asarray(u01, dtype=np.float32).view(np.int32)
        bb.resend(None if new_page else bb.head_total)
        for s in slots:
            grow[s] = 1
        return grow

    def launch(self) -> None:
        eng = self.engine
        saved = eng.env.workspace
        eng.env.workspace = self.ws
        try:
            if self.graph is None or self.ws_generation != self.ws.generation:
                self._run(self.batch)            # warm-up: loads kernels, sizes the scratch memory
                torch.cuda.current_stream().synchronize()
                before = kernels.launch_count()
                g = torch.cuda.CUDAGraph()
                self.ws.frozen = True
                try:
                    with torch.cuda.graph(g):
                        self._run(self.batch)
                finally:
                    self.ws.frozen = False
                self.launches = kernels.launch_count() - before
                self.graph, self.ws_generation = g, self.ws.generation
                # capturing executes nothing and the warm-up ran the step: it has run exactly once
            else:
                self.graph.replay()
        finally:
            eng.env.workspace = saved


class _StepInFlight:
    """A launched decode step whose chosen tokens the host has not read yet."""

    def __init__(self, number: int, slots: list[int], host: torch.Tensor, event: torch.cuda.Event):
        self.number, self.slots, self.host, self.event = number, slots, host, event


class GraphBackend(EngineBackend):
    """The generation loop's backend with graph-replayed decode steps, launched one step ahead.

    While the device runs step k the host has nothing to do but wait, and after it the device
    would wait for the host to read the tokens, decide and stage step k+1.  So when the loop
    says which requests can go on after step k (`lookahead`), step k+1 is launched for them
    before step k's tokens are read: it takes its tokens from step k's choices on the device.
    A request that step k ends with a stop token has then run one step too many; its row is
    dropped, and its slot is given back only after that step has finished, since the step
    still writes to its pages.  Rows do not depend on each other, so the other requests'
    tokens are those they would have got without it.
    """

    lookahead = True

    def __init__(self, engine, sampling: SamplingParams, max_batch: int = 64, max_seq_len: int | None = None):
        super().__init__(engine, sampling)
        page = engine.cache.page_size
        self.max_width = -(-(max_seq_len or engine.max_tokens) // page)
        # Captured graphs outlive one call: they belong to the engine, keyed by what is baked into
        # them: the sampling constants here, and per graph the bucket and the width of its page
        # tables.  The width follows the sequences that are live (the next power of two of their
        # pages), not the cache's capacity: the decode attention chooses its split for the width,
        # and a short sequence in a large cache must not be split and merged for lengths it has not.
        store = engine.__dict__.setdefault("_decode_graphs", {})
        self.graphs: dict = store.setdefault(sampling, {})
        self.h2d_bytes = 0
        self._ahead: _StepInFlight | None = None
        self._launched = 0
        self._held: list[tuple[int, list[int]]] = []     # (step number to wait for, slots to give back)
        self._fed: dict[int, int] = {}                    # slot -> the token the next step was given on the device

    def _chosen(self, n: int) -> torch.Tensor:
        """Where the steps put their chosen tokens: the buffer behind the device's status word (one
        copy then brings both to the host), or for very large batches a buffer of the backend's own."""
        if n <= kernels.RESULT_TOKENS:
            return kernels.result_tokens(self.engine.device)
        out = self.graphs.get("out")
        if out is None or out.numel() < n:
            # graphs point at the old buffer: they are captured again with the new one
            for k in [k for k in self.graphs if isinstance(k, tuple)]:
                del self.graphs[k]
            out = self.graphs["out"] = torch.zeros(n, dtype=torch.int32, device=self.engine.device)
        return out

    def _width_for(self, slots) -> int:
        """Pages the step's tables need: the next power of two of what the longest sequence holds
        after this step, at most the width of the longest sequence allowed."""
        cache = self.engine.cache
        need = max(-(-(cache.length(s) + 1) // cache.page_size) for s in slots)
        w = 1
        while w < need:
            w *= 2
        return max(need, min(w, self.max_width))

    def _history(self):
        """The rings of recent tokens per cache slot (made when the sampling has penalties)."""
        if not self.sampler.params.has_penalties:
            return None
        h = self.graphs.get("history")
        if h is None:
            n = self.engine.cache.max_seqs
            h = self.graphs["history"] = (torch.zeros((n, PENALTY_WINDOW), dtype=torch.int32, device=self.engine.device),
                                          torch.zeros(n, dtype=torch.int32, device=self.engine.device))
        return h

    def _launch(self, slots, tokens, u01, feed) -> _StepInFlight:
        eng = self.engine
        b = bucket_for(len(slots))
        out = self._chosen(b)
        width = self._width_for(slots)
        g = self.graphs.get((b, width))
        if g is None:
            ws = self.graphs.setdefault(("scratch", b), Workspace(eng.device))
            g = self.graphs[(b, width)] = DecodeGraph(eng, self.sampler, b, width, out=out, fed=True,
                                                      history=self._history(), workspace=ws)
        grow = g.restage(slots, tokens, u01, feed)
        if grow is None:
            grow = g.stage(slots, tokens, u01, feed)
        g.launch()
        eng.cache.commit(grow)
        g.cache_version = eng.cache.state_version
        n = len(slots)
        self._launched += 1
        host = torch.empty(n + 1, dtype=torch.int32, pin_memory=True) if n > 1024 else \
            self._hosts[self._launched % 2]
        # the status word and the tokens: one copy where they lie together
        if n <= kernels.RESULT_TOKENS:
            host[:n + 1].copy_(kernels.status_and_tokens(eng.device, n), non_blocking=True)
        else:
            host[:1].copy_(kernels.status_and_tokens(eng.device, 0), non_blocking=True)
            host[1:n + 1].copy_(out[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.h2d_bytes = g.builder.last_h2d_bytes
        self.d2h_bytes = (n + 1) * 4
        return _StepInFlight(self._launched, list(slots), host, ev)

    @property
    def _hosts(self):
        h = self.__dict__.get("_host_pair")
        if h is None:
            h = self.__dict__["_host_pair"] = [torch.empty(1025, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        return h

    def _wait(self, step: _StepInFlight, check: bool = True) -> list[int]:
        """The step's tokens, once it has finished.  The status word came with them: a kernel that
        gave up on a bounded wait in this step raises KernelError here (`check`)."""
        step.event.synchronize()
        vals = step.host[:len(step.slots) + 1].tolist()
        toks = vals[1:]
        still = []
        for number, slots in self._held:
            if number <= step.number:
                self.engine.release(slots)
            else:
                still.append((number, slots))
        self._held = still
        if check:
            kernels.raise_on_status(vals[0], self.engine.device)
        return toks

    def _drain(self, check: bool = True) -> None:
        if self._ahead is not None:
            step, self._ahead = self._ahead, None
            self._wait(step, check)
        self._fed = {}

    def abort(self, slots):
        """After a failed step: waits for what is in flight, then gives back `slots` and whatever
        was held until a step ahead had finished."""
        self._drain(check=False)
        torch.cuda.synchronize(self.engine.device)
        for _, held in self._held:
            self.engine.release(held)
        self._held = []
        self.engine.release([s for s in slots if self.engine.cache.slots.holds(s)])

    # Short prompts as captured steps: a prompt step launches some 125 kernels from the host, which
    # takes longer than the device needs for them below a few hundred rows.  Buckets of rows and of
    # sequences; a step that fits none, or sampling with penalties (whose first token looks at the
    # prompt on the host), runs uncaptured.
    PROMPT_ROWS = (32, 64, 128, 256, 512)
    PROMPT_SEQS = (1, 2, 4, 8)

    def _start_captured(self, prompts, u01):
        eng = self.engine
        n = len(prompts)
        if self.sampler.params.has_penalties or n > self.PROMPT_SEQS[-1] or any(len(p) == 0 for p in prompts):
            return None
        nb = next(b for b in self.PROMPT_SEQS if n <= b)
        need = sum(len(p) for p in prompts) + (nb - n) + 1
        rows = next((r for r in self.PROMPT_ROWS if need <= r), None)
        if rows is None:
            return None
        page = eng.cache.page_size
        width = 1
        while width * page < max(len(p) for p in prompts) + 1:
            width *= 2
        if width > self.max_width:
            return None
        slots = [eng.new_sequence() for _ in prompts]
        try:
            out = self._chosen(nb + 1)
            key = ("prompts", rows, nb, width)
            g = self.graphs.get(key)
            if g is None:
                ws = self.graphs.setdefault(("prompt scratch", rows), Workspace(eng.device))
                g = self.graphs[key] = DecodeGraph(eng, self.sampler, nb + 1, width, out=out, workspace=ws, rows=rows)
            grow = g.stage_prompts(slots, prompts, u01)
            g.launch()
            eng.cache.commit(grow)
            host = self._hosts[0]
            host[:n + 1].copy_(kernels.status_and_tokens(eng.device, n), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            vals = host[:n + 1].tolist()
            kernels.raise_on_status(vals[0], eng.device)
            self.h2d_bytes = g.builder.last_h2d_bytes
            return slots, vals[1:]
        except Exception:
            eng.release(slots)
            raise

    def start(self, prompts, u01, histories):
        self._drain()
        captured = self._start_captured(prompts, u01)
        slots, toks = captured if captured is not None else super().start(prompts, u01, histories)
        h = self._history()
        if h is not None:
            # the rings of the new sequences: their last tokens, the first chosen one among them
            rows = np.zeros((len(slots), PENALTY_WINDOW), dtype=np.int32)
            lens = np.zeros(len(slots), dtype=np.int32)
            for i, (p, t) in enumerate(zip(prompts, toks)):
                seen = len(p) + 1
                tail = (list(p) + [int(t)])[-PENALTY_WINDOW:]
                for j, tok in enumerate(tail):              # token number q of the sequence lies at q % window
                    rows[i, (seen - len(tail) + j) % PENALTY_WINDOW] = tok
                lens[i] = seen
            idx = torch.tensor(slots, dtype=torch.long, device=self.engine.device)
            h[0][idx] = torch.from_numpy(rows).to(self.engine.device)
            h[1][idx] = torch.from_numpy(lens).to(self.engine.device)
        return slots, toks

    def finish(self, slots):
        if self._ahead is None:
            self.engine.release(slots)
            return
        self._held.append((self._ahead.number, list(slots)))
        gone = {s for _, ss in self._held for s in ss}
        if all(s in gone for s in self._ahead.slots):
            self._drain()          # nothing of the step ahead is wanted any more

    def decode(self, slots, tokens, u01, histories, lookahead=None):
        """`lookahead` = (the uniform numbers of the step after this one or None, for each slot
        whether its request can go on after this step's token)."""
        step, self._ahead = self._ahead, None
        if step is not None:
            place = {s: i for i, s in enumerate(step.slots)}
            if any(s not in place or self._fed.get(s) != t for s, t in zip(slots, tokens)):
                self._wait(step)
                raise RuntimeError("decode was asked for a step other than the one launched ahead "
                                   "(a request that was said to end goes on, or a token other than the chosen one is fed)")
            pick = [place[s] for s in slots]
        else:
            step = self._launch(slots, tokens, u01, None)
            pick = list(range(len(slots)))
        if lookahead is not None:
            next_u01, goes_on = lookahead
            keep = [i for i, c in enumerate(goes_on) if c]
            if keep and (next_u01 is not None or not self.sampler.needs_uniform()):
                try:
                    self._ahead = self._launch([slots[i] for i in keep], None,
                                               [next_u01[i] for i in keep] if next_u01 is not None else None,
                                               [pick[i] for i in keep])
                except CacheFull:
                    self._ahead = None      # no room to run ahead: the next step is staged when it is asked for
        toks = self._wait(step)
        res = [toks[i] for i in pick]
        self._fed = dict(zip(slots, res)) if self._ahead is not None else {}
        return res
