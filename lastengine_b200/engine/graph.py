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

from ..ops import kernels
from ..sampling.params import SamplingParams
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

    def __init__(self, engine, sampler: Sampler, bucket: int, table_width: int, self_feeding: bool = False):
        self.engine, self.sampler, self.bucket, self.width = engine, sampler, bucket, table_width
        self.self_feeding = self_feeding
        self.ws = Workspace(engine.device)
        self.builder = BatchBuilder(engine.device)
        self.out = torch.zeros(bucket, dtype=torch.int32, device=engine.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.batch = None
        self.staged_slots: list[int] = []
        self.cache_version = -1
        self.launches = 0

    def _run(self, batch) -> None:
        eng = self.engine
        logits = eng.model.forward(batch, eng.cache)
        self.sampler.sample(self.out, logits, batch.u01)
        if self.self_feeding:
            kernels.advance(batch, self.out)

    def stage(self, slots: list[int], tokens: list[int], u01) -> dict[int, int]:
        """Lays the step's inputs out in this bucket's fixed device buffers (one copy)."""
        eng = self.engine
        pad = self.bucket - len(slots)
        seqs = list(slots) + [-1] * pad
        toks = [[t] for t in tokens] + [[0]] * pad
        u = None
        if self.sampler.needs_uniform():
            u = np.zeros(self.bucket, dtype=np.float32)
            u[:len(slots)] = u01
        batch, grow = eng.prepare(seqs, toks, "last", u01=u, builder=self.builder, table_width=self.width)
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

    def restage(self, slots: list[int], tokens: list[int], u01) -> dict[int, int] | None:
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
        bb.host_view("tokens")[:n] = tokens
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


class GraphBackend(EngineBackend):
    """The generation loop's backend with graph-replayed decode steps."""

    def __init__(self, engine, sampling: SamplingParams, max_batch: int = 64, max_seq_len: int | None = None):
        super().__init__(engine, sampling)
        page = engine.cache.page_size
        self.width = -(-(max_seq_len or engine.max_tokens) // page)
        # Captured graphs outlive one call: they belong to the engine, keyed by what is baked into
        # them (the sampling constants and the width of the page tables).
        store = engine.__dict__.setdefault("_decode_graphs", {})
        self.graphs: dict[int, DecodeGraph] = store.setdefault((sampling, self.width), {})
        self.h2d_bytes = 0

    def decode(self, slots, tokens, u01, histories):
        if self.sampler.params.has_penalties:
            return super().decode(slots, tokens, u01, histories)
        eng = self.engine
        b = bucket_for(len(slots))
        g = self.graphs.get(b)
        if g is None:
            g = self.graphs[b] = DecodeGraph(eng, self.sampler, b, self.width)
        grow = g.restage(slots, tokens, u01)
        if grow is None:
            grow = g.stage(slots, tokens, u01)
        g.launch()
        eng.cache.commit(grow)
        g.cache_version = eng.cache.state_version
        n = len(slots)
        self._host[:n].copy_(g.out[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.h2d_bytes = g.builder.last_h2d_bytes
        self.d2h_bytes = n * 4
        return self._host[:n].tolist()
