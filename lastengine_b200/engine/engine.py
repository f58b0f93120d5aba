"""The step function and what it stands on: model, cache, workspace.

`Engine.step` takes a batch of sequences that either all start (their prompts, of unequal
lengths, in one step) or all go on (one token each; any number of tokens each also works),
runs exactly the tokens it is given as one packed batch against the cache, and returns the
logits at the wanted rows.  The reference's counterpart serves one sequence: `prefill(ids)`
gives the last position's logits and `forward(token)` the next (src/gpu/dense.rs:348,371).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields, replace
from typing import Sequence

import numpy as np
import torch

from ..cache import Cache, CacheError
from ..config.base import read_config_json
from ..parts.base import BuildEnv, ModelPlan
from ..registry import plan_from_config
from .batch import BatchBuilder, StepBatch
from .model import Model
from .workspace import Workspace

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


class StepError(ValueError):
    """A step that cannot run: unknown sequence, empty token list, token id outside the vocabulary."""


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16, float32)")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{dtype}' (bfloat16, float32)") from None


@dataclass(frozen=True)
class EngineOptions:
    """What an engine is built with, beside the model.  The reference sets the like through `--ctx`
    and `LE_*` variables (src/cli.rs:47); its prompt pieces are 512 rows (src/gpu/dense.rs:28,376)."""
    dtype: str = "bfloat16"            # "bfloat16" or "float32" (true 32-bit arithmetic throughout)
    max_seqs: int | None = None        # sequences alive at once (default: as many as there are cache pages)
    max_tokens: int = 8192             # positions all live sequences may hold together, each rounded up to whole pages
    max_batch_tokens: int = 16384      # rows one pass over the layers takes; a longer step runs in pieces (0: no limit)
    use_graphs: bool = True            # decode steps of `generate` as captured CUDA graphs
    seed: int | None = None            # sampling seed for calls whose SamplingParams name none
    device: str = "cuda:0"

    def __post_init__(self):
        resolve_dtype(self.dtype)
        if self.max_tokens < 1 or (self.max_seqs is not None and self.max_seqs < 1) or self.max_batch_tokens < 0:
            raise ValueError(f"engine options out of range: {self}")

    @staticmethod
    def of(options: "EngineOptions | None", **overrides) -> "EngineOptions":
        """`options` (or the defaults) with the given fields replaced; unknown names are an error."""
        known = {f.name for f in fields(EngineOptions)}
        bad = sorted(set(overrides) - known)
        if bad:
            raise TypeError(f"unknown engine option(s) {bad}; known: {sorted(known)}")
        if "dtype" in overrides and isinstance(overrides["dtype"], torch.dtype):
            overrides["dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(overrides["dtype"], str(overrides["dtype"]))
        if "device" in overrides:
            overrides["device"] = str(overrides["device"])
        return replace(options or EngineOptions(), **overrides)


class Engine:
    def __init__(self, plan: ModelPlan, options: EngineOptions | None = None, **overrides):
        """`options`, or single fields of it by name (`dtype=`, `max_tokens=`, ...)."""
        self.options = opt = EngineOptions.of(options, **overrides)
        dtype, max_tokens, max_seqs, device = opt.dtype, opt.max_tokens, opt.max_seqs, opt.device
        dev = torch.device(device)
        if dev.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError("lastengine_b200 runs on a CUDA device only (no CPU path); "
                               f"asked for '{device}', torch.cuda.is_available() = {torch.cuda.is_available()}")
        torch.cuda.set_device(dev)
        from ..ops import kernels
        kernels.lib()   # build or load the kernels now: fail here, loudly, if they are missing
        self.device = dev
        self.dtype = resolve_dtype(dtype)
        self.plan = plan
        self.workspace = Workspace(dev)
        self.env = BuildEnv(device=dev, dtype=self.dtype, workspace=self.workspace)
        self.model = Model(plan, self.env)
        self.max_tokens = int(max_tokens)
        self.cache = Cache(self.model.cache_specs(), max_tokens=self.max_tokens, max_seqs=max_seqs,
                           dtype=self.dtype, device=dev)
        self.builder = BatchBuilder(dev)
        self.vocab_size = plan.vocab_size
        self.loaded = False

    # ---- construction --------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir: str, options: EngineOptions | None = None, **kw) -> "Engine":
        """A folder with config.json and model.safetensors; the model class is chosen by config.json."""
        from ..weights import load_model_dir
        raw = read_config_json(model_dir)
        eng = cls(plan_from_config(raw), options, **kw)
        load_model_dir(eng.model, model_dir)
        eng.loaded = True
        eng.config = raw
        return eng

    @classmethod
    def from_config(cls, config: dict | str, seed: int = 0, options: EngineOptions | None = None,
                    norm_init: str = "ones", **kw) -> "Engine":
        """Random weights made on the device from a configuration and a seed (the weights' seed;
        `EngineOptions.seed` is the sampling seed)."""
        from ..weights import load_random
        raw = read_config_json(config) if isinstance(config, (str, os.PathLike)) else config
        eng = cls(plan_from_config(raw), options, **kw)
        load_random(eng.model, seed, norm_init=norm_init)
        eng.loaded = True
        eng.config = raw
        return eng

    # ---- sequences ------------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.alloc_seq()

    def release(self, seqs: int | Sequence[int]) -> None:
        for s in ([seqs] if isinstance(seqs, int) else seqs):
            self.cache.free_seq(s)

    def length(self, seq: int) -> int:
        return self.cache.length(seq)

    def export_sequence(self, seq: int) -> bytes:
        """The sequence's cache as bytes (`Cache.export_seq`); waits for the device first."""
        torch.cuda.synchronize(self.device)
        return self.cache.export_seq(seq)

    def import_sequence(self, data: bytes) -> int:
        """A new sequence that goes on where the exported one stood."""
        return self.cache.import_seq(data)

    # ---- the step -------------------------------------------------------------------------
    def check_step(self, seqs, tokens, want) -> tuple[list[int], list[int]]:
        """Raises StepError for a step that cannot run; returns (each sequence's length before the
        step, the step's rows whose logits are wanted)."""
        if not self.loaded:
            raise RuntimeError("the engine has no weights yet")
        if len(seqs) != len(tokens) or len(seqs) == 0:
            raise StepError(f"a step needs as many token lists as sequences, and at least one "
                            f"({len(seqs)} sequences, {len(tokens)} token lists)")
        live = [s for s in seqs if s >= 0]
        if len(set(live)) != len(live):
            raise StepError("a sequence appears twice in one step")
        V = self.vocab_size
        pos0 = []
        for s, t in zip(seqs, tokens):
            if len(t) == 0:
                raise StepError(f"sequence {s} brings no tokens to the step")
            if s >= 0:
                try:
                    pos0.append(self.cache.length(s))
                except CacheError:
                    raise StepError(f"sequence {s} is not live (never started, or already released)") from None
                ta = np.asarray(t)
                if ta.min() < 0 or ta.max() >= V:
                    bad = int(ta[(ta < 0) | (ta >= V)][0])
                    raise StepError(f"token id {bad} of sequence {s} is outside the vocabulary [0, {V})")
            else:
                pos0.append(0)
        if isinstance(want, str) and want == "last":
            rows, r0 = [], 0
            for t in tokens:
                r0 += len(t)
                rows.append(r0 - 1)
        elif want is None:
            rows = []
        else:
            if isinstance(want, str) or len(want) != len(seqs):
                raise StepError("`want` is \"last\", None, or one list of places per sequence")
            rows, r0 = [], 0
            for t, w in zip(tokens, want):
                for i in w:
                    if not 0 <= i < len(t):
                        raise StepError(f"wanted place {i} is outside the {len(t)} tokens the sequence brings")
                    rows.append(r0 + i)
                r0 += len(t)
        return pos0, rows

    def prepare(self, seqs: Sequence[int], tokens: Sequence[Sequence[int]],
                want: str | Sequence[Sequence[int]] | None = "last",
                u01: np.ndarray | None = None, builder: BatchBuilder | None = None,
                table_width: int | None = None, feed: np.ndarray | None = None) -> tuple[StepBatch, dict[int, int]]:
        """Checks a step, reserves its cache room and lays it out on the device."""
        pos0, rows = self.check_step(seqs, tokens, want)
        live = [s for s in seqs if s >= 0]
        grow = {s: len(t) for s, t in zip(seqs, tokens) if s >= 0}
        self.cache.reserve(grow)
        tables = {}
        for gi, g in enumerate(self.cache.kv_groups):
            width = table_width or max(1, max((len(g.seq_pages.get(s, ())) for s in live), default=1))
            tables[gi] = g.table(list(seqs), width)
        b = (builder or self.builder).build(list(seqs), tokens, pos0, rows, tables, u01=u01, feed=feed)
        return b, grow

    def step(self, seqs: Sequence[int], tokens: Sequence[Sequence[int]],
             want: str | Sequence[Sequence[int]] | None = "last", check: bool = False) -> torch.Tensor:
        """Feeds `tokens[i]` to sequence `seqs[i]` and returns float logits [wanted rows, vocab].

        `want`: "last" (the last token of each sequence), None (nothing), or per sequence the
        places among its tokens of this step.  The result lives in workspace memory that the
        next step overwrites: copy it if it must outlive the step.  A step of more rows than
        `options.max_batch_tokens` runs in pieces of at most that many rows, one after the other
        against the cache, with the same result.  `check`: wait for the device and raise
        KernelError if a kernel of the step gave up on a bounded wait (`check_status`).
        """
        limit = self.options.max_batch_tokens
        if limit and sum(len(t) for t in tokens) > limit:
            logits = self._step_in_pieces(seqs, tokens, want, limit)
        else:
            batch, grow = self.prepare(seqs, tokens, want)
            logits = self.model.forward(batch, self.cache)
            self.cache.commit(grow)
        if check:
            self.check_status()
        return logits

    def check_status(self) -> None:
        """Waits for the device and raises KernelError if a tensor-core kernel gave up on one of its
        bounded waits since the last check: what such a step computed is not valid.  The
        generation loop reads the same word with every step's tokens."""
        from ..ops import kernels
        kernels.check_device_status()

    def _step_in_pieces(self, seqs, tokens, want, limit: int) -> torch.Tensor:
        """The step cut into pieces of at most `limit` rows (a sequence's tokens may be cut too:
        its later part finds the earlier one in the cache).  Checked and given cache room as a
        whole first, so that it runs entirely or not at all."""
        if isinstance(want, str) and want == "last":
            places = [[len(t) - 1] if len(t) else [] for t in tokens]
        elif want is None:
            places = [[] for _ in tokens]
        else:
            places = [list(w) for w in want]
        self.check_step(seqs, tokens, places)
        self.cache.reserve({s: len(t) for s, t in zip(seqs, tokens) if s >= 0})
        R = sum(len(w) for w in places)
        out = self.workspace.get("engine.logits_of_pieces", (R, self.vocab_size), torch.float32)
        pieces, cur, room = [], [], limit
        for i, t in enumerate(tokens):
            lo = 0
            while lo < len(t):
                n = min(room, len(t) - lo)
                cur.append((i, lo, lo + n))
                lo, room = lo + n, room - n
                if room == 0:
                    pieces.append(cur)
                    cur, room = [], limit
        if cur:
            pieces.append(cur)
        # rows of `out`: in the order of the sequences and of their places, as one step would give them
        first_row, r = [], 0
        for w in places:
            first_row.append(r)
            r += len(w)
        for piece in pieces:
            p_want, dst = [], []
            for i, lo, hi in piece:
                p_want.append([k - lo for k in places[i] if lo <= k < hi])
                dst += [first_row[i] + j for j, k in enumerate(places[i]) if lo <= k < hi]
            batch, grow = self.prepare([seqs[i] for i, _, _ in piece], [tokens[i][lo:hi] for i, lo, hi in piece], p_want)
            lg = self.model.forward(batch, self.cache)
            self.cache.commit(grow)
            r = 0
            while r < len(dst):          # runs of consecutive rows go over in one copy
                e = r + 1
                while e < len(dst) and dst[e] == dst[e - 1] + 1:
                    e += 1
                out[dst[r]:dst[r] + e - r].copy_(lg[r:e])
                r = e
        return out

    # ---- numbers for reports --------------------------------------------------------------
    def step_costs(self) -> dict:
        """What a step costs, summed over the schedule from what the parts say of themselves (no
        knowledge of the architecture): matrix-product flops per row through the layers and per
        row of logits, mixer flops per (row, cached position), cache bytes per position and state
        bytes per sequence."""
        esize = 2 if self.dtype == torch.bfloat16 else 4
        layer_flops = pair_flops = kv_bytes = state_bytes = 0
        for i, e in enumerate(self.plan.schedule):
            blk = self.model.blocks[e.layer]
            layer_flops += sum(p.flops_per_row() for p in blk.parts().values())
            pair_flops += blk.mixer.flops_per_query_key()
        for spec in self.model.cache_specs().values():
            if spec is None:
                continue
            if hasattr(spec, "n_kv_heads"):
                kv_bytes += spec.n_kv_heads * (spec.head_dim + spec.value_dim) * esize
            else:
                n = 1
                for d in spec.shape:
                    n *= int(d)
                state_bytes += n * torch.empty((), dtype=spec.dtype).element_size()
        return {"layer_flops_per_row": layer_flops, "head_flops_per_row": self.model.head.flops_per_row(),
                "flops_per_query_key": pair_flops, "kv_bytes_per_token": kv_bytes, "state_bytes_per_seq": state_bytes}

    def weight_bytes_read(self, rows: int) -> float:
        """Bytes of weights a step of `rows` rows is expected to read: all of them, less the experts
        that nobody is expected to choose."""
        return self.weight_bytes() - sum(p.unread_weight_bytes(rows) for _, p in self.model.named_parts())

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for _, part in self.model.named_parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    n += v.numel() * v.element_size()
        return n
