"""The cache: per-sequence keys/values and fixed-size state, for every layer that keeps any.

A sequence gets a slot when it starts and gives it back when it ends; slots and pages are
reused.  Layers are grouped by what they need:

* a KV group per distinct (kv heads, key head size, value head size, window): pools of pages of
  `page_size` positions, keys `[entry, page, kv_head, position in page, head_dim]` and values
  `[entry, page, kv_head, value_dim, position in page]`, with a page pool and a page list per
  sequence of its own.  A windowed group gives pages back once every position in
  them has left the window.
* a state group per distinct (shape, dtype): `[entry, slot, *shape]`, zeroed when a slot is
  given out (the reference zeroes its convolution state on reset, src/gpu/dense.rs:264-267).

The reference keeps one sequence: K/V `[ctx][kv_head][head_dim]` per attention layer and a
float convolution state per conv layer (src/gpu/dense.rs:91-107).  Lengths live on the host;
each step carries the positions, slots and page tables it needs to the device, so the device
holds nothing per sequence but the data itself.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np
import torch

from ..parts.base import KVSpec, StateSpec
from .allocator import CacheError, CacheFull, IdPool

PAGE_SIZE = 64


@dataclass
class CacheView:
    """What one schedule entry's mixer sees of the cache during a step."""
    writable: bool
    page_size: int = PAGE_SIZE
    k: torch.Tensor | None = None            # [page, kv_head, page_size, head_dim]
    v: torch.Tensor | None = None            # [page, kv_head, value_dim, page_size] (positions contiguous)
    block_table: torch.Tensor | None = None  # int32 [sequences of the step, pages]
    state: torch.Tensor | None = None        # [slot, *shape]


class KVGroup:
    def __init__(self, spec: KVSpec, entries: list[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device):
        self.spec, self.entries = spec, list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.page_size = page_size
        # keys as [.., position, dim], values as [.., dim, position]
        self.k_pool = torch.zeros((len(entries), n_pages, spec.n_kv_heads, page_size, spec.head_dim),
                                  dtype=dtype, device=device)
        self.v_pool = torch.zeros((len(entries), n_pages, spec.n_kv_heads, spec.value_dim, page_size),
                                  dtype=dtype, device=device)
        self.pages = IdPool(n_pages, "cache page")
        self.seq_pages: dict[int, list[int]] = {}   # slot -> page of each page index (-1: given back)

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.seq_pages.get(slot, ()))
        return max(0, -(-new_len // self.page_size) - have)

    def grow(self, slot: int, new_len: int) -> None:
        lst = self.seq_pages.setdefault(slot, [])
        lst.extend(self.pages.alloc_many(self.pages_needed(slot, new_len)))

    def trim(self, slot: int, length: int) -> None:
        """Gives back the pages no later query can reach (windowed groups only)."""
        w = self.spec.window
        if w <= 0:
            return
        first_needed = length + 1 - w     # the next query, at position `length`, reaches back to here
        lst = self.seq_pages.get(slot, [])
        for j, p in enumerate(lst):
            if p >= 0 and (j + 1) * self.page_size - 1 < first_needed:
                self.pages.free(p)
                lst[j] = -1

    def release(self, slot: int) -> None:
        for p in self.seq_pages.pop(slot, []):
            if p >= 0:
                self.pages.free(p)

    def table(self, slots: list[int], width: int) -> np.ndarray:
        t = np.full((len(slots), max(width, 1)), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            if s < 0:
                continue
            lst = self.seq_pages.get(s, [])
            if len(lst) > width:
                raise CacheError(f"sequence in slot {s} holds {len(lst)} pages, the step's table has {width}")
            t[i, :len(lst)] = lst
        return t


class StateGroup:
    def __init__(self, spec: StateSpec, entries: list[int], max_seqs: int, device):
        self.spec, self.entries = spec, list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.data = torch.zeros((len(entries), max_seqs, *spec.shape), dtype=spec.dtype, device=device)


class Cache:
    def __init__(self, specs: dict[int, KVSpec | StateSpec], max_tokens: int, max_seqs: int | None,
                 dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        """`specs`: cache entry id -> what it keeps.  `max_tokens`: positions all live sequences
        may hold together, each sequence rounded up to whole pages."""
        if page_size % 32 != 0:
            raise ValueError("page size must be a multiple of 32")
        self.page_size = page_size
        self.n_pages = max(1, -(-int(max_tokens) // page_size))
        self.max_seqs = int(max_seqs) if max_seqs else self.n_pages
        self.dtype, self.device = dtype, device
        self.slots = IdPool(self.max_seqs, "sequence slot")
        self.lens: dict[int, int] = {}
        self.state_version = 0      # bumped by every change of lengths, pages or slots
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self._where: dict[int, tuple[str, int]] = {}
        by_spec: dict[object, list[int]] = {}
        for entry, spec in sorted(specs.items()):
            if spec is not None:
                by_spec.setdefault(spec, []).append(entry)
        for spec, entries in by_spec.items():
            if isinstance(spec, KVSpec):
                self.kv_groups.append(KVGroup(spec, entries, self.n_pages, page_size, dtype, device))
                for e in entries:
                    self._where[e] = ("kv", len(self.kv_groups) - 1)
            elif isinstance(spec, StateSpec):
                self.state_groups.append(StateGroup(spec, entries, self.max_seqs, device))
                for e in entries:
                    self._where[e] = ("state", len(self.state_groups) - 1)
            else:
                raise TypeError(f"unknown cache spec {spec!r}")

    # ---- sequences -----------------------------------------------------------------------
    def alloc_seq(self) -> int:
        slot = self.slots.alloc()
        self.state_version += 1
        self.lens[slot] = 0
        for g in self.state_groups:
            g.data[:, slot].zero_()
        return slot

    def free_seq(self, slot: int) -> None:
        if not self.slots.holds(slot):
            raise CacheError(f"sequence slot {slot} is not held (freed twice, or never given out)")
        self.state_version += 1
        for g in self.kv_groups:
            g.release(slot)
        del self.lens[slot]
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        try:
            return self.lens[slot]
        except KeyError:
            raise CacheError(f"sequence slot {slot} is not held") from None

    def reserve(self, grow: dict[int, int]) -> None:
        """Makes room for `grow[slot]` more positions per sequence, or raises CacheFull and
        leaves everything as it was."""
        for g in self.kv_groups:
            need = sum(g.pages_needed(s, self.length(s) + n) for s, n in grow.items())
            if need > g.pages.n_free:
                raise CacheFull(f"the step needs {need} more cache pages of {self.page_size} positions, "
                                f"{g.pages.n_free} of {g.pages.n} are free")
        for g in self.kv_groups:
            for s, n in grow.items():
                g.grow(s, self.lens[s] + n)

    def commit(self, grow: dict[int, int]) -> None:
        """After the step ran: the sequences are `grow[slot]` positions longer."""
        self.state_version += 1
        for s, n in grow.items():
            self.lens[s] += n
            for g in self.kv_groups:
                g.trim(s, self.lens[s])

    def pages_held(self, slot: int) -> int:
        return max((len(g.seq_pages.get(slot, ())) for g in self.kv_groups), default=0)

    # ---- a sequence as bytes --------------------------------------------------------------
    def _entry_nbytes(self, entry: int, length: int) -> int:
        kind, gi = self._where[entry]
        if kind == "state":
            g = self.state_groups[gi]
            return int(np.prod(g.spec.shape, dtype=np.int64)) * g.data.element_size()
        sp = self.kv_groups[gi].spec
        return length * sp.n_kv_heads * (sp.head_dim + sp.value_dim) * self.kv_groups[gi].k_pool.element_size()

    def export_seq(self, slot: int) -> bytes:
        """What a sequence holds, as bytes: its length (u64, little-endian), then for every cache
        entry in order its state, or its keys and then its values as `[position][kv head][dim]`
        in the cache's dtype.  The reference writes one sequence the same way: position count,
        then per layer the state or K and V up to that position (src/gpu/dense.rs:391-399).
        Positions that a windowed group has given back are written as zeros."""
        n = self.length(slot)
        out = [struct.pack("<Q", n)]
        raw = lambda t: t.contiguous().view(torch.uint8).cpu().numpy().tobytes()
        ps = self.page_size
        for entry in sorted(self._where):
            kind, gi = self._where[entry]
            if kind == "state":
                g = self.state_groups[gi]
                out.append(raw(g.data[g.index[entry], slot].reshape(-1)))
                continue
            g = self.kv_groups[gi]
            i, sp = g.index[entry], g.spec
            pages = g.seq_pages.get(slot, [])
            k = torch.zeros((len(pages) * ps, sp.n_kv_heads, sp.head_dim), dtype=self.dtype, device=self.device)
            v = torch.zeros((len(pages) * ps, sp.n_kv_heads, sp.value_dim), dtype=self.dtype, device=self.device)
            for j, p in enumerate(pages):
                if p >= 0:
                    k[j * ps:(j + 1) * ps] = g.k_pool[i, p].permute(1, 0, 2)
                    v[j * ps:(j + 1) * ps] = g.v_pool[i, p].permute(2, 0, 1)
            out.append(raw(k[:n].reshape(-1)))
            out.append(raw(v[:n].reshape(-1)))
        return b"".join(out)

    def import_seq(self, data: bytes) -> int:
        """A new sequence that holds what `export_seq` wrote (same model, same dtype).  Raises
        CacheError when the bytes do not fit this model and CacheFull when there is no room; the
        cache is then as it was (the reference checks the same two things, src/gpu/dense.rs:400-412)."""
        if len(data) < 8:
            raise CacheError("sequence data is too short to hold a length")
        (n,) = struct.unpack_from("<Q", data, 0)
        need = 8 + sum(self._entry_nbytes(e, n) for e in self._where)
        if len(data) != need:
            raise CacheError(f"sequence data of {len(data)} bytes does not match this model and dtype "
                             f"({need} bytes for {n} positions)")
        slot = self.alloc_seq()
        try:
            self.reserve({slot: n})
        except CacheFull:
            self.free_seq(slot)
            raise
        ps, o = self.page_size, 8
        buf = torch.frombuffer(bytearray(data), dtype=torch.uint8).to(self.device)
        for entry in sorted(self._where):
            kind, gi = self._where[entry]
            nb = self._entry_nbytes(entry, n)
            if kind == "state":
                g = self.state_groups[gi]
                dst = g.data[g.index[entry], slot]
                dst.copy_(buf[o:o + nb].clone().view(g.data.dtype).view(dst.shape))
                o += nb
                continue
            g = self.kv_groups[gi]
            i, sp = g.index[entry], g.spec
            pages = g.seq_pages.get(slot, [])
            for which, width in ((0, sp.head_dim), (1, sp.value_dim)):
                part = nb * width // (sp.head_dim + sp.value_dim)
                t = torch.zeros((len(pages) * ps, sp.n_kv_heads, width), dtype=self.dtype, device=self.device)
                if n:
                    t[:n] = buf[o:o + part].clone().view(self.dtype).view(n, sp.n_kv_heads, width)
                o += part
                for j, p in enumerate(pages):
                    rows = t[j * ps:(j + 1) * ps]
                    if which == 0:
                        g.k_pool[i, p] = rows.permute(1, 0, 2)
                    else:
                        g.v_pool[i, p] = rows.permute(1, 2, 0)
        self.commit({slot: n})
        return slot

    # ---- views ---------------------------------------------------------------------------
    def group_of(self, entry: int) -> tuple[str, int] | None:
        return self._where.get(entry)

    def view(self, entry: int, writable: bool, tables: dict[int, torch.Tensor]) -> CacheView:
        w = self._where.get(entry)
        if w is None:
            return CacheView(writable=writable, page_size=self.page_size)
        kind, gi = w
        if kind == "kv":
            g = self.kv_groups[gi]
            i = g.index[entry]
            sp = g.spec
            return CacheView(writable=writable, page_size=self.page_size, k=g.k_pool[i], v=g.v_pool[i],
                             block_table=tables[gi])
        g = self.state_groups[gi]
        return CacheView(writable=writable, page_size=self.page_size, state=g.data[g.index[entry]])

    def check(self) -> None:
        """Bookkeeping invariants (used by tests): nothing lost, nothing held twice."""
        self.slots.check()
        assert set(self.lens) == self.slots._held
        for g in self.kv_groups:
            g.pages.check()
            held = [p for lst in g.seq_pages.values() for p in lst if p >= 0]
            assert len(held) == len(set(held)), "a page belongs to two sequences"
            assert set(held) == g.pages._held, "held pages and page lists disagree"
            assert set(g.seq_pages) <= self.slots._held, "a freed sequence still owns pages"

    def nbytes(self) -> int:
        n = sum((g.k_pool.numel() + g.v_pool.numel()) * g.k_pool.element_size() for g in self.kv_groups)
        return n + sum(g.data.numel() * g.data.element_size() for g in self.state_groups)
