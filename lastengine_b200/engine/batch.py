"""The rows of one step, as the kernels see them.

A step holds the next tokens of B sequences, packed row after row without padding:
sequence b owns rows [seq_qstart[b], seq_qstart[b] + seq_qlen[b]).  Everything the device
needs to know about the step (tokens, the sequence and position of each row, slots, lengths,
page tables, the rows whose logits are wanted) is laid out in one pinned host buffer and goes
over in one copy.  A sequence with slot -1 is padding: its rows are computed and thrown away,
they touch no cache and change no other row.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepBatch:
    n_rows: int
    n_seqs: int
    max_qlen: int
    max_kvlen: int
    tokens: torch.Tensor       # int32 [rows]
    row_seq: torch.Tensor      # int32 [rows]   index of the row's sequence in this step
    row_pos: torch.Tensor      # int32 [rows]   absolute position of the row's token
    seq_slot: torch.Tensor     # int32 [seqs]   cache slot, -1 for padding
    seq_pos0: torch.Tensor     # int32 [seqs]   length of the sequence before this step
    seq_qstart: torch.Tensor   # int32 [seqs]   first row
    seq_qlen: torch.Tensor     # int32 [seqs]   number of rows
    logit_rows: torch.Tensor   # int32 [wanted] rows whose logits are computed
    n_logit_rows: int
    tables: dict[int, torch.Tensor] = field(default_factory=dict)   # kv group -> int32 [seqs, pages]
    u01: torch.Tensor | None = None   # float32 [seqs] uniform numbers for sampling
    feed: torch.Tensor | None = None  # int32 [seqs] place in the previous step's choices to take the token from, or -1
    slots_host: list[int] = field(default_factory=list)

    @property
    def row_slot(self) -> torch.Tensor:
        """Cache slot of every row (for parts written with tensor operations)."""
        return self.seq_slot[self.row_seq.long()]


class BatchBuilder:
    """Lays a step out in a pinned staging buffer and copies it to the device in one go."""

    def __init__(self, device: torch.device):
        self.device = device
        self._host: torch.Tensor | None = None
        self._dev: torch.Tensor | None = None
        self._copied: torch.cuda.Event | None = None   # the last copy out of the staging buffer

    def _ensure(self, n: int) -> None:
        if self._host is None or self._host.numel() < n:
            cap = max(1024, int(n * 1.5))
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)

    def build(self, slots: list[int], tokens: list[list[int]] | list[np.ndarray], pos0: list[int],
              logit_rows: list[int], tables: dict[int, np.ndarray],
              u01: np.ndarray | None = None, feed: np.ndarray | None = None) -> StepBatch:
        B = len(slots)
        qlen = np.fromiter((len(t) for t in tokens), dtype=np.int32, count=B)
        M = int(qlen.sum())
        qstart = np.zeros(B, dtype=np.int32)
        if B > 1:
            np.cumsum(qlen[:-1], out=qstart[1:])
        pos0a = np.asarray(pos0, dtype=np.int32)
        tok = np.concatenate([np.asarray(t, dtype=np.int32) for t in tokens]) if M else np.zeros(0, np.int32)
        row_seq = np.repeat(np.arange(B, dtype=np.int32), qlen)
        row_pos = (np.arange(M, dtype=np.int32) - np.repeat(qstart, qlen) + np.repeat(pos0a, qlen)).astype(np.int32)
        lr = np.asarray(logit_rows, dtype=np.int32)
        pieces = [tok, row_seq, row_pos, np.asarray(slots, dtype=np.int32), pos0a, qstart, qlen, lr]
        tkeys = sorted(tables)
        if u01 is not None:
            pieces.append(np.asarray(u01, dtype=np.float32).view(np.int32))
        if feed is not None:
            pieces.append(np.asarray(feed, dtype=np.int32))
        n_head = len(pieces)      # the page tables come last: they change least often
        pieces += [np.ascontiguousarray(tables[k], dtype=np.int32).reshape(-1) for k in tkeys]
        # 4-int alignment keeps every piece 16-byte aligned
        offs, total = [], 0
        for p in pieces:
            offs.append(total)
            total += (p.size + 3) // 4 * 4
        if self._copied is not None:
            self._copied.synchronize()   # the previous step's copy has read the staging buffer
        self._ensure(total + 4)
        host = self._host.numpy()
        for o, p in zip(offs, pieces):
            host[o:o + p.size] = p
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()
        self.last_h2d_bytes = total * 4
        names = ["tokens", "row_seq", "row_pos", "seq_slot", "seq_pos0", "seq_qstart", "seq_qlen", "logit_rows"]
        names += (["u01"] if u01 is not None else []) + (["feed"] if feed is not None else [])
        names += [f"table{k}" for k in tkeys]
        self.layout = {n: (o, p.size) for n, o, p in zip(names, offs, pieces)}
        self.total = total
        self.head_total = offs[n_head] if tkeys else total     # everything before the page tables
        d = self._dev

        def piece(i):
            return d[offs[i]:offs[i] + pieces[i].size]

        tabs = {}
        for j, k in enumerate(tkeys):
            tabs[k] = piece(n_head + j).view(B, -1)
        u = piece(8).view(torch.float32) if u01 is not None else None
        fd = piece(8 + (u01 is not None)) if feed is not None else None
        return StepBatch(
            n_rows=M, n_seqs=B, max_qlen=int(qlen.max()) if B else 0,
            max_kvlen=int((pos0a + qlen).max()) if B else 0,
            tokens=piece(0), row_seq=piece(1), row_pos=piece(2), seq_slot=piece(3), seq_pos0=piece(4),
            seq_qstart=piece(5), seq_qlen=piece(6), logit_rows=piece(7), n_logit_rows=int(lr.size),
            tables=tabs, u01=u, feed=fd, slots_host=list(slots))

    # ---- the same step again, one position later -----------------------------------------------
    def host_view(self, name: str) -> np.ndarray:
        """The staged copy of one piece of the last built step (int32; `u01` as raw bits)."""
        o, n = self.layout[name]
        return self._host.numpy()[o:o + n]

    def resend(self, n_ints: int | None = None) -> None:
        """Copies the staging buffer (or its first `n_ints` words) to the device again, after
        the caller changed pieces of it in place.  The device addresses stay what they were."""
        if self._copied is not None:
            self._copied.synchronize()
        n = self.total if n_ints is None else n_ints
        self._dev[:n].copy_(self._host[:n], non_blocking=True)
        self._copied.record()
        self.last_h2d_bytes = n * 4
