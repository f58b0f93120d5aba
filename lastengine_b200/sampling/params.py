"""Sampling options, with the reference's names, meanings and defaults.

src/backend.rs:6 (the struct) and src/server/mod.rs:106-110 (the defaults a request gets):
temperature 0.7 (<= 0 means greedy), top_p 0.95, top_k 40 (0 means 64; at most 256),
min_p 0, presence_penalty 0, repeat_penalty 1.0 (both over the last 256 tokens), seed.
"""
from __future__ import annotations

from dataclasses import dataclass

GOLDEN = 0x9E3779B97F4A7C15
MASK64 = (1 << 64) - 1
PENALTY_WINDOW = 256   # src/local.rs:61


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.95
    top_k: int = 40
    min_p: float = 0.0
    presence_penalty: float = 0.0
    repeat_penalty: float = 1.0
    seed: int | None = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return self.repeat_penalty > 1.0 or self.presence_penalty != 0.0   # src/local.rs:60

    @staticmethod
    def greedy_params() -> "SamplingParams":
        return SamplingParams(temperature=0.0)


class XorShift64:
    """The reference's generator (src/local.rs:57): s ^= s<<13; s ^= s>>7; s ^= s<<17;
    the top 24 bits over 2^24.  Seeded as (seed * GOLDEN) | 1 (src/local.rs:244); without a
    seed the state starts at GOLDEN (src/local.rs:38)."""

    def __init__(self, seed: int | None = None, stream: int = 0):
        # every request of a call has a stream of its own, so a request draws the same numbers
        # alone or in any batch; stream 0 is the reference's generator
        s = (seed if seed is not None else 1) + stream
        self.state = ((s * GOLDEN) & MASK64) | 1

    @staticmethod
    def _advance(s: int) -> int:
        s ^= (s << 13) & MASK64
        s ^= s >> 7
        s ^= (s << 17) & MASK64
        return s

    def next(self) -> float:
        self.state = self._advance(self.state)
        return (self.state >> 40) / float(1 << 24)

    def peek(self) -> float:
        """The number the next call of `next` will give; the state stays."""
        return (self._advance(self.state) >> 40) / float(1 << 24)
