"""What a part of a layer is, and what a model is made of.

A layer is put together from parts: a mixer (attention, short convolution, ...), a
feed-forward (dense or experts), norms and a position encoding, arranged by a block.
Each part gets its sizes and constants as constructor arguments and knows nothing of the
model around it.  Which parts a layer has is data (`PartSpec`), chosen layer by layer; the
order in which layers run is data too (`ScheduleEntry`).

Interfaces
----------
Every part:
    tensors()  -> {relative name: TensorSpec}     what it reads from the checkpoint
    load(tensors, env)                             takes its tensors (already on the device,
                                                   in the dtype of their role) and may fuse them
Mixer:
    cache_spec() -> KVSpec | StateSpec | None      what it keeps per sequence
    forward(h, out, accumulate, batch, cache, env) h: [rows, hidden] normed input in the
                                                   activation dtype; writes (or adds) its
                                                   result into the float tensor `out`
FeedForward:
    forward(h, out, accumulate, batch, env)
Norm:
    forward(out, x, rows=None, add=False)          x float; out in any activation dtype
PositionEncoding:
    fused_rotary() -> (inv_freq, rope_dim, neox)   a rotation that the mixer's kernel applies itself
                      | None                       while it norms q and k and stores k and v, or
    apply(q, k, row_pos)                           any other encoding, in place on the normed
                                                   q [rows, heads, head_dim] and k [rows, kv heads, head_dim]
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

# roles decide the random initialisation and the dtype a tensor is kept in
MATRIX = "matrix"        # operand of a matrix product: kept in the compute dtype
EMBEDDING = "embedding"  # token table: compute dtype
NORM = "norm"            # norm weight: kept float
VECTOR = "vector"        # small per-channel parameters (conv taps, router rows): kept float
BIAS = "bias"            # additive terms: kept float

FLOAT_ROLES = (NORM, VECTOR, BIAS)


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple[int, ...]
    role: str
    std: float | None = None      # random init: normal(0, std); None: the model's default
    optional: bool = False        # may be absent from the checkpoint
    shared_name: str | None = None  # the tensor's full name where it belongs to the model, not to the
                                    # part's prefix (several parts may then name the same tensor)


@dataclass(frozen=True)
class KVSpec:
    """Keys and values that grow with the sequence; `window` > 0 keeps only the last ones.
    `v_head_dim`: width of a value head where it differs from a key head's (None: the same)."""
    n_kv_heads: int
    head_dim: int
    window: int = 0
    v_head_dim: int | None = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per sequence, zero when the sequence starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PartSpec:
    kind: str                      # name in the registry of its family
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                    # tensor-name prefix of the layer, e.g. "layers.3"
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    post_mixer_norm: PartSpec | None = None
    post_ffn_norm: PartSpec | None = None
    block: str = "pre_norm_residual"
    # tensor-name prefixes of the parts, relative to `prefix`
    names: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One step of the layer order: run `layer` with the cache entry `cache`.

    By default entry i runs layer i with its own cache entry i.  Naming a layer twice runs
    its weights twice; `cache` pointing at an earlier entry with `writes_cache=False` lets a
    layer read what that entry stored instead of storing its own.
    """
    layer: int
    cache: int | None = None
    writes_cache: bool = True


@dataclass
class ModelPlan:
    """Everything needed to build a model: parts, their order, and the tensor names."""
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    init_std: float = 0.02
    init_stds: dict[str, float] = field(default_factory=dict)   # tensor-name suffix -> std, before init_std
    eos_token_ids: tuple[int, ...] = ()
    names: dict[str, str] = field(default_factory=dict)   # prefixes of embedding / final_norm / head
    tensor_aliases: Any = None     # callable: checkpoint name -> canonical name (or None)
    unused_tensors: tuple[str, ...] = ()   # canonical names a checkpoint of the architecture may hold that this
                                           # model has no use for (an optional tensor of a part no layer has): skipped

    def __post_init__(self):
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule[{i}] names layer {e.layer}, the model has {n}")
            c = i if e.cache is None else e.cache
            if not 0 <= c < len(self.schedule):
                raise ValueError(f"schedule[{i}] names cache entry {c}, outside the schedule")
            if not e.writes_cache and c >= i:
                raise ValueError(f"schedule[{i}] reads cache entry {c}, which has not run yet")


@dataclass
class BuildEnv:
    """What parts need at build and run time besides their own parameters."""
    device: torch.device
    dtype: torch.dtype                 # activation / matrix dtype: float32 or bfloat16
    workspace: Any = None              # engine.workspace.Workspace
    # A norm split between two products (ops.kernels.SplitNorm), handed from a block to a part for
    # one call.  A part that sets `split_norm = True` takes `split_in` (its input rows are then
    # the split's values, and its first product scales by the split) and `split_out` (its last
    # adding product leaves the split's values and sums); the others never look at them.
    split_in: Any = None
    split_out: Any = None
    next_block_norm: Any = None        # the norm that reads the residual after this block (set by the model)

    def take_split_in(self):
        s, self.split_in = self.split_in, None
        return s

    def take_split_out(self):
        s, self.split_out = self.split_out, None
        return s

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32


class Part:
    split_norm = False     # True: forward() honours env.split_in / env.split_out (see BuildEnv)

    def split_reader_weight(self):
        """For parts with `split_norm`: the weight [N, K] of the product that reads the part's input
        (the one that gets `scale=`), so that a block offers a split only where that product can
        take it.  None: the block offers it only for steps the weight stream runs."""
        return None

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: dict[str, torch.Tensor], env: BuildEnv) -> None:
        pass

    # ---- what a row costs, for reports (a roofline needs no knowledge of the architecture) ----
    def flops_per_row(self) -> int:
        """Floating-point operations of one row through the part's matrix products (2 per multiply-add)."""
        n = 0
        for spec in self.tensors().values():
            if spec.role == MATRIX:
                k = 1
                for d in spec.shape:
                    k *= int(d)
                n += 2 * k
        return n

    def unread_weight_bytes(self, rows: int) -> float:
        """Bytes of the part's weights that a step of `rows` rows is expected NOT to read (experts nobody chose)."""
        return 0.0


class Mixer(Part):
    def cache_spec(self) -> KVSpec | StateSpec | None:
        return None

    def forward(self, h, out, accumulate, batch, cache, env) -> None:
        raise NotImplementedError

    def flops_per_query_key(self) -> int:
        """Operations per (query row, cached position) pair, for mixers that look back over the sequence."""
        return 0


class FeedForward(Part):
    def forward(self, h, out, accumulate, batch, env) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions.  A part either names a rotation the
    mixer's fused kernel can apply (`fused_rotary`), or encodes q and k itself (`apply`); the
    mixer asks in this order and knows nothing else about the encoding."""

    def fused_rotary(self):
        """(inverse frequencies [rope_dim/2] float or None for no rotation, rope_dim, split-half
        pairing?) when the encoding is a rotation by position * frequency; None otherwise."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor | None, row_pos: torch.Tensor) -> None:
        """Encodes in place: q [rows, heads, head_dim], k [rows, kv heads, head_dim] (None when the
        layer stores no keys), row_pos int32 [rows] absolute positions."""
        raise NotImplementedError
