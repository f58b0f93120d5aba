"""Python face of the CUDA kernels: checks shapes and types, then calls the C entry points.

Every function launches on torch's current stream and returns at once.  Tensors are only
containers here: no torch arithmetic runs on the product path.  A call on a machine without
the built library, or with tensors that are not on a CUDA device, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

from . import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_lib = None
_timer = None      # a KernelTimer while one is active


def lib():
    global _lib
    if _lib is None:
        _lib = _build.load()
        _declare(_lib)
    return _lib if _timer is None else _timer.proxy


class KernelTimer:
    """Device time of every kernel entry point called while it is active, by name.

        with kernels.KernelTimer() as t:
            engine.step(...)
        t.summary()  ->  {entry point: (calls, milliseconds)}, longest first

    Every call is bracketed by two CUDA events on the launching stream, as the reference's per-kernel
    timer does behind LE_EVT (src/gpu/dense.rs:47-51, :348-388).  An event between two kernels keeps
    the second from starting under the first (programmatic dependent launch), so the times are
    those of kernels run one after the other: they add up to more than the step takes, and their
    shares are what to read.  `head_start_ms` > 0 first occupies the device for about that long, so
    that the host has queued the step's launches before the device reaches them and no event pair
    contains the host's time between two launches.  Not for captured graphs or timed runs."""

    def __init__(self, head_start_ms: float = 0.0):
        self.head_start_ms = float(head_start_ms)
        self.events: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        real = lib()
        timer = self

        class _Proxy:
            def __getattr__(self, name):
                fn = getattr(real, name)
                if not name.startswith("leb_") or fn.argtypes is None or not fn.argtypes or fn.argtypes[-1] is not c_void_p:
                    return fn          # queries and settings: no stream, nothing to time

                def timed(*args):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    rc = fn(*args)
                    b.record()
                    timer.events.append((name, a, b))
                    return rc
                return timed
        self.proxy = _Proxy()

    def __enter__(self):
        global _timer
        if _timer is not None:
            raise KernelError("a KernelTimer is already active")
        if self.head_start_ms > 0:
            torch.cuda._sleep(int(self.head_start_ms * 1.5e6))      # cycles, at some 1.5 GHz
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None
        torch.cuda.synchronize()
        return False

    def summary(self) -> dict[str, tuple[int, float]]:
        acc: dict[str, list] = {}
        for name, a, b in self.events:
            e = acc.setdefault(name, [0, 0.0])
            e[0] += 1
            e[1] += a.elapsed_time(b)
        return {k: (v[0], v[1]) for k, v in sorted(acc.items(), key=lambda kv: -kv[1][1])}


def _declare(L) -> None:
    P, I, F, S = c_void_p, c_int, c_float, c_size_t
    sig = {
        "leb_embed": [P, P, I, P, I, I, I, P],
        "leb_rmsnorm": [P, I, P, P, P, I, I, F, I, P],
        "leb_swiglu": [P, I, P, I, I, I, P],
        "leb_gather_rows": [P, P, I, P, I, I, I, P],
        "leb_add": [P, P, S, P],
        "leb_shortconv": [P, P, I, P, P, P, P, P, P, P, I, I, I, I, P],
        "leb_qk_rope_store": [P, P, I, P, P, I, P, P, I, P, I, P, P, P, P, P, F, P, I, I, I, I, I, I, I, P],
        "leb_attention": [P, P, P, P, P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P],
        "leb_gemm_f32": [P, P, P, I, I, I, I, I, I, P, I, S, P],
        "leb_gemm_bf16_small": [P, I, P, P, I, I, I, I, I, I, P, I, S, I, P],
        "leb_gemm_bf16_stream": [P, I, P, P, I, I, I, I, I, I, P, I, I, F, P, P, P, P],
        "leb_gemm_bf16_stream_grouped": [P, I, P, P, I, I, I, I, I, I, P, I, S, P],
        "leb_gemm_bf16_stream_conv": [P, P, P, I, I, I, I, I, P, P, P, P, P, I, P, I, I, F, P],
        "leb_gemm_bf16_tc_grouped": [P, I, P, P, I, I, I, I, I, I, P, I, P, P],
        "leb_gemm_bf16_tc2": [P, I, P, P, I, I, I, I, I, I, P, P],
        "leb_moe_router": [P, P, P, I, P, P, I, I, I, I, I, F, P],
        "leb_moe_align": [P, P, P, P, I, I, P],
        "leb_moe_combine": [P, P, P, P, I, I, I, I, P],
        "leb_penalties": [P, P, P, I, I, I, F, F, P],
        "leb_argmax": [P, P, I, I, P],
        "leb_sample": [P, P, P, I, I, I, F, F, F, P],
        "leb_advance": [P, P, P, P, P, I, P],
        "leb_feed_tokens": [P, P, P, I, P],
        "leb_penalties_slots": [P, P, P, P, I, I, I, F, F, P],
        "leb_history_append": [P, P, P, P, I, I, P],
        "leb_attention_decode_supported": [I, I, I, I],
        "leb_attention_decode": [P, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "leb_attention_merge": [P, P, I, P, I, I, I, I, I, P],
        "leb_attention_decode_prep_supported": [I, I, I, I, I, I],
        "leb_attention_decode_prep": [P, P, P, I, P, P, I, P, P, P, I, P, P, P, P, P, F, P, I, I, P, I, I, I, I, I, I, I, F, I, P],
        "leb_attention_prefill_supported": [I, I, I, I],
        "leb_attention_prefill_tc_supported": [I, I, I, I],
        "leb_attention_prefill_tc": [P, P, I, I, P, P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P],
        "leb_attention_prefill": [P, P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "leb_gemm_bf16_skinny_slices": [I, I],
        "leb_gemm_bf16_skinny_supported": [P, P, I, I, I],
        "leb_gemm_bf16_skinny": [P, I, P, P, I, I, I, I, I, I, P, I, P, I, I, F, P, P, P, P, P],
        "leb_gemm_bf16_skinny_conv": [P, P, P, I, I, I, I, I, P, P, P, P, P, I, P, I, P, I, I, F, P, P],
        "leb_gemm_bf16_tc_supported": [P, P, I, I],
        "leb_gemm_bf16_tc": [P, I, P, P, I, I, I, I, I, I, P, P],
        "leb_selftest_bounded_wait": [P, I, I, P],
        "leb_gemm_bf16_tc_slices": [I, I, I],
        "leb_gemm_bf16_tc_sliced": [P, I, P, P, I, I, I, I, I, I, P, I, P, P],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = c_int
    L.leb_launch_count.restype = ctypes.c_longlong
    L.leb_launch_count.argtypes = []
    L.leb_sm_count.restype = c_int
    L.leb_sm_count.argtypes = []
    for name, args in _OPTIONAL.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = c_int


# entry points that later files add; declared when present
_OPTIONAL: dict[str, list] = {}


class KernelError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().leb_last_error().decode())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (torch's raw accessor where it has one: a launch from Python
    costs some 25 us otherwise, most of it the Stream object)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _cuda(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}, the kernels run on CUDA only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")


def _dt(t: torch.Tensor, name: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{name}: unsupported dtype {t.dtype}") from None


# ----------------------------------------------------------------------------------------------
def embed(x: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor) -> None:
    """x[m] = table[tokens[m]] as float."""
    _cuda(x, "embed.x", torch.float32)
    _cuda(table, "embed.table")
    _cuda(tokens, "embed.tokens", torch.int32)
    M, D = x.shape
    V = table.shape[0]
    assert table.shape[1] == D and tokens.numel() >= M
    _check(lib().leb_embed(_ptr(x), _ptr(table), _dt(table, "embed.table"), _ptr(tokens), M, D, V, _stream()))


def rmsnorm(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float,
            rows: torch.Tensor | None = None, add: bool = False) -> None:
    """out = x * rsqrt(mean(x^2) + eps) * w  (out += ... when add).  x is float."""
    _cuda(out, "rmsnorm.out")
    _cuda(x, "rmsnorm.x", torch.float32)
    _cuda(w, "rmsnorm.w", torch.float32)
    M, D = out.shape
    assert x.shape[1] == D and w.numel() == D
    if rows is not None:
        _cuda(rows, "rmsnorm.rows", torch.int32)
        assert rows.numel() >= M
    else:
        assert x.shape[0] >= M
    _check(lib().leb_rmsnorm(_ptr(out), _dt(out, "rmsnorm.out"), _ptr(x), _ptr(w), _ptr(rows), M, D,
                             float(eps), 1 if add else 0, _stream()))


def swiglu(out: torch.Tensor, gu: torch.Tensor) -> None:
    """out[m, j] = silu(gu[m, j]) * gu[m, F + j]."""
    _cuda(out, "swiglu.out")
    _cuda(gu, "swiglu.gu")
    M, Fd = out.shape
    assert gu.shape == (M, 2 * Fd)
    _check(lib().leb_swiglu(_ptr(out), _dt(out, "swiglu.out"), _ptr(gu), _dt(gu, "swiglu.gu"), M, Fd, _stream()))


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor, div: int = 1) -> None:
    """out[p] = src[rows[p] // div]."""
    _cuda(out, "gather_rows.out")
    _cuda(src, "gather_rows.src", out.dtype)
    _cuda(rows, "gather_rows.rows", torch.int32)
    P_, D = out.shape
    assert src.shape[1] == D and rows.numel() >= P_
    _check(lib().leb_gather_rows(_ptr(out), _ptr(src), _dt(out, "gather_rows"), _ptr(rows), div, P_, D, _stream()))


def add_(x: torch.Tensor, y: torch.Tensor) -> None:
    _cuda(x, "add.x", torch.float32)
    _cuda(y, "add.y", torch.float32)
    assert x.numel() == y.numel()
    _check(lib().leb_add(_ptr(x), _ptr(y), x.numel(), _stream()))


def shortconv(y: torch.Tensor, bcx: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
              state: torch.Tensor, batch, Lc: int) -> None:
    """Gated short convolution over the step's rows; updates `state` [slots, D, Lc-1] (float)."""
    _cuda(y, "shortconv.y")
    _cuda(bcx, "shortconv.bcx", y.dtype)
    _cuda(w, "shortconv.w", torch.float32)
    _cuda(state, "shortconv.state", torch.float32)
    M, D = y.shape
    assert bcx.shape == (M, 3 * D) and w.numel() == D * Lc
    assert state.shape[1:] == (D, Lc - 1)
    if bias is not None:
        _cuda(bias, "shortconv.bias", torch.float32)
    single = batch.max_qlen == 1 and M == batch.n_seqs     # decode: the one-launch form
    _check(lib().leb_shortconv(_ptr(y), _ptr(bcx), _dt(y, "shortconv"), _ptr(w), _ptr(bias), _ptr(state),
                               _ptr(batch.row_seq), _ptr(batch.seq_slot), _ptr(batch.seq_qstart),
                               None if single else _ptr(batch.seq_qlen), M, batch.n_seqs, D, Lc, _stream()))


CONV_FUSED_MAX_LC = 5    # conv lengths the fused decode kernel takes


def shortconv_decode_fused(y: torch.Tensor, h: torch.Tensor, w_in: torch.Tensor, w: torch.Tensor,
                           bias: torch.Tensor | None, state: torch.Tensor, batch, Lc: int,
                           scale: "SplitNorm | None" = None) -> bool:
    """The conv mixer's in_proj and convolution of a decode step without a kernel of the
    convolution's own: y = conv(h . w_in^T), state updated.  Up to SMALL_M sequences it is the epilogue
    of the weight stream (one launch); up to SKINNY_M sequences the second kernel of the sliced
    tcgen05 product.  False (nothing done) when the step is not one of so many sequences with one
    bfloat16 row each, or the sizes are not the kernels'."""
    M, D = y.shape
    K = h.shape[1]
    if not (h.dtype == torch.bfloat16 and y.dtype == torch.bfloat16 and 0 < M <= SKINNY_M
            and batch.max_qlen == 1 and M == batch.n_seqs and 2 <= Lc <= CONV_FUSED_MAX_LC and K % 8 == 0
            and h.stride(0) % 8 == 0 and h.stride(1) == 1 and y.stride(1) == 1):
        return False
    if M > SMALL_M:
        L = lib()
        slices = L.leb_gemm_bf16_skinny_slices(3 * D, K)
        if slices < 2 or 3 * D >= SKINNY_MAX_N or not _tma_ok(h, w_in, K) or not w_in.is_contiguous():
            return False
        _cuda(w_in, "shortconv.w_in", torch.bfloat16)
        _cuda(w, "shortconv.w", torch.float32)
        _cuda(state, "shortconv.state", torch.float32)
        assert w_in.shape == (3 * D, K) and w.numel() == D * Lc and state.shape[1:] == (D, Lc - 1)
        if bias is not None:
            _cuda(bias, "shortconv.bias", torch.float32)
        ssq, parts, d_in, eps = _scale_args(scale, M, K)
        part = _skinny_workspace(h.device, slices * M * 3 * D)
        _check(L.leb_gemm_bf16_skinny_conv(_ptr(y), _ptr(h), _ptr(w_in), M, D, K, h.stride(0), y.stride(0), _ptr(w),
                                           _ptr(bias), _ptr(state), _ptr(batch.row_seq), _ptr(batch.seq_slot), Lc,
                                           _ptr(part), slices, ssq, parts, d_in, eps, _ptr(_status_word(h.device)),
                                           _stream()))
        return True
    _cuda(h, "shortconv.h", contiguous=False)
    _cuda(w_in, "shortconv.w_in", torch.bfloat16)
    _cuda(w, "shortconv.w", torch.float32)
    _cuda(state, "shortconv.state", torch.float32)
    assert w_in.shape == (3 * D, K) and w.numel() == D * Lc and state.shape[1:] == (D, Lc - 1)
    if bias is not None:
        _cuda(bias, "shortconv.bias", torch.float32)
    ssq, parts, d_in, eps = _scale_args(scale, M, K)
    _check(lib().leb_gemm_bf16_stream_conv(_ptr(y), _ptr(h), _ptr(w_in), M, D, K, h.stride(0), y.stride(0), _ptr(w),
                                           _ptr(bias), _ptr(state), _ptr(batch.row_seq), _ptr(batch.seq_slot), Lc,
                                           ssq, parts, d_in, eps, _stream()))
    return True


def qk_rope_store(q_out: torch.Tensor, q_in: torch.Tensor, k_in: torch.Tensor | None,
                  v_in: torch.Tensor | None, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
                  block_table: torch.Tensor, batch, q_norm_w, k_norm_w, eps: float,
                  inv_freq: torch.Tensor | None, rope_dim: int, neox: bool, nh: int, nkv: int, hd: int,
                  page_size: int) -> None:
    """Per-head norm and rotation of q and k; k and v go to the paged cache, q to q_out.

    q_in/k_in/v_in may be column slices of one fused projection (row stride = its width).
    """
    _cuda(q_out, "qk_rope_store.q_out")
    _cuda(q_in, "qk_rope_store.q_in", q_out.dtype, contiguous=False)
    M = q_out.shape[0]
    assert q_in.stride(-1) == 1 and q_in.shape == (M, nh * hd)
    q_stride = q_in.stride(0)
    kv_stride = 0
    if k_in is not None:
        _cuda(k_in, "qk_rope_store.k_in", q_out.dtype, contiguous=False)
        _cuda(v_in, "qk_rope_store.v_in", q_out.dtype, contiguous=False)
        assert k_in.shape == (M, nkv * hd) and v_in.shape == (M, nkv * hd)
        assert k_in.stride(0) == v_in.stride(0) and k_in.stride(-1) == 1 and v_in.stride(-1) == 1
        kv_stride = k_in.stride(0)
        _cuda(k_pool, "qk_rope_store.k_pool", q_out.dtype)
        _cuda(v_pool, "qk_rope_store.v_pool", q_out.dtype)
        assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, hd, page_size)
    _cuda(block_table, "qk_rope_store.block_table", torch.int32)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("inv_freq", inv_freq)):
        if t is not None:
            _cuda(t, f"qk_rope_store.{name}", torch.float32)
    if inv_freq is not None:
        assert inv_freq.numel() == rope_dim // 2
    _check(lib().leb_qk_rope_store(
        _ptr(q_out), _ptr(q_in), q_stride, _ptr(k_in), _ptr(v_in), kv_stride, _ptr(k_pool), _ptr(v_pool),
        _dt(q_out, "qk_rope_store"), _ptr(block_table), block_table.shape[1], _ptr(batch.row_seq),
        _ptr(batch.row_pos), _ptr(batch.seq_slot), _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
        _ptr(inv_freq), rope_dim, 1 if neox else 0, M, nh, nkv, hd, page_size, _stream()))


_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """SMs of the current device, asked once per device."""
    d = torch.cuda.current_device()
    n = _sm_counts.get(d)
    if n is None:
        n = _sm_counts[d] = max(1, int(lib().leb_sm_count()))
    return n


def attention_splits(batch, nkv: int, G: int, sm_count: int | None = None, hd: int = 64) -> int:
    """How many blocks share one sequence's key range in a decode step (1 for prompts).

    Measured on B200 (head size 64, 8 kv heads, times with the merge of the splits): a block has a
    fixed cost of some microseconds, so a split must leave a block 256 positions or more (128 when
    there are so few blocks that the step waits on each one's latency); the blocks
    of a launch should all run at once (three per SM at head size 64: with 8 sequences of 4,096
    positions 6 splits, 384 blocks, take 14.7 us a layer and 7 splits, 448 blocks, 18.8 us); and
    when the sequences alone fill the GPU twice over, splitting pays only for long ranges (64
    sequences of 640 positions: 20.3 us unsplit, 27.4 us in 4 splits; of 4,096 positions: 110 us
    unsplit, 89 us in 4 splits).
    """
    if batch.max_qlen != 1:
        return 1
    if sm_count is None:
        sm_count = globals()["sm_count"]()
    kv = max(int(batch.max_kvlen), 1)
    per = max(batch.n_seqs * nkv * ((G + 15) // 16), 1)
    stage_bytes = 2 * 32 * hd * 2 * (3 if hd <= 32 else 2) * 4          # a block's rings: 4 warps, keys and values
    slots = sm_count * max(1, min(3, (227 * 1024) // stage_bytes))      # blocks that run at once
    if per >= 2 * sm_count:
        return 1 if kv < 2048 else min(4, kv // 1024)
    least = 128 if per * 8 <= sm_count else 256       # one or two sequences: latency counts, shorter blocks pay
    return max(1, min(slots // per, kv // least, 32))


TC_ATTENTION_MIN_ROWS = 8   # longest row count of a sequence from which prompts go to the tcgen05 attention


class RawQKV:
    """A decode step's q, k and v as the projection left them, for the decode attention kernel that
    norms, rotates and stores them itself (`decode_attention_takes_raw` says when it can)."""

    def __init__(self, q_in, k_in, v_in, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, neox):
        self.q_in, self.k_in, self.v_in = q_in, k_in, v_in
        self.q_norm_w, self.k_norm_w, self.eps = q_norm_w, k_norm_w, float(eps)
        self.inv_freq, self.rope_dim, self.neox = inv_freq, int(rope_dim), bool(neox)


def decode_attention_takes_raw(dtype: torch.dtype, batch, M: int, nh: int, nkv: int, hd: int, page_size: int,
                               inv_freq, rope_dim: int, neox: bool) -> bool:
    """Whether `attention(..., raw=...)` will do the per-head norm, the rotation and the cache write
    of this step itself: a bfloat16 decode step (one row per sequence) whose sizes the tensor-core
    decode kernel takes, with a split-half rotation over the whole head."""
    return bool(dtype == torch.bfloat16 and batch.max_qlen == 1 and M == batch.n_seqs and inv_freq is not None
                and lib().leb_attention_decode_prep_supported(nh, nkv, hd, page_size, int(rope_dim), 1 if neox else 0))


def attention(out: torch.Tensor, q: torch.Tensor | None, k_pool: torch.Tensor, v_pool: torch.Tensor,
              block_table: torch.Tensor, batch, nh: int, nkv: int, hd: int, page_size: int,
              window: int, scale: float, gate: torch.Tensor | None = None,
              n_splits: int = 1, scratch: torch.Tensor | None = None, raw: RawQKV | None = None) -> None:
    """Causal attention of the step's rows over the paged cache (which already holds their keys;
    with `raw`, the kernel puts the step's keys and values there itself and `q` is not used)."""
    _cuda(out, "attention.out")
    if raw is not None:
        return _attention_decode_raw(out, raw, k_pool, v_pool, block_table, batch, nh, nkv, hd, page_size, window,
                                     scale, gate, n_splits, scratch)
    _cuda(q, "attention.q", out.dtype)
    _cuda(k_pool, "attention.k_pool", out.dtype)
    _cuda(v_pool, "attention.v_pool", out.dtype)
    _cuda(block_table, "attention.block_table", torch.int32)
    M = out.shape[0]
    assert out.shape == (M, nh * hd) and q.shape == (M, nh * hd)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, hd, page_size)
    gate_stride = 0
    if gate is not None:
        _cuda(gate, "attention.gate", out.dtype, contiguous=False)
        assert gate.shape == (M, nh) and gate.stride(-1) == 1
        gate_stride = gate.stride(0)
    if n_splits > 1:
        need = M * nh * n_splits * (hd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention: {n_splits} splits need {need} floats of scratch")
        _cuda(scratch, "attention.scratch", torch.float32)
    L = lib()
    if (out.dtype == torch.bfloat16 and batch.max_qlen == 1 and M == batch.n_seqs
            and L.leb_attention_decode_supported(nh, nkv, hd, page_size)):
        # one row per sequence: the tensor-core decode kernel, then the merge of its splits
        _check(L.leb_attention_decode(
            _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
            block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
            _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale), n_splits,
            _stream()))
        if n_splits > 1:
            _check(L.leb_attention_merge(_ptr(out), _ptr(scratch), BF16, _ptr(gate), gate_stride, M, nh, hd,
                                         n_splits, _stream()))
        return
    if (out.dtype == torch.bfloat16 and n_splits == 1 and batch.max_qlen >= TC_ATTENTION_MIN_ROWS
            and q.stride(0) % 8 == 0 and L.leb_attention_prefill_tc_supported(nh, nkv, hd, page_size)):
        # prompts: tcgen05 tiles of 128 (position, head) rows, pages brought in by TMA
        _check(L.leb_attention_prefill_tc(
            _ptr(out), _ptr(q), q.stride(0), M, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
            block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
            _ptr(batch.seq_qlen), _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
            batch.max_qlen, _ptr(_status_word(out.device)), _stream()))
        return
    if (out.dtype == torch.bfloat16 and n_splits == 1
            and L.leb_attention_prefill_supported(nh, nkv, hd, page_size)):
        # rows of prompts (or decode without splits): the tensor-core kernel over (position, head) rows
        _check(L.leb_attention_prefill(
            _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
            _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart), _ptr(batch.seq_qlen),
            _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
            batch.max_qlen, _stream()))
        return
    _check(L.leb_attention(
        _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _dt(out, "attention"),
        _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
        _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(gate), gate_stride, M, batch.n_seqs, nh, nkv,
        hd, page_size, window, float(scale), batch.max_qlen, n_splits, _stream()))


def _attention_decode_raw(out, raw: RawQKV, k_pool, v_pool, block_table, batch, nh, nkv, hd, page_size, window,
                          scale, gate, n_splits, scratch) -> None:
    M = out.shape[0]
    if not decode_attention_takes_raw(out.dtype, batch, M, nh, nkv, hd, page_size, raw.inv_freq, raw.rope_dim, raw.neox):
        raise KernelError("attention: this step's q, k and v must be normed, rotated and stored before the call")
    _cuda(k_pool, "attention.k_pool", out.dtype)
    _cuda(v_pool, "attention.v_pool", out.dtype)
    _cuda(block_table, "attention.block_table", torch.int32)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, hd, page_size)
    _cuda(raw.q_in, "attention.q_in", out.dtype, contiguous=False)
    assert raw.q_in.shape == (M, nh * hd) and raw.q_in.stride(-1) == 1 and out.shape == (M, nh * hd)
    kv_stride = 0
    if raw.k_in is not None:
        _cuda(raw.k_in, "attention.k_in", out.dtype, contiguous=False)
        _cuda(raw.v_in, "attention.v_in", out.dtype, contiguous=False)
        assert raw.k_in.shape == (M, nkv * hd) and raw.v_in.shape == (M, nkv * hd)
        assert raw.k_in.stride(0) == raw.v_in.stride(0) and raw.k_in.stride(-1) == 1 and raw.v_in.stride(-1) == 1
        kv_stride = raw.k_in.stride(0)
    for name, t in (("q_norm_w", raw.q_norm_w), ("k_norm_w", raw.k_norm_w), ("inv_freq", raw.inv_freq)):
        if t is not None:
            _cuda(t, f"attention.{name}", torch.float32)
    assert raw.inv_freq.numel() == hd // 2
    gate_stride = 0
    if gate is not None:
        _cuda(gate, "attention.gate", out.dtype, contiguous=False)
        assert gate.shape == (M, nh) and gate.stride(-1) == 1
        gate_stride = gate.stride(0)
    if n_splits > 1:
        need = M * nh * n_splits * (hd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention: {n_splits} splits need {need} floats of scratch")
    L = lib()
    _check(L.leb_attention_decode_prep(
        _ptr(out), _ptr(scratch), _ptr(raw.q_in), raw.q_in.stride(0), _ptr(raw.k_in), _ptr(raw.v_in), kv_stride,
        _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
        _ptr(batch.seq_qstart), _ptr(raw.q_norm_w), _ptr(raw.k_norm_w), raw.eps, _ptr(raw.inv_freq), raw.rope_dim,
        1 if raw.neox else 0, _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
        n_splits, _stream()))
    if n_splits > 1:
        _check(L.leb_attention_merge(_ptr(out), _ptr(scratch), BF16, _ptr(gate), gate_stride, M, nh, hd, n_splits, _stream()))


# ----------------------------------------------------------------------------------------------
STORE, ACCUMULATE, SWIGLU = 0, 1, 2
SMALL_M = 16  # rows up to which the weight-streaming kernel is used; above, tcgen05 tiles


# Forming the norm inside a product (in the consumer's prologue, or in the tail of the product
# before it) was built and measured slower than the separate norm kernel each time: with
# programmatic dependent launch the small norm kernel between two products is the window in which
# the next product starts up and fetches its first weights.  So the norm stays a kernel of its own.


class SplitNorm:
    """An RMSNorm split between the product before it and the product after it (decode steps).

    `values` [M, D] is bfloat16(x * weight) and `ssq` [M, ceil(D/16)] holds partial sums of x^2,
    both left by the product that added into the residual x (`linear(..., emit=...)`); the product
    that takes `values` as its input multiplies its float sums by rsqrt(sum(ssq) / D + eps)
    (`linear(..., scale=...)`).  The products of steps of up to SKINNY_M rows do both (the weight
    stream up to SMALL_M rows, the sliced tcgen05 product above, in its second kernel);
    `split_norm_ok` says whether a step qualifies."""

    def __init__(self, values: torch.Tensor, ssq: torch.Tensor, weight: torch.Tensor, eps: float):
        self.values, self.ssq, self.weight, self.eps = values, ssq, weight, float(eps)
        self.filled = False      # set by the product that wrote values and ssq


def split_norm_ok(M: int, dtype: torch.dtype, reader_weight: torch.Tensor | None = None) -> bool:
    """Whether a step of M rows may split a norm in front of a product with `reader_weight`
    [N, K].  Once the norm is split its input exists only as bfloat16(x * g), so the product that
    reads it must be one that can scale its rows: the weight stream (up to SMALL_M rows) or the
    sliced tcgen05 product (up to SKINNY_M rows, N below its limit, operands TMA can fetch).  A
    reader that does not say what it multiplies with gets the split only where the weight stream
    runs."""
    if dtype != torch.bfloat16 or not 0 < M <= SKINNY_M:
        return False
    if reader_weight is None:
        return M <= SMALL_M
    if reader_weight.dim() != 2 or reader_weight.dtype != torch.bfloat16:
        return False
    N, K = reader_weight.shape
    if K % 8 != 0 or reader_weight.data_ptr() % 16 != 0:
        return False
    return M <= SMALL_M or N < SKINNY_MAX_N


def _scale_args(scale: "SplitNorm | None", M: int, K: int):
    if scale is None:
        return None, 0, 0, 0.0
    assert scale.filled and scale.values.shape == (M, K) and scale.ssq.shape[0] >= M
    return _ptr(scale.ssq), scale.ssq.shape[1], K, scale.eps


def linear(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE,
           group_offsets: torch.Tensor | None = None, rows_hint: int = 0, streaming: bool = False,
           scale: SplitNorm | None = None, emit: SplitNorm | None = None) -> None:
    """out (+)= x . w^T  with w [N, K] (or [E, N, K] with group_offsets [E+1] over the rows).

    float32 operands run on the CUDA cores in true 32-bit; bfloat16 operands on the tensor
    cores with float accumulation.  `epilogue`: STORE, ACCUMULATE (out is the float residual)
    or SWIGLU (w holds gate and up rows interleaved in blocks of 16; out has N/2 columns).
    Up to SMALL_M rows bfloat16 products stream W through shared memory with asynchronous copies;
    with more rows they go to the tcgen05 kernels: up to SKINNY_M rows with W as the wide operand
    and K cut into slices (a second kernel adds them up), above that 128 x BN tiles (K cut as well
    where a few hundred rows and a long K leave most SMs without a tile), from PAIRS_MIN_ROWS rows
    and large matrices 256 x 256 tiles on pairs of SMs; `streaming` asks for the register-fed
    weight-streaming kernel (the one that also serves grouped products) whatever the row count.
    """
    _cuda(x, "linear.x", contiguous=False)
    _cuda(w, "linear.w", x.dtype)
    _cuda(out, "linear.out", contiguous=False)
    M, K = x.shape
    assert x.stride(1) == 1 and out.stride(1) == 1
    lda, ldc = x.stride(0), out.stride(0)
    if group_offsets is not None:
        _cuda(group_offsets, "linear.group_offsets", torch.int32)
        E, N, Kw = w.shape
        assert group_offsets.numel() == E + 1
        stride = N * Kw
    else:
        N, Kw = w.shape
        E, stride = 1, 0
    assert Kw == K, f"linear: x has {K} columns, w has {Kw}"
    n_out = N // 2 if epilogue == SWIGLU else N
    assert out.shape == (M, n_out), f"linear: out is {tuple(out.shape)}, expected {(M, n_out)}"
    if M == 0:
        return
    L = lib()
    if x.dtype == torch.float32:
        if epilogue == SWIGLU:
            raise KernelError("linear: the float path keeps SwiGLU as its own kernel")
        if out.dtype != torch.float32:
            raise KernelError("linear: float operands need a float result")
        _check(L.leb_gemm_f32(_ptr(out), _ptr(x), _ptr(w), M, N, K, lda, ldc, epilogue, _ptr(group_offsets),
                              E, stride, _stream()))
        return
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported operand dtype {x.dtype}")
    hint = rows_hint if rows_hint > 0 else M
    tc = _OPTIONAL_TC[0]
    ssq, parts, d_in, eps = _scale_args(scale, M, K)
    ev = eg = es = None
    if emit is not None and group_offsets is None and not streaming and M <= SKINNY_M:
        assert epilogue == ACCUMULATE and emit.values.shape == (M, N) and emit.ssq.shape == (M, -(-N // 16))
        assert emit.values.is_contiguous() and emit.ssq.is_contiguous() and emit.weight.numel() == N
        ev, eg, es = _ptr(emit.values), _ptr(emit.weight), _ptr(emit.ssq)
    if not streaming and group_offsets is None and M <= SMALL_M:
        # the decode step: W streamed through rings of asynchronous copies in shared memory
        _check(L.leb_gemm_bf16_stream(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                      epilogue, ssq, parts, d_in, eps, ev, eg, es, _stream()))
        if ev is not None:
            emit.filled = True
        return
    # few dozen rows: W as the wide operand with K sliced over blocks, unless N alone already gives
    # every SM several tiles (the output head), where the persistent kernel streams W better
    if (not streaming and group_offsets is None and SMALL_M < M <= SKINNY_M and N < SKINNY_MAX_N
            and linear_skinny(out, x, w, epilogue, norm_args=(ssq, parts, d_in, eps, ev, eg, es))):
        if ev is not None:
            emit.filled = True
        return
    if scale is not None:
        raise KernelError("linear: a split norm goes with the decode products of up to SKINNY_M rows only")
    if (not streaming and group_offsets is None and M >= PAIRS_MIN_ROWS and (N >= 4096 or K >= 4096)
            and linear_tc2(out, x, w, epilogue)):
        return      # many rows and a large weight matrix: 256 x 256 tiles on pairs of SMs
    if tc is not None and not streaming and group_offsets is None and M > SMALL_M and tc(out, x, w, epilogue):
        return
    if (not streaming and group_offsets is not None and E <= 256 and M > 16 * E and w.is_contiguous()
            and _tma_ok(x, w, K)):
        # experts with many rows each (prompts): tcgen05 tiles over the experts' row ranges
        _check(L.leb_gemm_bf16_tc_grouped(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                          epilogue, _ptr(group_offsets), E, _ptr(_status_word(x.device)), _stream()))
        return
    if not streaming and group_offsets is not None and E <= 256 and M <= 16 * E:
        # experts with a few rows each (decode steps): the ring-fed stream over the experts that have rows
        _check(L.leb_gemm_bf16_stream_grouped(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                              epilogue, _ptr(group_offsets), E, stride, _stream()))
        return
    _check(L.leb_gemm_bf16_small(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                 epilogue, _ptr(group_offsets), E, stride, hint, _stream()))


# set by ops.tc_gemm when the tensor-core (tcgen05) kernel is present
_OPTIONAL_TC: list = [None]


# ----------------------------------------------------------------------------------------------
def moe_router(topk_ids: torch.Tensor, topk_w: torch.Tensor, h: torch.Tensor, wr: torch.Tensor,
               bias: torch.Tensor | None, norm_topk: bool, scaling: float) -> None:
    _cuda(topk_ids, "moe_router.topk_ids", torch.int32)
    _cuda(topk_w, "moe_router.topk_w", torch.float32)
    _cuda(h, "moe_router.h")
    _cuda(wr, "moe_router.wr", torch.float32)
    M, k = topk_ids.shape
    E, D = wr.shape
    assert h.shape == (M, D) and topk_w.shape == (M, k)
    if bias is not None:
        _cuda(bias, "moe_router.bias", torch.float32)
        assert bias.numel() == E
    _check(lib().leb_moe_router(_ptr(topk_ids), _ptr(topk_w), _ptr(h), _dt(h, "moe_router.h"), _ptr(wr),
                                _ptr(bias), M, D, E, k, 1 if norm_topk else 0, float(scaling), _stream()))


def moe_align(offsets: torch.Tensor, sorted_pair: torch.Tensor, pair_row: torch.Tensor,
              topk_ids: torch.Tensor, E: int) -> None:
    for n, t in (("offsets", offsets), ("sorted_pair", sorted_pair), ("pair_row", pair_row),
                 ("topk_ids", topk_ids)):
        _cuda(t, f"moe_align.{n}", torch.int32)
    P_ = topk_ids.numel()
    assert offsets.numel() >= E + 1 and sorted_pair.numel() >= P_ and pair_row.numel() >= P_
    _check(lib().leb_moe_align(_ptr(offsets), _ptr(sorted_pair), _ptr(pair_row), _ptr(topk_ids), P_, E, _stream()))


def moe_combine(x: torch.Tensor, ys: torch.Tensor, pair_row: torch.Tensor, topk_w: torch.Tensor,
                accumulate: bool) -> None:
    _cuda(x, "moe_combine.x", torch.float32)
    _cuda(ys, "moe_combine.ys", torch.float32)
    _cuda(pair_row, "moe_combine.pair_row", torch.int32)
    _cuda(topk_w, "moe_combine.topk_w", torch.float32)
    M, D = x.shape
    k = topk_w.shape[1]
    assert ys.shape[1] == D and ys.shape[0] >= M * k and topk_w.shape[0] == M
    _check(lib().leb_moe_combine(_ptr(x), _ptr(ys), _ptr(pair_row), _ptr(topk_w), M, D, k,
                                 1 if accumulate else 0, _stream()))


# ----------------------------------------------------------------------------------------------
def penalties(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor,
              repeat_penalty: float, presence_penalty: float) -> None:
    _cuda(logits, "penalties.logits", torch.float32)
    _cuda(hist, "penalties.hist", torch.int32)
    _cuda(hist_len, "penalties.hist_len", torch.int32)
    n, V = logits.shape
    assert hist.shape[0] >= n
    _check(lib().leb_penalties(_ptr(logits), _ptr(hist), _ptr(hist_len), hist.shape[1], n, V,
                               float(repeat_penalty), float(presence_penalty), _stream()))


def penalties_slots(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, seq_slot: torch.Tensor,
                    repeat_penalty: float, presence_penalty: float) -> None:
    """Penalises, in place, the tokens in each sequence's ring of recent tokens (hist [slots, window])."""
    _cuda(logits, "penalties_slots.logits", torch.float32)
    _cuda(hist, "penalties_slots.hist", torch.int32)
    _cuda(hist_len, "penalties_slots.hist_len", torch.int32)
    _cuda(seq_slot, "penalties_slots.seq_slot", torch.int32)
    n, V = logits.shape
    assert seq_slot.numel() >= n and hist_len.numel() == hist.shape[0]
    _check(lib().leb_penalties_slots(_ptr(logits), _ptr(hist), _ptr(hist_len), _ptr(seq_slot), hist.shape[1], n, V,
                                     float(repeat_penalty), float(presence_penalty), _stream()))


def history_append(hist: torch.Tensor, hist_len: torch.Tensor, seq_slot: torch.Tensor, chosen: torch.Tensor, n: int) -> None:
    """The chosen token of each of the first n sequences goes into its slot's ring."""
    _cuda(hist, "history_append.hist", torch.int32)
    _cuda(hist_len, "history_append.hist_len", torch.int32)
    _cuda(chosen, "history_append.chosen", torch.int32)
    assert seq_slot.numel() >= n and chosen.numel() >= n
    _check(lib().leb_history_append(_ptr(hist), _ptr(hist_len), _ptr(seq_slot), _ptr(chosen), hist.shape[1], n, _stream()))


def argmax(out: torch.Tensor, logits: torch.Tensor) -> None:
    _cuda(out, "argmax.out", torch.int32)
    _cuda(logits, "argmax.logits", torch.float32)
    n, V = logits.shape
    assert out.numel() >= n
    _check(lib().leb_argmax(_ptr(out), _ptr(logits), n, V, _stream()))


def sample(out: torch.Tensor, logits: torch.Tensor, u01: torch.Tensor, top_k: int, temperature: float,
           top_p: float, min_p: float) -> None:
    _cuda(out, "sample.out", torch.int32)
    _cuda(logits, "sample.logits", torch.float32)
    _cuda(u01, "sample.u01", torch.float32)
    n, V = logits.shape
    assert out.numel() >= n and u01.numel() >= n
    _check(lib().leb_sample(_ptr(out), _ptr(logits), _ptr(u01), n, V, int(top_k), float(temperature),
                            float(top_p), float(min_p), _stream()))


def advance(batch, chosen: torch.Tensor) -> None:
    """The chosen tokens become the step's input and every live sequence moves one position on."""
    _cuda(chosen, "advance.chosen", torch.int32)
    _check(lib().leb_advance(_ptr(batch.tokens), _ptr(batch.row_pos), _ptr(batch.seq_pos0), _ptr(batch.seq_slot),
                             _ptr(chosen), batch.n_seqs, _stream()))


def feed_tokens(batch, chosen: torch.Tensor) -> None:
    """Sequences with batch.feed[b] >= 0 take as their token what `chosen` holds at that place."""
    _cuda(chosen, "feed_tokens.chosen", torch.int32)
    _check(lib().leb_feed_tokens(_ptr(batch.tokens), _ptr(chosen), _ptr(batch.feed), batch.n_seqs, _stream()))


def launch_count() -> int:
    """Kernels this library has launched in this process (launches inside a replayed graph are
    counted once, when the graph was captured)."""
    return int(lib().leb_launch_count())


# ---- the tcgen05 matrix product ----------------------------------------------------------------
# The status word of a device sits right in front of the buffer the chosen tokens of a step go
# to, so that the copy that brings the tokens to the host brings the word along.
RESULT_TOKENS = 8192      # chosen tokens the shared buffer holds; larger steps use a buffer of their own
_STATUS_AT = 3            # the tokens then start on a 16-byte boundary
_tc_block: dict[int, torch.Tensor] = {}
_tc_status: dict[int, torch.Tensor] = {}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _status_block(device: torch.device) -> torch.Tensor:
    i = _device_index(device)
    if i not in _tc_block:
        _tc_block[i] = torch.zeros(_STATUS_AT + 1 + RESULT_TOKENS, dtype=torch.int32, device=device)
        _tc_status[i] = _tc_block[i][_STATUS_AT:_STATUS_AT + 1]
    return _tc_block[i]


def _status_word(device: torch.device) -> torch.Tensor:
    _status_block(device)
    return _tc_status[_device_index(device)]


def result_tokens(device: torch.device) -> torch.Tensor:
    """int32 [RESULT_TOKENS] for a step's chosen tokens, directly behind the device's status word."""
    return _status_block(device)[_STATUS_AT + 1:]


def status_and_tokens(device: torch.device, n: int) -> torch.Tensor:
    """The status word followed by the first n chosen tokens: what one copy brings to the host."""
    return _status_block(device)[_STATUS_AT:_STATUS_AT + 1 + n]


def raise_on_status(value: int, device: torch.device) -> None:
    """`value`: the status word as the host read it.  Non-zero: a kernel gave up on a bounded wait
    and what the step computed is not valid; the word is cleared and KernelError raised."""
    if value != 0:
        _status_word(device).zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting (role {value}) on cuda:{_device_index(device)}; "
                          "the step's result is not valid")


def check_device_status() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for i, t in _tc_status.items():
        raise_on_status(int(t.item()), t.device)


def selftest_bounded_wait(device: torch.device, limit: int = 2000, role: int = 9) -> None:
    """Launches one block that waits, with the kernels' own bounded wait, on a barrier nobody
    arrives on; it gives up after `limit` polls and sets the device's status word to `role`."""
    _check(lib().leb_selftest_bounded_wait(_ptr(_status_word(device)), int(limit), int(role), _stream()))


def _tma_ok(x: torch.Tensor, w: torch.Tensor, K: int) -> bool:
    """What leb_gemm_bf16_tc_supported checks (16-byte aligned bases and row strides), without the call."""
    return K > 0 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def linear_tc(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE) -> bool:
    """out (+)= x . w^T on tcgen05 with TMA-fed tiles; False when the operands cannot go through TMA."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not _tma_ok(x, w, K):
        return False
    slices = L.leb_gemm_bf16_tc_slices(M, N, K) if N % 4 == 0 else 1
    if slices > 1:      # a few hundred rows and a long K: fewer tiles than SMs, so K is cut as well
        part = _skinny_workspace(x.device, slices * M * N)
        _check(L.leb_gemm_bf16_tc_sliced(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                         out.stride(0), epilogue, _ptr(part), slices,
                                         _ptr(_status_word(x.device)), _stream()))
        return True
    _check(L.leb_gemm_bf16_tc(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                              out.stride(0), epilogue, _ptr(_status_word(x.device)), _stream()))
    return True


PAIRS_MIN_ROWS = 1024   # rows from which the paired kernel is used (measured: 3-9% faster there, slower on small products)


def linear_tc2(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE) -> bool:
    """out (+)= x . w^T on pairs of SMs (tcgen05 cta_group::2, 256 x 256 tiles); False when the operands cannot go through TMA."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not _tma_ok(x, w, K):
        return False
    _check(L.leb_gemm_bf16_tc2(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                               out.stride(0), epilogue, _ptr(_status_word(x.device)), _stream()))
    return True


SKINNY_M = 128   # rows up to which W is the wide tcgen05 operand and K is sliced over blocks
SKINNY_MAX_N = 128 * 296   # from here on N alone gives every SM several tiles and the persistent kernel streams W better
_skinny_ws: dict[int, list[torch.Tensor]] = {}


def _skinny_workspace(device: torch.device, n_floats: int) -> torch.Tensor:
    """Float scratch for the K slices.  Grows by adding buffers and never frees one, so that a
    captured graph that points at an older buffer stays valid."""
    i = device.index if device.index is not None else torch.cuda.current_device()
    bufs = _skinny_ws.setdefault(i, [])
    if not bufs or bufs[-1].numel() < n_floats:
        bufs.append(torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device))
    return bufs[-1]


def linear_skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE,
                  norm_args: tuple | None = None) -> bool:
    """out (+)= x . w^T for 1..128 rows with W as the wide tcgen05 operand and K sliced over blocks.
    `norm_args`: the halves of a split norm as `linear` unpacks them (its second kernel applies them)."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not (1 <= M <= SKINNY_M and _tma_ok(x, w, K)):
        return False
    slices = L.leb_gemm_bf16_skinny_slices(N, K)
    ssq, parts, d_in, eps, ev, eg, es = norm_args or (None, 0, 0, 0.0, None, None, None)
    part = _skinny_workspace(x.device, slices * M * N) if slices > 1 else None
    _check(L.leb_gemm_bf16_skinny(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                  out.stride(0), epilogue, _ptr(part), slices, ssq, parts, d_in, eps, ev, eg, es,
                                  _ptr(_status_word(x.device)), _stream()))
    return True


_OPTIONAL_TC[0] = linear_tc
