"""The decode-attention entry point that allocates nothing.

Some hosts of this library cannot allocate device memory once they are running: everything
is in their own pool, or they sit inside another framework's captured region, or their rules
forbid cudaMalloc after start-up.  For them `leb_attention_decode_static` keeps its scratch in
an array built into the library.  This test calls it through its exported C symbol, twice in
a row (the second call finds the first one's leftovers in the array), and compares it with the
ordinary entry point, which takes scratch from the caller.  It also checks the size limit.
It is collected last, so a run that stops at the first failure has run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

import harness as H  # noqa: F401

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gen(*shape, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


def oracle(q, kp, vp, table, lens, nh, nkv, hd, page, window, scale, gate):
    """Decode attention in double precision from the paged cache: one row per sequence at position
    len-1, keys inside the window only, the head's output times sigmoid(gate)."""
    out = torch.zeros(len(lens), nh, hd, dtype=torch.float64)
    kp, vp, q = kp.double().cpu(), vp.double().cpu(), q.double().cpu().view(len(lens), nh, hd)
    for b, n in enumerate(lens):
        k = torch.stack([kp[table[b, t // page], :, t % page] for t in range(n)])          # [n, nkv, hd]
        v = torch.stack([vp[table[b, t // page], :, :, t % page] for t in range(n)])
        lo = max(0, n - window) if window > 0 else 0
        for h in range(nh):
            s = (k[lo:, h // (nh // nkv)] @ q[b, h]) * scale
            out[b, h] = torch.softmax(s, 0) @ v[lo:, h // (nh // nkv)]
            if gate is not None:
                out[b, h] *= torch.sigmoid(gate[b, h].double().cpu())
    return out.view(len(lens), nh * hd)


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from lastengine_b200.engine.batch import BatchBuilder
    from lastengine_b200.ops import kernels
    L = kernels.lib()
    fn = L.leb_attention_decode_static          # the exported C symbol
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    nh, nkv, hd, page = 8, 2, 64, 64
    lens = [130, 1, 77, 192]
    B = len(lens)
    n_pages = 16
    kp = gen(n_pages, nkv, page, hd, seed=1).to(DEV)
    vp = gen(n_pages, nkv, hd, page, seed=2).to(DEV)
    table = np.full((B, 4), -1, dtype=np.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for j in range(-(-n // page)):
            table[b, j] = nxt
            nxt += 1
    scale = 1 / math.sqrt(hd)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with the array laid out differently (the second finds the first one's
    # leftovers), then a window with a head gate, then one split (no scratch; the gate is applied
    # by the first kernel)
    for call, (splits, window, gated) in enumerate(((4, 0, False), (3, 0, False), (2, 50, True), (1, 50, True), (1, 0, False))):
        q = gen(B, nh * hd, seed=10 + call).to(DEV)
        gate = gen(B, nh, seed=20 + call).to(DEV) if gated else None
        batch = BatchBuilder(torch.device(DEV)).build(list(range(B)), [[0]] * B, [n - 1 for n in lens], [], {0: table})
        want = torch.empty(B, nh * hd, device=DEV, dtype=torch.bfloat16)
        scratch = torch.empty(B * nh * splits * (hd + 2), device=DEV)
        kernels.attention(want, q, kp, vp, batch.tables[0], batch, nh, nkv, hd, page, window, scale, gate=gate,
                          n_splits=splits, scratch=scratch)
        got = torch.full_like(want, float("nan"))
        rc = fn(got.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), batch.tables[0].data_ptr(), 4,
                batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), batch.seq_qstart.data_ptr(),
                gate.data_ptr() if gated else None, nh if gated else 0,
                B, nh, nkv, hd, page, window, scale, splits, stream)
        assert rc == 0, L.leb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= H.TOL_BF16, f"call {call}: {err:.3e}"
        assert torch.equal(got, want)            # same kernels, same order of sums: the same bits
        exact = oracle(q, kp, vp, table, lens, nh, nkv, hd, page, window, scale, gate)
        err = float((got.double().cpu() - exact).abs().max() / exact.abs().max())
        assert err <= 8e-3, f"call {call} against double precision: {err:.3e}"     # the kernel tests' bfloat16 bound
    # a row index beyond the launch's rows (a seq_qstart that is no permutation of 0..B-1) is skipped:
    # the other rows come out as before and nothing is written outside q, out or the array
    qs = batch.seq_qstart.clone()
    qs[1] = B + 5
    again = torch.full_like(want, float("nan"))
    rc = fn(again.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), batch.tables[0].data_ptr(), 4,
            batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), qs.data_ptr(), None, 0,
            B, nh, nkv, hd, page, 0, scale, 1, stream)
    assert rc == 0, L.leb_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(again[[0, 2, 3]], got[[0, 2, 3]]) and torch.isnan(again[1].float()).all()
    # a request beyond the built-in array is refused with a message, and nothing is launched
    rc = fn(got.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), batch.tables[0].data_ptr(), 4,
            batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), batch.seq_qstart.data_ptr(), None, 0,
            4096, 64, 2, 64, page, 0, scale, 32, stream)
    assert rc != 0 and "built-in array" in L.leb_last_error().decode()
