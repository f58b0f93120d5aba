"""Each kernel alone against plain arithmetic, at sizes the tiny models do not use:
widths and vocabularies that are no power of two, head sizes 16/48/80, odd group sizes,
rows that are no multiple of any tile."""
import math

import numpy as np
import pytest
import torch

import harness as H  # noqa: F401  (path setup)
import plain_lfm3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from lastengine_b200.ops import kernels
    return kernels


def builder():
    from lastengine_b200.engine.batch import BatchBuilder
    return BatchBuilder(torch.device(DEV))


def gen(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(dtype)


def err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / (want.abs().max() + 1e-30))


# ---- rows ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = gen(301, 72, seed=1).to(dtype)
    toks = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    x = torch.empty(5, 72, device=DEV)
    K().embed(x, table.to(DEV), toks.to(DEV))
    assert torch.equal(x.cpu(), table.float()[toks.long()])


@pytest.mark.parametrize("D", [100, 64, 2048, 5000])
def test_rmsnorm(D):
    x, w = gen(7, D, seed=2, scale=3.0), 1 + 0.1 * gen(D, seed=3)
    want = P.rms_norm(x.double(), w.double(), 1e-3)
    out = torch.empty(7, D, device=DEV)
    K().rmsnorm(out, x.to(DEV), w.to(DEV), 1e-3)
    assert err(out, want) < 1e-6
    ob = torch.empty(7, D, device=DEV, dtype=torch.bfloat16)
    K().rmsnorm(ob, x.to(DEV), w.to(DEV), 1e-3)
    assert err(ob, want) < 5e-3                     # its own order of sums: equal up to one bfloat16 rounding
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    o3 = torch.empty(3, D, device=DEV)
    K().rmsnorm(o3, x.to(DEV), w.to(DEV), 1e-3, rows=rows)
    assert torch.equal(o3.cpu(), out.cpu()[[6, 0, 3]])
    res = gen(7, D, seed=4).to(DEV)
    r0 = res.clone()
    K().rmsnorm(res, x.to(DEV), w.to(DEV), 1e-3, add=True)
    assert err(res, r0.cpu().double() + want) < 1e-6


def test_swiglu():
    gu = gen(9, 2 * 37, seed=5, scale=2.0)
    want = P.silu(gu[:, :37].double()) * gu[:, 37:].double()
    out = torch.empty(9, 37, device=DEV)
    K().swiglu(out, gu.to(DEV))
    assert err(out, want) < 1e-6
    ob = torch.empty(9, 37, device=DEV, dtype=torch.bfloat16)
    K().swiglu(ob, gu.to(DEV))
    assert err(ob, want) < 5e-3


# ---- matrix products ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K_", [(1, 50, 70), (37, 129, 33), (64, 64, 16), (130, 70, 200)])
def test_linear_f32(M, N, K_):
    x, w = gen(M, K_, seed=6), gen(N, K_, seed=7)
    want = x.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV))
    assert err(out, want) < 2e-6
    base = gen(M, N, seed=8).to(DEV)
    b0 = base.clone()
    K().linear(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    assert err(base, b0.cpu().double() + want) < 2e-6
    # a row's result does not depend on the other rows of the launch
    one = torch.empty(1, N, device=DEV)
    K().linear(one, x[M - 1:].to(DEV), w.to(DEV))
    assert torch.equal(one.cpu()[0], out.cpu()[M - 1])


@pytest.mark.parametrize("M", [1, 5, 8, 9, 33, 64, 65, 200])
@pytest.mark.parametrize("N,K_", [(48, 72), (100, 200), (17, 40)])
def test_linear_bf16_small(M, N, K_):
    x, w = gen(M, K_, seed=9, dtype=torch.bfloat16), gen(N, K_, seed=10, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV), streaming=True)
    assert err(out, want) < 1e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear(ob, x.to(DEV), w.to(DEV), streaming=True)
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=11).to(DEV)
    b0 = base.clone()
    K().linear(base, x.to(DEV), w.to(DEV), K().ACCUMULATE, streaming=True)
    assert err(base, b0.cpu().double() + want) < 1e-5
    one = torch.empty(1, N, device=DEV)
    K().linear(one, x[M - 1:].to(DEV), w.to(DEV), streaming=True)
    assert torch.equal(one.cpu()[0], out.cpu()[M - 1])


@pytest.mark.parametrize("M", [1, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K_", [(48, 72), (100, 200), (17, 40), (2048, 2048), (6144, 136), (352, 5632), (9600, 64)])
def test_linear_bf16_stream(M, N, K_):
    """The decode product (weights through rings of asynchronous copies): widths that leave part
    of a tile, K that leaves part of a chunk or gives some warps nothing, more tiles than blocks."""
    x, w = gen(M, K_, seed=9, dtype=torch.bfloat16), gen(N, K_, seed=10, scale=0.05, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV))
    assert err(out, want) < 1e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear(ob, x.to(DEV), w.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=11).to(DEV)
    b0 = base.clone()
    K().linear(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    assert err(base, b0.cpu().double() + want) < 1e-5
    one = torch.empty(1, N, device=DEV)
    K().linear(one, x[M - 1:].to(DEV), w.to(DEV))
    assert torch.equal(one.cpu()[0], out.cpu()[M - 1])      # a row does not depend on the other rows
    if N % 32 == 0:
        from lastengine_b200.parts.ffn import fuse_gate_up
        F = N // 2
        w13 = fuse_gate_up(w[:F], w[F:], True).to(DEV)
        sw = P.silu(want[:, :F]) * want[:, F:]
        o2 = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
        K().linear(o2, x.to(DEV), w13, K().SWIGLU)
        assert err(o2, sw) < 6e-3


@pytest.mark.parametrize("M,F,D", [(3, 48, 72), (40, 160, 96), (70, 16, 40)])
def test_linear_bf16_swiglu_epilogue(M, F, D):
    from lastengine_b200.parts.ffn import fuse_gate_up
    x = gen(M, D, seed=12, dtype=torch.bfloat16)
    w1, w3 = gen(F, D, seed=13, dtype=torch.bfloat16), gen(F, D, seed=14, dtype=torch.bfloat16)
    want = P.silu(x.double() @ w1.double().T) * (x.double() @ w3.double().T)
    w13 = fuse_gate_up(w1, w3, True).to(DEV)
    out = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    K().linear(out, x.to(DEV), w13, K().SWIGLU, streaming=True)
    assert err(out, want) < 6e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_grouped(dtype):
    E, N, K_ = 5, 40, 56
    counts = [3, 0, 70, 1, 9]
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    Ptot = int(offs[-1])
    x, w = gen(Ptot, K_, seed=15, dtype=dtype), gen(E, N, K_, seed=16, dtype=dtype)
    want = torch.zeros(Ptot, N, dtype=torch.float64)
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        want[a:b] = x[a:b].double() @ w[e].double().T
    out = torch.empty(Ptot, N, device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV), rows_hint=Ptot)
    assert err(out, want) < 1e-5


@pytest.mark.parametrize("counts,N,K_", [([3, 0, 0, 1, 9, 0, 2], 48, 72), ([1, 0, 0, 0, 0, 0, 0, 4], 3584, 2048),
                                         ([17, 8, 0, 33, 1, 16, 9, 5], 96, 200), ([5] * 32, 352, 136),
                                         ([0, 0, 0, 0, 0, 0, 0, 0, 0, 7], 64, 64)])
def test_linear_grouped_stream(counts, N, K_):
    """Grouped products through the ring-fed kernel: experts without rows, with one row, with more
    rows than one block of 8 or 16 takes; store, add, both result types, and the SwiGLU epilogue."""
    E = len(counts)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    Ptot = int(offs[-1])
    assert Ptot <= 16 * E                                   # the sizes this kernel is chosen for
    x, w = gen(Ptot, K_, seed=15, dtype=torch.bfloat16), gen(E, N, K_, seed=16, scale=0.05, dtype=torch.bfloat16)
    want = torch.zeros(Ptot, N, dtype=torch.float64)
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        want[a:b] = x[a:b].double() @ w[e].double().T
    out = torch.full((Ptot, N), float("nan"), device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV), rows_hint=Ptot)
    assert err(out, want) < 1e-5
    old = torch.empty(Ptot, N, device=DEV)
    K().linear(old, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV), rows_hint=Ptot, streaming=True)
    assert err(old, want) < 1e-5                            # the register-fed kernel on the same groups
    ob = torch.empty(Ptot, N, device=DEV, dtype=torch.bfloat16)
    K().linear(ob, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(Ptot, N, seed=17).to(DEV)
    b0 = base.clone()
    K().linear(base, x.to(DEV), w.to(DEV), K().ACCUMULATE, group_offsets=offs.to(DEV))
    assert err(base, b0.cpu().double() + want) < 1e-5
    if N % 32 == 0:
        from lastengine_b200.parts.ffn import fuse_gate_up
        F = N // 2
        w13 = torch.stack([fuse_gate_up(w[e, :F], w[e, F:], True) for e in range(E)]).to(DEV)
        sw = P.silu(want[:, :F]) * want[:, F:]
        o2 = torch.empty(Ptot, F, device=DEV, dtype=torch.bfloat16)
        K().linear(o2, x.to(DEV), w13, K().SWIGLU, group_offsets=offs.to(DEV))
        assert err(o2, sw) < 6e-3


@pytest.mark.parametrize("counts,N,K_", [([300, 0, 129, 1, 700, 128], 96, 200), ([5, 260, 0, 0, 131], 352, 136),
                                         ([128, 128, 128], 512, 64), ([0, 0, 1000, 0], 3584, 256)])
def test_linear_grouped_tcgen05(counts, N, K_):
    """Grouped products with many rows per expert (prompts) on tcgen05: experts without rows, with
    one row, with rows that end inside a tile (the tile's other rows belong to the next expert and
    must not be written by this one), widths that end inside a weight tile."""
    E = len(counts)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    Ptot = int(offs[-1])
    assert Ptot > 16 * E
    x, w = gen(Ptot, K_, seed=15, dtype=torch.bfloat16), gen(E, N, K_, seed=16, scale=0.05, dtype=torch.bfloat16)
    want = torch.zeros(Ptot, N, dtype=torch.float64)
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        want[a:b] = x[a:b].double() @ w[e].double().T
    out = torch.full((Ptot, N), float("nan"), device=DEV)
    K().linear(out, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV), rows_hint=Ptot)
    K().check_device_status()
    assert err(out, want) < 2e-5
    ob = torch.empty(Ptot, N, device=DEV, dtype=torch.bfloat16)
    K().linear(ob, x.to(DEV), w.to(DEV), group_offsets=offs.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(Ptot, N, seed=17).to(DEV)
    b0 = base.clone()
    K().linear(base, x.to(DEV), w.to(DEV), K().ACCUMULATE, group_offsets=offs.to(DEV))
    assert err(base, b0.cpu().double() + want) < 2e-5
    if N % 32 == 0:
        from lastengine_b200.parts.ffn import fuse_gate_up
        F = N // 2
        w13 = torch.stack([fuse_gate_up(w[e, :F], w[e, F:], True) for e in range(E)]).to(DEV)
        sw = P.silu(want[:, :F]) * want[:, F:]
        o2 = torch.empty(Ptot, F, device=DEV, dtype=torch.bfloat16)
        K().linear(o2, x.to(DEV), w13, K().SWIGLU, group_offsets=offs.to(DEV))
        assert err(o2, sw) < 6e-3
    K().check_device_status()


# ---- short convolution ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Lc,D", [(3, 72), (4, 130), (2, 64)])
def test_shortconv_with_state(dtype, Lc, D):
    """Three sequences with unequal rows in two consecutive steps, one of them shorter than the
    convolution reaches back; compared with the plain convolution over the joined rows."""
    lens1, lens2 = [1, 5, 2], [3, 1, 1]
    slots = [4, 0, 2]
    w = gen(D, Lc, seed=17)
    bcx_all = [gen(a + b, 3 * D, seed=20 + i, dtype=dtype) for i, (a, b) in enumerate(zip(lens1, lens2))]
    state = torch.full((6, D, Lc - 1), 7.0, device=DEV)   # stale contents of other slots
    for s in slots:
        state[s].zero_()
    bb = builder()
    got = [[] for _ in slots]
    for step, lens in enumerate((lens1, lens2)):
        lo = [0] * 3 if step == 0 else lens1
        rows = torch.cat([bcx_all[i][lo[i]:lo[i] + lens[i]] for i in range(3)]).to(DEV)
        batch = bb.build(slots, [[0] * n for n in lens], lo, [], {})
        y = torch.empty(sum(lens), D, device=DEV, dtype=dtype)
        K().shortconv(y, rows, w.to(DEV), None, state, batch, Lc)
        r0 = 0
        for i, n in enumerate(lens):
            got[i].append(y[r0:r0 + n].float().cpu())
            r0 += n
    for i in range(3):
        bcx = bcx_all[i].double()
        bx = bcx[:, :D] * bcx[:, 2 * D:]
        padded = torch.cat([torch.zeros(Lc - 1, D, dtype=torch.float64), bx])
        acc = sum(padded[j:j + bx.shape[0]] * w.double()[:, j][None] for j in range(Lc))
        want = bcx[:, D:2 * D] * acc
        assert err(torch.cat(got[i]), want) < (1e-6 if dtype == torch.float32 else 5e-3)
        assert err(state[slots[i]].cpu().T, padded[-(Lc - 1):]) < 1e-6      # oldest first
    assert float(state[1].min()) == 7.0 and float(state[5].max()) == 7.0     # other slots untouched


@pytest.mark.parametrize("Lc,D", [(3, 136), (4, 72), (3, 2048)])
def test_shortconv_many_rows(Lc, D):
    """Prompts long enough for the kernel that walks several rows per thread: sequences start in
    the middle of a thread's rows, one is shorter than the filter, one slot is padding, and one
    starts from a state that is not zero."""
    lens = [1, 301, 2, 130, 77]
    slots = [3, 1, -1, 0, 2]
    w = gen(D, Lc, seed=18)
    bcx = [gen(n, 3 * D, seed=40 + i, dtype=torch.bfloat16) for i, n in enumerate(lens)]
    state = torch.zeros(4, D, Lc - 1, device=DEV)
    old = gen(D, Lc - 1, seed=19)
    state[2] = old.to(DEV)
    batch = builder().build(slots, [[0] * n for n in lens], [0, 0, 0, 0, 5], [], {})
    y = torch.full((sum(lens), D), float("nan"), device=DEV, dtype=torch.bfloat16)
    K().shortconv(y, torch.cat(bcx).to(DEV), w.to(DEV), None, state, batch, Lc)
    r0 = 0
    for i, n in enumerate(lens):
        got = y[r0:r0 + n].float().cpu()
        r0 += n
        if slots[i] < 0:
            assert float(got.abs().max()) == 0.0
            continue
        x = bcx[i].double()
        bx = x[:, :D] * x[:, 2 * D:]
        before = old.double().T if slots[i] == 2 else torch.zeros(Lc - 1, D, dtype=torch.float64)
        padded = torch.cat([before, bx])
        acc = sum(padded[j:j + n] * w.double()[:, j][None] for j in range(Lc))
        assert err(got, x[:, D:2 * D] * acc) < 5e-3, i
        assert err(state[slots[i]].cpu().T, padded[-(Lc - 1):]) < 1e-6, i


@pytest.mark.parametrize("B,D,K_,Lc", [(8, 2048, 2048, 3), (1, 72, 40, 2), (13, 136, 200, 4), (16, 48, 64, 5), (5, 100, 72, 3),
                                       (40, 2048, 2048, 3), (100, 136, 1024, 4), (18, 48, 512, 5), (90, 136, 1024, 4)])
def test_shortconv_decode_fused(B, D, K_, Lc):
    """Projection and convolution of a decode step without a convolution kernel (up to 16 sequences:
    one launch; more: the sliced product, whose second kernel convolves), three steps in a row so that the
    state it writes is the state it reads next; one sequence is padding, the slots are not in order
    and other slots hold stale values.  Compared with the plain formulas (projection rounded to
    bfloat16 as the two-kernel path stores it) and with the two-kernel path itself."""
    h_all = [gen(B, K_, seed=60 + t, dtype=torch.bfloat16) for t in range(3)]
    w_in = gen(3 * D, K_, seed=63, scale=0.05, dtype=torch.bfloat16)
    w = gen(D, Lc, seed=64)
    slots = [(5 * i + 3) % (B + 3) for i in range(B)]
    assert len(set(slots)) == B
    if B > 2:
        slots[1] = -1
    state = torch.full((B + 3, D, Lc - 1), 7.0, device=DEV)
    start = gen(B, D, Lc - 1, seed=65)
    for i, s in enumerate(slots):
        if s >= 0:
            state[s] = start[i].to(DEV)
    state2 = state.clone()
    hist = start.double().permute(0, 2, 1).clone()          # [B, Lc-1, D], oldest first
    bb = builder()
    for t in range(3):
        batch = bb.build(slots, [[0]] * B, [t] * B, [], {})
        y = torch.full((B, D), float("nan"), device=DEV, dtype=torch.bfloat16)
        assert K().shortconv_decode_fused(y, h_all[t].to(DEV), w_in.to(DEV), w.to(DEV), None, state, batch, Lc)
        bcx = torch.empty(B, 3 * D, device=DEV, dtype=torch.bfloat16)
        K().linear(bcx, h_all[t].to(DEV), w_in.to(DEV))
        y2 = torch.empty(B, D, device=DEV, dtype=torch.bfloat16)
        K().shortconv(y2, bcx, w.to(DEV), None, state2, batch, Lc)
        p = (h_all[t].double() @ w_in.double().T).to(torch.bfloat16).double()
        bx = p[:, :D] * p[:, 2 * D:]
        taps = torch.cat([hist, bx[:, None]], dim=1)          # [B, Lc, D]
        want = p[:, D:2 * D] * (taps * w.double().T[None]).sum(1)
        hist = taps[:, 1:]
        for i, s in enumerate(slots):
            if s < 0:
                assert float(y[i].abs().max()) == 0.0
                continue
            assert err(y[i], want[i]) < 6e-3, (t, i)
            assert err(y[i], y2[i].float().cpu()) < 6e-3, (t, i)
            assert err(state[s].cpu().T, hist[i]) < 6e-3, (t, i)
    used = [s for s in slots if s >= 0]
    for s in range(B + 3):
        if s not in used:
            assert float(state[s].min()) == 7.0 and float(state[s].max()) == 7.0


@pytest.mark.parametrize("M,D,K_,N2", [(8, 2048, 2048, 6144), (1, 72, 40, 64), (13, 136, 200, 96), (16, 104, 64, 32),
                                       (64, 2048, 5632, 6144), (17, 72, 40, 64), (100, 136, 200, 96), (128, 104, 64, 32),
                                       (80, 2048, 5632, 6144), (96, 136, 200, 96)])
def test_norm_split_between_two_products(M, D, K_, N2):
    """An RMSNorm split between the product that adds into the residual and the product that reads
    the normed rows (decode steps): the first leaves bfloat16(x * g) and partial sums of x^2, the
    second scales its sums by rsqrt(mean + eps).  Up to 16 rows through the weight stream, above
    through the sliced tcgen05 product.  Compared with norm and products in float64."""
    from lastengine_b200.parts.ffn import fuse_gate_up
    eps = 3e-5
    a, w = gen(M, K_, seed=70, dtype=torch.bfloat16), gen(D, K_, seed=71, scale=0.05, dtype=torch.bfloat16)
    x0, g = gen(M, D, seed=72, scale=3.0), 1.0 + gen(D, seed=73, scale=0.3)
    x = x0.to(DEV)
    sp = K().SplitNorm(torch.empty(M, D, device=DEV, dtype=torch.bfloat16),
                       torch.full((M, -(-D // 16)), float("nan"), device=DEV), g.to(DEV), eps)
    K().linear(x, a.to(DEV), w.to(DEV), K().ACCUMULATE, emit=sp)
    assert sp.filled
    xn = x0.double() + a.double() @ w.double().T
    assert err(x, xn) < 2e-5
    assert err(sp.values, xn * g.double()) < 5e-3
    assert err(sp.ssq.sum(1), (xn ** 2).sum(1)) < 1e-5
    normed = xn * torch.rsqrt((xn ** 2).mean(1, keepdim=True) + eps) * g.double()
    w2 = gen(N2, D, seed=74, scale=0.05, dtype=torch.bfloat16)
    out = torch.empty(M, N2, device=DEV, dtype=torch.bfloat16)
    K().linear(out, sp.values, w2.to(DEV), scale=sp)
    assert err(out, normed @ w2.double().T) < 6e-3
    F = N2 // 2
    o2 = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    K().linear(o2, sp.values, fuse_gate_up(w2[:F], w2[F:], True).to(DEV), K().SWIGLU, scale=sp)
    assert err(o2, P.silu(normed @ w2[:F].double().T) * (normed @ w2[F:].double().T)) < 6e-3
    K().check_device_status()


# ---- rotation and cache write ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rope_dim,lens", [(4, 2, 16, 16, [3, 70]), (3, 1, 48, 32, [3, 70]), (5, 5, 80, 80, [3, 70]),
                                                      (2, 1, 64, 64, [3, 70]), (6, 2, 128, 128, [3, 70]),
                                                      (9, 3, 64, 64, [60, 100]), (13, 1, 64, 64, [400, 290])])
def test_qk_rope_store(dtype, nh, nkv, hd, rope_dim, lens):
    if dtype == torch.float32 and max(lens) > 128:
        # a float angle is off by up to position x 6e-8: the float path is compared at short positions
        # only; the long case is there for the bfloat16 kernel that takes several heads per warp
        lens = [n // 4 for n in lens]
    page = 64
    pos0 = [62, 5]                                  # rows cross a page boundary
    M = sum(lens)
    width = nh * hd + 2 * nkv * hd
    qkv = gen(M, width, seed=30, dtype=dtype)
    qn, kn = 1 + 0.1 * gen(hd, seed=31), 1 + 0.1 * gen(hd, seed=32)
    theta, eps = 12345.0, 1e-4
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rope_dim // 2, dtype=torch.float64) / rope_dim).float()
    width = max(-(-(p + n) // page) for p, n in zip(pos0, lens))
    n_pages = 2 * width + 2
    order = np.random.default_rng(5).permutation(n_pages)[:2 * width].astype(np.int32)   # pages in no order
    tables = {0: order.reshape(2, width)}
    kp = torch.zeros(n_pages, nkv, page, hd, device=DEV, dtype=dtype)
    vp = torch.zeros(n_pages, nkv, hd, page, device=DEV, dtype=dtype)      # values: positions contiguous
    batch = builder().build([0, 1], [[0] * n for n in lens], pos0, [], tables)
    q_out = torch.empty(M, nh * hd, device=DEV, dtype=dtype)
    qd = qkv.to(DEV)
    K().qk_rope_store(q_out, qd[:, :nh * hd], qd[:, nh * hd:(nh + nkv) * hd], qd[:, (nh + nkv) * hd:], kp, vp,
                      batch.tables[0], batch, qn.to(DEV), kn.to(DEV), eps, inv.to(DEV), rope_dim, True, nh, nkv, hd, page)
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    r0 = 0
    for b, n in enumerate(lens):
        rows = qkv[r0:r0 + n].double()
        pos = torch.arange(pos0[b], pos0[b] + n)
        q = P.rope(P.rms_norm(rows[:, :nh * hd].view(n, nh, hd), qn.double(), eps), pos, rope_dim, theta)
        k = P.rope(P.rms_norm(rows[:, nh * hd:(nh + nkv) * hd].view(n, nkv, hd), kn.double(), eps), pos, rope_dim, theta)
        v = rows[:, (nh + nkv) * hd:].view(n, nkv, hd)
        assert err(q_out[r0:r0 + n].view(n, nh, hd), q) < tol
        for i, p_ in enumerate(pos.tolist()):
            pg = int(tables[0][b, p_ // page])
            assert err(kp[pg, :, p_ % page, :], k[i]) < tol
            assert err(vp[pg, :, :, p_ % page], v[i]) < tol
        r0 += n


# ---- attention ---------------------------------------------------------------------------------------
def plain_attention(q, k, v, qpos, window, scale):
    """q [Tq, nh, hd], k/v [Tk, nkv, hd] (positions 0..Tk-1), qpos [Tq]."""
    Tq, nh, hd = q.shape
    nkv = k.shape[1]
    out = torch.zeros_like(q)
    t = torch.arange(k.shape[0])
    for h in range(nh):
        s = (q[:, h] @ k[:, h // (nh // nkv)].T) * scale
        ok = t[None] <= qpos[:, None]
        if window > 0:
            ok &= t[None] > qpos[:, None] - window
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // (nh // nkv)]
    return out


def fill_cache(k, v, pages, nkv, hd, page, dtype):
    n_pages = max(pages) + 2
    kp = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)   # unused places hold NaN
    vp = torch.full((n_pages, nkv, hd, page), float("nan"), dtype=dtype)   # values: positions contiguous
    for t in range(k.shape[0]):
        kp[pages[t // page], :, t % page] = k[t].to(dtype)
        vp[pages[t // page], :, :, t % page] = v[t].to(dtype)
    return kp.to(DEV), vp.to(DEV)


@pytest.mark.parametrize("nh,nkv,hd", [(32, 8, 64), (6, 2, 128), (5, 5, 64), (16, 1, 64)])
@pytest.mark.parametrize("window,gated,with_norm", [(0, False, True), (40, True, True), (0, False, False)])
def test_decode_attention_that_norms_rotates_and_stores_the_step_itself(nh, nkv, hd, window, gated, with_norm):
    """A decode step handed to the attention kernel as the projection left it (raw q, k and v) against
    the same step with the rotary kernel first: the same output bits and the same cache, at every
    split count, for sequences whose new position starts a page, ends one, or is the first of all;
    a padding sequence among them; and against double-precision arithmetic."""
    page, dtype = 64, torch.bfloat16
    lens = [130, 1, 64, 65, 257, 7]                 # lengths after the step: the new token sits at len - 1
    slots = [0, 1, -1, 2, 3, 4]
    B = len(lens)
    width = max(-(-n // page) for n in lens)
    n_pages = B * width + 1
    order = np.random.default_rng(6).permutation(n_pages)[:B * width].astype(np.int32).reshape(B, width)
    kp0 = gen(n_pages, nkv, page, hd, seed=50, dtype=dtype).to(DEV)
    vp0 = gen(n_pages, nkv, hd, page, seed=51, dtype=dtype).to(DEV)
    qkv = gen(B, (nh + 2 * nkv) * hd + nh, seed=52, dtype=dtype).to(DEV)        # q | k | v | gate as one projection
    q_in, k_in = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd]
    v_in, gate = qkv[:, (nh + nkv) * hd:(nh + 2 * nkv) * hd], (qkv[:, (nh + 2 * nkv) * hd:] if gated else None)
    qn = (1 + 0.1 * gen(hd, seed=53)).to(DEV) if with_norm else None
    kn = (1 + 0.1 * gen(hd, seed=54)).to(DEV) if with_norm else None
    theta, eps, scale = 5e4, 1e-5, 1 / math.sqrt(hd)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float().to(DEV)
    batch = builder().build(slots, [[0]] * B, [n - 1 for n in lens], [], {0: order})
    assert K().decode_attention_takes_raw(dtype, batch, B, nh, nkv, hd, page, inv, hd, True)
    for splits in (1, 2, 5):
        scratch = torch.empty(B * nh * splits * (hd + 2), device=DEV)
        # the two-kernel way
        kp_a, vp_a = kp0.clone(), vp0.clone()
        q_rot = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
        K().qk_rope_store(q_rot, q_in, k_in, v_in, kp_a, vp_a, batch.tables[0], batch, qn, kn, eps, inv, hd, True, nh, nkv, hd, page)
        want = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
        K().attention(want, q_rot, kp_a, vp_a, batch.tables[0], batch, nh, nkv, hd, page, window, scale, gate=gate,
                      n_splits=splits, scratch=scratch)
        # the kernel that does it all
        kp_b, vp_b = kp0.clone(), vp0.clone()
        got = torch.full_like(want, float("nan"))
        K().attention(got, None, kp_b, vp_b, batch.tables[0], batch, nh, nkv, hd, page, window, scale, gate=gate,
                      n_splits=splits, scratch=scratch, raw=K().RawQKV(q_in, k_in, v_in, qn, kn, eps, inv, hd, True))
        torch.cuda.synchronize()
        assert torch.equal(kp_a, kp_b) and torch.equal(vp_a, vp_b), f"{splits} splits: the caches differ"
        assert not torch.equal(kp_a, kp0)
        assert torch.equal(got, want), f"{splits} splits: {err(got, want):.3e}"
    # against double precision, from the cache the kernel left
    for b, n in enumerate(lens):
        if slots[b] < 0:
            assert float(got[b].float().abs().max()) == 0.0
            continue
        k = torch.stack([kp_b[int(order[b, t // page]), :, t % page].double().cpu() for t in range(n)])
        v = torch.stack([vp_b[int(order[b, t // page]), :, :, t % page].double().cpu() for t in range(n)])
        row = qkv[b].double().cpu()
        q = row[:nh * hd].view(1, nh, hd)
        if with_norm:
            q = P.rms_norm(q, qn.double().cpu(), eps)
        q = P.round_bf16(P.rope(q, torch.tensor([n - 1]), hd, theta))
        o = plain_attention(q, k, v, torch.tensor([n - 1]), window, scale)[0]
        if gated:
            o = o * torch.sigmoid(row[(nh + 2 * nkv) * hd:])[:, None]
        assert err(got[b].view(nh, hd), o) < 8e-3, b
        # the new key is the normed and rotated one
        kn_new = row[nh * hd:(nh + nkv) * hd].view(1, nkv, hd)
        if with_norm:
            kn_new = P.rms_norm(kn_new, kn.double().cpu(), eps)
        assert err(k[n - 1], P.rope(kn_new, torch.tensor([n - 1]), hd, theta)[0]) < 6e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 48), (10, 5, 80), (16, 1, 32), (8, 8, 128), (32, 8, 64), (12, 2, 96)])
@pytest.mark.parametrize("window", [0, 40])
def test_attention_prompt_and_decode(dtype, nh, nkv, hd, window):
    page, Tk = 64, 150
    k, v = gen(Tk, nkv, hd, seed=40, dtype=dtype), gen(Tk, nkv, hd, seed=41, dtype=dtype)
    pages = [3, 0, 5]
    kp, vp = fill_cache(k, v, pages, nkv, hd, page, dtype)
    scale = 1 / math.sqrt(hd)
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    tables = {0: np.array([pages], dtype=np.int32)}
    # a chunk of 37 rows continuing at position 100, then a single row at the end, split four ways
    for q0, n, splits in ((100, 37, 1), (0, 150, 1), (149, 1, 1), (149, 1, 4), (70, 1, 16)):
        q = gen(n, nh, hd, seed=42 + n, dtype=dtype)
        batch = builder().build([0], [[0] * n], [q0], [], tables)
        out = torch.empty(n, nh * hd, device=DEV, dtype=dtype)
        scratch = torch.empty(n * nh * splits * (hd + 2), device=DEV) if splits > 1 else None
        K().attention(out, q.reshape(n, nh * hd).to(DEV), kp, vp, batch.tables[0], batch, nh, nkv, hd, page,
                      window, scale, n_splits=splits, scratch=scratch)
        want = plain_attention(q.double(), k.double(), v.double(), torch.arange(q0, q0 + n), window, scale)
        assert err(out.view(n, nh, hd), want) < tol, (q0, n, splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_far_key_and_window_edge(dtype):
    """One early key is made to dominate: among hundreds of keys the output must be its value;
    with a window that ends just before it, it must vanish, and one position earlier it must not."""
    nh, nkv, hd, page, Tk = 4, 2, 64, 64, 300
    k, v = gen(Tk, nkv, hd, seed=50, scale=0.1), gen(Tk, nkv, hd, seed=51)
    q = gen(1, nh, hd, seed=52, scale=0.1)
    far = 3
    k[far] = 0
    k[far, :, 0] = 40.0
    q[..., 0] = 40.0                       # score 1600/8 = 200 against O(1) elsewhere
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    pages = [1, 4, 2, 0, 6]
    kp, vp = fill_cache(k, v, pages, nkv, hd, page, dtype)
    tables = {0: np.array([pages], dtype=np.int32)}
    scale = 1 / math.sqrt(hd)
    for splits in (1, 5):
        for window, sees in ((0, True), (Tk - far, True), (Tk - far - 1, False)):
            batch = builder().build([0], [[0]], [Tk - 1], [], tables)
            out = torch.empty(1, nh * hd, device=DEV, dtype=dtype)
            scratch = torch.empty(nh * splits * (hd + 2), device=DEV)
            K().attention(out, q.reshape(1, nh * hd).to(DEV), kp, vp, batch.tables[0], batch, nh, nkv, hd, page,
                          window, scale, n_splits=splits, scratch=scratch)
            want = plain_attention(q.double(), k.double(), v.double(), torch.tensor([Tk - 1]), window, scale)
            assert err(out.view(1, nh, hd), want) < (2e-5 if dtype == torch.float32 else 8e-3)
            hit = err(out.view(1, nh, hd)[0, 0], v[far, 0].double()) < 1e-2
            assert hit == sees, (splits, window)


@pytest.mark.parametrize("nh,nkv", [(4, 4), (4, 2), (8, 2), (8, 1)])
@pytest.mark.parametrize("window", [0, 150])
def test_attention_long_prompts_on_tcgen05(nh, nkv, window):
    """Head size 64 with 1, 2, 4 and 8 query heads per kv head: the tcgen05 prompt kernel.  Two
    sequences of several tiles and pages; the second continues at a position that is no multiple
    of anything.  Keys grow along the sequence, so every row's maximum moves many times by more
    than the factor the kernel tolerates before it rescales; one early key dominates a late query;
    unused places of the cache hold NaN."""
    hd, page, dtype = 64, 64, torch.bfloat16
    lens_k, pos0, qn = [700, 333], [0, 203], [700, 130]
    ks = [gen(n, nkv, hd, seed=160 + i) * torch.linspace(0.2, 3.0, n)[:, None, None] for i, n in enumerate(lens_k)]
    vs = [gen(n, nkv, hd, seed=170 + i) for i, n in enumerate(lens_k)]
    qs = [gen(n, nh, hd, seed=180 + i) for i, n in enumerate(qn)]
    far = 5
    ks[0][far] = 0
    ks[0][far, :, 0] = 60.0
    qs[0][650, :, :] = 0
    qs[0][650, :, 0] = 8.0                       # score 480/8 = 60 against a few elsewhere
    ks, vs, qs = [t.to(dtype) for t in ks], [t.to(dtype) for t in vs], [t.to(dtype) for t in qs]
    n_pages = 20
    order = np.random.default_rng(7).permutation(n_pages).astype(np.int32)
    page_lists = [order[:11].tolist(), order[11:17].tolist()]
    pools_k = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)
    pools_v = torch.full((n_pages, nkv, hd, page), float("nan"), dtype=dtype)
    for i in range(2):
        for t in range(lens_k[i]):
            pools_k[page_lists[i][t // page], :, t % page] = ks[i][t]
            pools_v[page_lists[i][t // page], :, :, t % page] = vs[i][t]
    table = np.full((2, 11), -1, dtype=np.int32)
    for i, pl in enumerate(page_lists):
        table[i, :len(pl)] = pl
    batch = builder().build([0, 1], [[0] * n for n in qn], pos0, [], {0: table})
    M = sum(qn)
    out = torch.full((M, nh * hd), float("nan"), device=DEV, dtype=dtype)
    K().attention(out, torch.cat(qs).reshape(M, nh * hd).to(DEV), pools_k.to(DEV), pools_v.to(DEV), batch.tables[0],
                  batch, nh, nkv, hd, page, window, 0.125)
    K().check_device_status()
    r0 = 0
    for i, n in enumerate(qn):
        want = plain_attention(qs[i].double(), ks[i].double(), vs[i].double(), torch.arange(pos0[i], pos0[i] + n), window, 0.125)
        assert err(out[r0:r0 + n].view(n, nh, hd), want) < 8e-3, i
        r0 += n
    if window == 0:
        assert err(out[650].view(nh, hd)[0], vs[0][far, 0].double()) < 1e-2     # the far key's value, alone


@pytest.mark.parametrize("dtype,nh,nkv,hd", [(torch.float32, 6, 2, 48), (torch.bfloat16, 6, 2, 64), (torch.bfloat16, 6, 2, 48),
                                             (torch.bfloat16, 8, 2, 64), (torch.bfloat16, 8, 1, 64)])
def test_attention_batch_of_unequal_sequences(dtype, nh, nkv, hd):
    """Several sequences in one launch, each with its own pages, lengths and row counts; one is padding."""
    page = 64
    lens_k, pos0, qn = [90, 10, 130], [60, 0, 129], [30, 10, 1]
    ks = [gen(n, nkv, hd, seed=60 + i, dtype=dtype) for i, n in enumerate(lens_k)]
    vs = [gen(n, nkv, hd, seed=70 + i, dtype=dtype) for i, n in enumerate(lens_k)]
    pools_k = torch.full((12, nkv, page, hd), float("nan"), dtype=dtype)
    pools_v = torch.full((12, nkv, hd, page), float("nan"), dtype=dtype)
    page_lists = [[7, 2], [9], [0, 11, 4]]
    for i in range(3):
        for t in range(lens_k[i]):
            pools_k[page_lists[i][t // page], :, t % page] = ks[i][t]
            pools_v[page_lists[i][t // page], :, :, t % page] = vs[i][t]
    table = np.full((4, 3), -1, dtype=np.int32)
    for i, pl in enumerate(page_lists):
        table[i if i < 2 else 3, :len(pl)] = pl
    slots, rows = [0, 1, -1, 2], [qn[0], qn[1], 2, qn[2]]
    qs = [gen(n, nh, hd, seed=80 + i, dtype=dtype) for i, n in enumerate(rows)]
    batch = builder().build(slots, [[0] * n for n in rows], [pos0[0], pos0[1], 0, pos0[2]], [], {0: table})
    M = sum(rows)
    out = torch.empty(M, nh * hd, device=DEV, dtype=dtype)
    K().attention(out, torch.cat(qs).reshape(M, nh * hd).to(DEV), pools_k.to(DEV), pools_v.to(DEV), batch.tables[0],
                  batch, nh, nkv, hd, page, 0, 0.2)
    r0 = 0
    for j, (s, n) in enumerate(zip(slots, rows)):
        if s >= 0:
            p0 = [pos0[0], pos0[1], 0, pos0[2]][j]
            want = plain_attention(qs[j].double(), ks[s].double(), vs[s].double(), torch.arange(p0, p0 + n), 0, 0.2)
            assert err(out[r0:r0 + n].view(n, nh, hd), want) < (2e-5 if dtype == torch.float32 else 8e-3)
        else:
            assert float(out[r0:r0 + n].abs().max()) == 0.0
        r0 += n


# ---- experts ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,k,norm,bias,scaling", [(8, 2, True, True, 1.0), (5, 1, False, False, 1.5), (32, 4, True, True, 2.0)])
def test_moe_router_align_combine(dtype, E, k, norm, bias, scaling):
    M, D = 77, 104
    h = gen(M, D, seed=90, dtype=dtype)
    wr, b = gen(E, D, seed=91, scale=0.3), gen(E, seed=92, scale=0.1)
    ids_w, wts_w, _ = P.moe_route(h.double(), wr.double(), b.double() if bias else None, k, norm, scaling)
    ids = torch.empty(M, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(M, k, device=DEV)
    K().moe_router(ids, wts, h.to(DEV), wr.to(DEV), b.to(DEV) if bias else None, norm, scaling)
    assert torch.equal(ids.cpu().long(), ids_w)
    assert err(wts, wts_w) < 1e-5
    offs = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    sp = torch.empty(M * k, dtype=torch.int32, device=DEV)
    pr = torch.empty(M * k, dtype=torch.int32, device=DEV)
    K().moe_align(offs, sp, pr, ids, E)
    flat = ids_w.reshape(-1)
    order = torch.sort(flat, stable=True).indices              # stable in the pair index
    assert torch.equal(sp.cpu().long(), order)
    assert torch.equal(offs.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), torch.bincount(flat, minlength=E).cumsum(0)]))
    assert torch.equal(pr.cpu().long()[order], torch.arange(M * k))
    ys = gen(M * k, D, seed=93)
    x = gen(M, D, seed=94).to(DEV)
    x0 = x.cpu().double()
    K().moe_combine(x, ys.to(DEV), pr, wts, True)
    want = x0 + (wts_w[:, :, None] * ys.double()[pr.cpu().long().view(M, k)]).sum(1)
    assert err(x, want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,k,D", [(32, 4, 2048), (8, 2, 104), (5, 1, 72), (64, 6, 520)])
def test_moe_router_gives_a_row_the_same_bits_whatever_the_step(dtype, E, k, D):
    """The router has a form for single rows and one for four rows per block (many rows): a row's
    experts and weights are the same bits in both, so that a token is routed the same way alone, in a
    decode batch and inside a prompt."""
    M = 700
    h = gen(M, D, seed=97, dtype=dtype).to(DEV)
    wr, b = gen(E, D, seed=98, scale=0.3).to(DEV), gen(E, seed=99, scale=0.1).to(DEV)
    def route(rows):
        ids = torch.empty(rows.shape[0], k, dtype=torch.int32, device=DEV)
        wts = torch.empty(rows.shape[0], k, device=DEV)
        K().moe_router(ids, wts, rows, wr, b, True, 1.5)
        return ids, wts
    all_ids, all_w = route(h)                                  # many rows: four per block
    some_ids, some_w = route(h[:200].contiguous())
    assert torch.equal(some_ids, all_ids[:200]) and torch.equal(some_w, all_w[:200])
    for lo in (0, 199, 693):
        one_ids, one_w = route(h[lo:lo + 7].contiguous())      # a row per block
        assert torch.equal(one_ids, all_ids[lo:lo + 7]) and torch.equal(one_w, all_w[lo:lo + 7])
    want_ids, want_w, _ = P.moe_route(h.double().cpu(), wr.double().cpu(), b.double().cpu(), k, True, 1.5)
    agree = (all_ids.cpu().long() == want_ids).all(dim=1)
    assert agree.float().mean() > 0.97                        # the rest: near-ties at float rounding
    assert err(all_w[agree.to(DEV)], want_w[agree]) < 1e-5


# ---- sampling ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("V", [256, 1000, 65536])
def test_argmax_and_sampling(V):
    n = 6
    logits = gen(n, V, seed=95, scale=3.0)
    logits[2, 17] = logits[2, 400 % V] = logits[2].max() + 1       # a tie: the lower id wins
    if V >= 4096:
        # a row laid out against the kernel's quick way: the largest values all fall to the same few
        # threads (ids that are equal modulo 1024), so thousands of values reach the bound it takes
        # from the threads' maxima and it has to select over the whole row
        order = torch.argsort(logits[5], descending=True)
        ids = torch.arange(V)
        place = (ids % 1024) * (V // 1024) + ids // 1024            # rank of id i in that layout
        logits[5] = logits[5][order][place]
    ld = logits.to(DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    K().argmax(out, ld)
    assert out.cpu().tolist() == [int(np.argmax(r)) for r in logits.numpy()]
    for temperature, top_k, top_p, min_p in ((0.8, 40, 0.95, 0.0), (1.3, 0, 1.0, 0.05), (0.5, 500, 0.5, 0.0), (1.0, 1, 0.0, 0.0)):
        for trial in range(4):
            u = np.random.default_rng(trial).random(n).astype(np.float32)
            K().sample(out, ld, torch.from_numpy(u).to(DEV), top_k, temperature, top_p, min_p)
            want = [P.sample(logits[i].numpy(), temperature, top_k, top_p, min_p, float(u[i])) for i in range(n)]
            assert out.cpu().tolist() == want, (temperature, top_k, top_p, min_p, trial)


def test_penalties():
    V = 50
    logits = gen(2, V, seed=96)
    hist = torch.zeros(2, 256, dtype=torch.int32)
    hist[0, :4] = torch.tensor([3, 7, 3, 9])
    ln = torch.tensor([4, 0], dtype=torch.int32)
    want = logits.clone()
    for t in [3, 7, 3, 9]:
        v = want[0, t]
        want[0, t] = (v / 1.3 if v > 0 else v * 1.3) - 0.2
    ld = logits.to(DEV)
    K().penalties(ld, hist.to(DEV), ln.to(DEV), 1.3, 0.2)
    assert err(ld, want) < 1e-6


# ---- the tcgen05 matrix product ------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (128, 256, 128), (65, 48, 72), (200, 100, 200), (300, 520, 136),
                                    (2048, 2048, 2048), (513, 6144, 2048), (1000, 2048, 5632),
                                    (17, 2048, 256), (64, 352, 128), (100, 6144, 64), (33, 11264, 192)])
def test_linear_tc(M, N, K_):
    """Tensor-memory accumulation against float64, at tile-aligned sizes and at sizes where rows,
    columns and k all run past the last tile; store, add-to-residual, and both result types."""
    x, w = gen(M, K_, seed=100, dtype=torch.bfloat16), gen(N, K_, seed=101, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    assert K().linear_tc(out, x.to(DEV), w.to(DEV))
    K().check_device_status()
    assert err(out, want) < 2e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear_tc(ob, x.to(DEV), w.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=102).to(DEV)
    b0 = base.clone()
    K().linear_tc(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    K().check_device_status()
    assert err(base, b0.cpu().double() + want) < 2e-5


@pytest.mark.parametrize("M,N,K_", [(300, 2048, 4096), (512, 2048, 5632), (200, 3072, 8192), (130, 264, 6080), (257, 1000, 4104)])
def test_linear_tc_with_k_in_slices(M, N, K_):
    """Products of a few hundred rows with a long K (prompts of that length, the down projection):
    fewer 128 x 256 tiles than SMs, so K is cut into slices whose partial tiles a second kernel adds
    up.  Store, add to the residual and SwiGLU against float64; a last slice with fewer k-blocks,
    rows and columns past the tiles."""
    from lastengine_b200.parts.ffn import fuse_gate_up
    assert K().lib().leb_gemm_bf16_tc_slices(M, N, K_) > 1
    x, w = gen(M, K_, seed=110, dtype=torch.bfloat16), gen(N, K_, seed=111, scale=0.05, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    assert K().linear_tc(out, x.to(DEV), w.to(DEV))
    assert err(out, want) < 2e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear_tc(ob, x.to(DEV), w.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=112).to(DEV)
    b0 = base.clone()
    K().linear_tc(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    assert err(base, b0.cpu().double() + want) < 2e-5
    again = b0.clone()
    K().linear_tc(again, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    assert torch.equal(again, base)                  # the slices are added in a fixed order
    if N % 32 == 0:
        F = N // 2
        o2 = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
        K().linear_tc(o2, x.to(DEV), fuse_gate_up(w[:F], w[F:], True).to(DEV), K().SWIGLU)
        assert err(o2, P.silu(want[:, :F]) * want[:, F:]) < 6e-3
    K().check_device_status()


@pytest.mark.parametrize("M,F,D", [(128, 64, 64), (70, 16, 40), (300, 160, 96), (2048, 5632, 2048), (40, 5632, 128), (64, 1024, 64)])
def test_linear_tc_swiglu_epilogue(M, F, D):
    from lastengine_b200.parts.ffn import fuse_gate_up
    x = gen(M, D, seed=103, dtype=torch.bfloat16)
    w1, w3 = gen(F, D, seed=104, scale=0.05, dtype=torch.bfloat16), gen(F, D, seed=105, scale=0.05, dtype=torch.bfloat16)
    want = P.silu(x.double() @ w1.double().T) * (x.double() @ w3.double().T)
    w13 = fuse_gate_up(w1, w3, True).to(DEV)
    out = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    assert K().linear_tc(out, x.to(DEV), w13, K().SWIGLU)
    K().check_device_status()
    assert err(out, want) < 6e-3


def test_linear_tc_strided_operand_and_small_kernel_agree():
    """A column slice as the left operand (row stride larger than its width), and agreement with the
    weight-streaming kernel on the same product."""
    M, N, K_ = 150, 96, 128
    big = gen(M, 3 * K_, seed=106, dtype=torch.bfloat16).to(DEV)
    x = big[:, K_:2 * K_]
    w = gen(N, K_, seed=107, dtype=torch.bfloat16).to(DEV)
    a = torch.empty(M, N, device=DEV)
    b = torch.empty(M, N, device=DEV)
    assert K().linear_tc(a, x, w)
    K().lib().leb_gemm_bf16_small(b.data_ptr(), 0, x.data_ptr(), w.data_ptr(), M, N, K_, x.stride(0), N, 0, None, 1, 0, M,
                                  torch.cuda.current_stream().cuda_stream)
    assert err(a, x.double().cpu() @ w.double().cpu().T) < 2e-5
    assert err(a, b) < 2e-6


def test_shortconv_kernels_against_the_references_own():
    """The engine's convolution kernels (rows + state, and the one-launch decode form) on the inputs
    of tests/golden/shortconv_golden.npz, which holds what the reference's kernels gave."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "shortconv_golden.npz"))
    for case in range(3):
        bcx, w = torch.from_numpy(g[f"bcx{case}"]), torch.from_numpy(g[f"w{case}"])
        T, n, lc = bcx.shape[0], w.shape[0], w.shape[1]
        for mode in ("chunk", "steps"):
            state = torch.zeros(3, n, lc - 1, device=DEV)
            state[2] = torch.from_numpy(g[f"state_in{case}"]).to(DEV)
            y = torch.empty(T, n, device=DEV)
            bb = builder()
            if mode == "chunk":
                K().shortconv(y, bcx.to(DEV), w.to(DEV), None, state, bb.build([2], [[0] * T], [0], [], {}), lc)
            else:
                for t in range(T):
                    K().shortconv(y[t:t + 1], bcx[t:t + 1].to(DEV), w.to(DEV), None, state, bb.build([2], [[0]], [t], [], {}), lc)
            assert err(y, torch.from_numpy(g[f"y{case}"])) < 1e-6, (case, mode)
            assert err(state[2], torch.from_numpy(g[f"state_out{case}"])) < 1e-6, (case, mode)


@pytest.mark.parametrize("M,N,K_", [(256, 256, 64), (300, 520, 136), (129, 100, 72), (1000, 2048, 5632), (2048, 6144, 2048)])
def test_linear_tc_pairs(M, N, K_):
    """The product on pairs of SMs (cta_group::2, 256 x 256 tiles): tile-aligned sizes and sizes where
    rows, columns and k run past the last tile; store, add to the residual, SwiGLU, both result types."""
    x, w = gen(M, K_, seed=100, dtype=torch.bfloat16), gen(N, K_, seed=101, scale=0.05, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    assert K().linear_tc2(out, x.to(DEV), w.to(DEV))
    K().check_device_status()
    assert err(out, want) < 2e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear_tc2(ob, x.to(DEV), w.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=102).to(DEV)
    b0 = base.clone()
    K().linear_tc2(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    assert err(base, b0.cpu().double() + want) < 2e-5
    if N % 32 == 0:
        from lastengine_b200.parts.ffn import fuse_gate_up
        F = N // 2
        w13 = fuse_gate_up(w[:F], w[F:], True).to(DEV)
        o2 = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
        K().linear_tc2(o2, x.to(DEV), w13, K().SWIGLU)
        assert err(o2, P.silu(want[:, :F]) * want[:, F:]) < 6e-3
    K().check_device_status()


@pytest.mark.parametrize("M,N,K_", [(17, 2048, 2048), (64, 352, 128), (100, 6144, 64), (33, 11264, 192), (128, 100, 200),
                                    (1, 128, 64), (16, 48, 72), (48, 2048, 5632), (64, 65536, 256),
                                    (65, 2048, 2048), (96, 352, 5632), (90, 100, 200), (97, 6144, 136)])
def test_linear_skinny(M, N, K_):
    """The swapped-operand tcgen05 product with K sliced over blocks: store, add to residual, both
    result types, sizes that leave partial tiles and slices."""
    x, w = gen(M, K_, seed=120, dtype=torch.bfloat16), gen(N, K_, seed=121, scale=0.05, dtype=torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    assert K().linear_skinny(out, x.to(DEV), w.to(DEV))
    K().check_device_status()
    assert err(out, want) < 2e-5
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    K().linear_skinny(ob, x.to(DEV), w.to(DEV))
    assert err(ob, want) < 5e-3
    base = gen(M, N, seed=122).to(DEV)
    b0 = base.clone()
    K().linear_skinny(base, x.to(DEV), w.to(DEV), K().ACCUMULATE)
    K().check_device_status()
    assert err(base, b0.cpu().double() + want) < 2e-5


@pytest.mark.parametrize("M,F,D", [(64, 5632, 2048), (20, 16, 40), (100, 160, 96), (80, 5632, 2048), (96, 160, 96)])
def test_linear_skinny_swiglu(M, F, D):
    from lastengine_b200.parts.ffn import fuse_gate_up
    x = gen(M, D, seed=123, dtype=torch.bfloat16)
    w1, w3 = gen(F, D, seed=124, scale=0.05, dtype=torch.bfloat16), gen(F, D, seed=125, scale=0.05, dtype=torch.bfloat16)
    want = P.silu(x.double() @ w1.double().T) * (x.double() @ w3.double().T)
    out = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    assert K().linear_skinny(out, x.to(DEV), fuse_gate_up(w1, w3, True).to(DEV), K().SWIGLU)
    K().check_device_status()
    assert err(out, want) < 6e-3

