"""Makes tests/golden/dense_kernels_golden.npz from the reference's own CUDA kernels.

The reference's model code is Rust and cannot be built here, but the kernels of its dense GPU path
are plain CUDA C.  This script takes the text of `rmsnorm` and `swiglu_gu` (src/cuda/kernels.cu:409-417,
:430) and of `dn_prep`, `dn_cvt_half` and `dn_attn` (src/cuda/dense.cu:3-28, :94-123) with the three
one-line helpers they call (`warp_sum`, `silu_f`, `sigm_f`, src/cuda/kernels.cu:7-9) UNCHANGED out of a
reference checkout given on the command line (nothing of it is stored in this repository), adds a
few host functions that launch them, compiles that with nvcc for the GPU at hand, runs them once
on seeded random inputs of tiny sizes and stores inputs and outputs.  tests/test_plain.py checks the
plain implementation's norm, SwiGLU, rotation (both pairings, part of the head, frequency
factors) and attention (norm before rotation, kv-head mapping, window edge, head gate, scale)
against the stored numbers.  The kernels have no waits or flags; every launch is a few blocks.

    python tests/golden/make_dense_kernels_golden.py PATH_TO_REFERENCE_CHECKOUT [OUT.npz]
"""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HOST = r"""
#define CHECKED(call) do { call; cudaError_t e_ = cudaDeviceSynchronize(); if (e_ != cudaSuccess) return (int)e_; } while (0)
extern "C" int run_rmsnorm(const float* x, const float* w, float* o, int rows, int n, float eps) {
  for (int r = 0; r < rows; r++) rmsnorm<<<1, 256>>>(x + (size_t)r * n, w, o + (size_t)r * n, n, eps);
  CHECKED((void)0);
  return 0;
}
extern "C" int run_swiglu_gu(const float* gu, float* o, int ffn, int tokens) {
  int n = ffn * tokens;
  CHECKED((swiglu_gu<<<(n + 255) / 256, 256>>>(gu, o, ffn, n)));
  return 0;
}
// heads x tokens blocks; token t is rotated for position pos0 + t
extern "C" int run_prep(const float* in, void* out, int out_half, int heads, int tokens, int hd, int rope_dim, int pos0,
                        float base, const float* ff, int neox, const float* nw, float eps) {
  CHECKED((dn_prep<<<dim3(heads, tokens), 64>>>(in, out, out_half, hd, rope_dim, pos0, base, ff, neox, nw, eps, nullptr, 0)));
  return 0;
}
extern "C" int run_cvt_half(const float* in, void* out, int n) {
  CHECKED((dn_cvt_half<<<(n + 255) / 256, 256>>>(in, (__half*)out, n)));
  return 0;
}
// row y of q sees keys 0 .. n0 + y - 1 of the cache
extern "C" int run_attn(const float* q, const void* kc, const void* vc, const float* gate, float* o, int win, int n0,
                        int nh, int nkv, int hd, int rows) {
  CHECKED((dn_attn<<<dim3(nh, rows), 256>>>(q, (const __half*)kc, (const __half*)vc, gate, o, win, n0, nh, nkv, hd, nullptr)));
  return 0;
}
"""


def block_text(src: str, start_pattern: str) -> str:
    """The definition that starts at `start_pattern`, up to its closing brace."""
    m = re.search(start_pattern, src)
    if m is None:
        raise RuntimeError(f"not found in the reference: {start_pattern}")
    depth, i = 0, src.index("{", m.start())
    for j in range(i, len(src)):
        depth += {"{": 1, "}": -1}.get(src[j], 0)
        if depth == 0:
            return src[m.start():j + 1]
    raise RuntimeError(start_pattern)


def build(ref: str, workdir: str):
    kern = open(os.path.join(ref, "src", "cuda", "kernels.cu")).read()
    dense = open(os.path.join(ref, "src", "cuda", "dense.cu")).read()
    helper = lambda name: block_text(kern, r"__device__ __forceinline__ float " + name + r"\(")
    kernel = lambda src, name: block_text(src, r'extern "C" __global__ void ' + name + r"\(")
    code = "\n".join(["#include <cuda_fp16.h>", "#include <cuda_runtime.h>", "#define FULL 0xffffffffu",
                      helper("warp_sum"), helper("silu_f"), helper("sigm_f"),
                      kernel(kern, "rmsnorm"), kernel(kern, "swiglu_gu"),
                      kernel(dense, "dn_prep"), kernel(dense, "dn_cvt_half"), kernel(dense, "dn_attn"), HOST])
    cu, so = os.path.join(workdir, "ref_kernels.cu"), os.path.join(workdir, "ref_kernels.so")
    open(cu, "w").write(code)
    subprocess.check_call(["nvcc", "-O2", "-arch=native", "-shared", "-Xcompiler", "-fPIC", "-o", so, cu])
    return ctypes.CDLL(so)


def main(ref: str, out_path: str) -> None:
    import torch
    dev = "cuda:0"
    f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    out = {}
    with tempfile.TemporaryDirectory() as d:
        lib = build(ref, d)
        for fn in (lib.run_rmsnorm, lib.run_swiglu_gu, lib.run_prep, lib.run_cvt_half, lib.run_attn):
            fn.restype = ctypes.c_int
        I, F = ctypes.c_int, ctypes.c_float

        def ok(rc, what):
            if rc != 0:
                raise RuntimeError(f"{what}: CUDA error {rc}")

        # ---- RMSNorm: widths that are no power of two, two eps ----
        for case, (rows, n, eps) in enumerate([(3, 72, 1e-5), (2, 200, 1e-6), (1, 1000, 1e-5)]):
            rng = np.random.default_rng(200 + case)
            x, w = f32(rng.standard_normal((rows, n)) * 3), f32(1 + 0.2 * rng.standard_normal(n))
            o = torch.empty_like(x)
            ok(lib.run_rmsnorm(ptr(x), ptr(w), ptr(o), I(rows), I(n), F(eps)), "rmsnorm")
            out.update({f"norm_x{case}": x.cpu().numpy(), f"norm_w{case}": w.cpu().numpy(),
                        f"norm_eps{case}": np.float64(eps), f"norm_y{case}": o.cpu().numpy()})
        # ---- SwiGLU over [gate | up] rows ----
        rng = np.random.default_rng(210)
        gu = f32(rng.standard_normal((5, 2 * 40)) * 2.5)
        o = torch.empty(5, 40, device=dev)
        ok(lib.run_swiglu_gu(ptr(gu), ptr(o), I(40), I(5)), "swiglu_gu")
        out.update({"swiglu_gu": gu.cpu().numpy(), "swiglu_y": o.cpu().numpy()})
        # ---- per-head norm + rotation: (heads, hd, rope_dim, split-half?, factors?, norm?, base, pos0, tokens) ----
        prep_cases = [(3, 32, 32, 1, 0, 1, 10000.0, 0, 16), (2, 64, 32, 1, 0, 1, 1e6, 7, 12), (2, 32, 32, 0, 0, 1, 10000.0, 3, 9),
                      (2, 64, 64, 1, 1, 1, 5e4, 30, 12), (2, 32, 16, 0, 1, 0, 100.0, 1, 6)]
        for case, (heads, hd, rd, neox, with_ff, with_norm, base, pos0, T) in enumerate(prep_cases):
            rng = np.random.default_rng(220 + case)
            x = f32(rng.standard_normal((T, heads, hd)))
            nw = f32(1 + 0.2 * rng.standard_normal(hd)) if with_norm else None
            ff = f32(1 + 7 * rng.random(rd // 2)) if with_ff else None
            o = torch.empty_like(x)
            ok(lib.run_prep(ptr(x), ptr(o), I(0), I(heads), I(T), I(hd), I(rd), I(pos0), F(base), ptr(ff), I(neox), ptr(nw),
                            F(1e-5)), "dn_prep")
            out.update({f"prep_x{case}": x.cpu().numpy(), f"prep_y{case}": o.cpu().numpy(),
                        f"prep_meta{case}": np.array([heads, hd, rd, neox, pos0, T], dtype=np.int64),
                        f"prep_base{case}": np.float64(base)})
            if with_norm:
                out[f"prep_nw{case}"] = nw.cpu().numpy()
            if with_ff:
                out[f"prep_ff{case}"] = ff.cpu().numpy()
        # ---- the attention chain of a prompt: norm + rotation of q (float) and k (half, the cache), v to half,
        #      then row t over keys 0..t: (nh, nkv, hd, rope_dim, window, gate?, factors?, base, T) ----
        attn_cases = [(4, 2, 32, 32, 0, 0, 0, 10000.0, 20), (6, 2, 64, 64, 0, 1, 0, 1e6, 14), (4, 4, 32, 16, 8, 1, 0, 10000.0, 20),
                      (8, 2, 64, 64, 13, 0, 1, 5e4, 18), (3, 1, 32, 32, 0, 1, 1, 100.0, 1)]
        for case, (nh, nkv, hd, rd, win, with_gate, with_ff, base, T) in enumerate(attn_cases):
            rng = np.random.default_rng(240 + case)
            q, k, v = (f32(rng.standard_normal((T, n, hd)) * s) for n, s in ((nh, 1.5), (nkv, 1.5), (nkv, 1.0)))
            qn, kn = f32(1 + 0.2 * rng.standard_normal(hd)), f32(1 + 0.2 * rng.standard_normal(hd))
            gate = f32(rng.standard_normal((T, nh)) * 2) if with_gate else None
            ff = f32(1 + 7 * rng.random(rd // 2)) if with_ff else None
            qr = torch.empty_like(q)
            kc = torch.empty(T, nkv, hd, dtype=torch.float16, device=dev)
            vc = torch.empty(T, nkv, hd, dtype=torch.float16, device=dev)
            ok(lib.run_prep(ptr(q), ptr(qr), I(0), I(nh), I(T), I(hd), I(rd), I(0), F(base), ptr(ff), I(1), ptr(qn), F(1e-5)), "dn_prep q")
            ok(lib.run_prep(ptr(k), ptr(kc), I(1), I(nkv), I(T), I(hd), I(rd), I(0), F(base), ptr(ff), I(1), ptr(kn), F(1e-5)), "dn_prep k")
            ok(lib.run_cvt_half(ptr(v), ptr(vc), I(T * nkv * hd)), "dn_cvt_half")
            o = torch.empty(T, nh, hd, device=dev)
            ok(lib.run_attn(ptr(qr), ptr(kc), ptr(vc), ptr(gate), ptr(o), I(win), I(1), I(nh), I(nkv), I(hd), I(T)), "dn_attn")
            out.update({f"attn_q{case}": q.cpu().numpy(), f"attn_k{case}": k.cpu().numpy(), f"attn_v{case}": v.cpu().numpy(),
                        f"attn_qn{case}": qn.cpu().numpy(), f"attn_kn{case}": kn.cpu().numpy(), f"attn_o{case}": o.cpu().numpy(),
                        f"attn_meta{case}": np.array([nh, nkv, hd, rd, win, T], dtype=np.int64),
                        f"attn_base{case}": np.float64(base)})
            if with_gate:
                out[f"attn_gate{case}"] = gate.cpu().numpy()
            if with_ff:
                out[f"attn_ff{case}"] = ff.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays, {os.path.getsize(out_path)} bytes")


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else os.path.join(here, "dense_kernels_golden.npz"))
