"""Makes tests/golden/shortconv_golden.npz from the reference's own short-convolution kernels.

The reference is Rust plus CUDA and cannot be built here, but the bodies of its two
short-convolution kernels (`dn_shortconv`, one token; `dn_shortconv_b`, a chunk of tokens;
src/cuda/dense.cu:124-148) are plain C.  This script takes their text out of the reference
checkout given on the command line (nothing of it is stored in this repository), puts a few
lines in front that stand in for the CUDA built-ins, compiles that with g++, runs both kernels
on seeded random inputs and stores inputs and outputs.  tests/test_plain.py checks the plain
implementation's convolution against the stored numbers.

    python tests/golden/make_shortconv_golden.py PATH_TO_REFERENCE_CHECKOUT
"""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

SHIM = r"""
#include <cstddef>
struct Dim3 { int x, y, z; };
static Dim3 blockIdx, blockDim, threadIdx;
#define __global__
"""
DRIVER = r"""
extern "C" void run_step(const float* bcx, const float* w, float* st, float* y, int n, int lc) {
  blockDim = {128, 1, 1};
  for (int b = 0; b * 128 < n; b++) for (int t = 0; t < 128; t++) { blockIdx = {b, 0, 0}; threadIdx = {t, 0, 0}; dn_shortconv(bcx, w, st, y, n, lc); }
}
extern "C" void run_chunk(const float* bcx, const float* w, float* st, float* y, int n, int lc, int T) {
  blockDim = {128, 1, 1};
  for (int b = 0; b * 128 < n; b++) for (int t = 0; t < 128; t++) { blockIdx = {b, 0, 0}; threadIdx = {t, 0, 0}; dn_shortconv_b(bcx, w, st, y, n, lc, T); }
}
"""


def kernel_text(src: str, name: str) -> str:
    m = re.search(r'extern "C" __global__ void ' + name + r"\(", src)
    depth, i = 0, src.index("{", m.start())
    for j in range(i, len(src)):
        depth += {"{": 1, "}": -1}.get(src[j], 0)
        if depth == 0:
            return src[m.start():j + 1]
    raise RuntimeError(name)


def main(ref: str) -> None:
    src = open(os.path.join(ref, "src", "cuda", "dense.cu")).read()
    code = SHIM + kernel_text(src, "dn_shortconv") + "\n" + kernel_text(src, "dn_shortconv_b") + "\n" + DRIVER
    with tempfile.TemporaryDirectory() as d:
        cpp, so = os.path.join(d, "k.cpp"), os.path.join(d, "k.so")
        open(cpp, "w").write(code)
        subprocess.check_call(["g++", "-O1", "-shared", "-fPIC", "-o", so, cpp])
        lib = ctypes.CDLL(so)
        fp = ctypes.POINTER(ctypes.c_float)
        out = {}
        for case, (n, lc, T) in enumerate([(6, 3, 9), (10, 4, 7), (5, 2, 4)]):
            rng = np.random.default_rng(100 + case)
            bcx = rng.standard_normal((T, 3 * n)).astype(np.float32)
            w = rng.standard_normal((n, lc)).astype(np.float32)
            st0 = rng.standard_normal((n, lc - 1)).astype(np.float32)        # a non-zero starting state
            y_chunk, st_chunk = np.zeros((T, n), np.float32), st0.copy()
            lib.run_chunk(bcx.ctypes.data_as(fp), w.ctypes.data_as(fp), st_chunk.ctypes.data_as(fp),
                          y_chunk.ctypes.data_as(fp), n, lc, T)
            y_step, st_step = np.zeros((T, n), np.float32), st0.copy()
            for t in range(T):
                lib.run_step(bcx[t].ctypes.data_as(fp), w.ctypes.data_as(fp), st_step.ctypes.data_as(fp),
                             y_step[t].ctypes.data_as(fp), n, lc)
            assert np.array_equal(y_chunk, y_step) and np.array_equal(st_chunk, st_step)
            out.update({f"bcx{case}": bcx, f"w{case}": w, f"state_in{case}": st0, f"y{case}": y_chunk,
                        f"state_out{case}": st_chunk})
        np.savez(os.path.join(os.path.dirname(os.path.abspath(__file__)), "shortconv_golden.npz"), **out)
        print("wrote shortconv_golden.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
