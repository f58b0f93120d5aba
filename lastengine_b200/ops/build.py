"""Builds the kernels under csrc/ into one shared library for sm_100a and loads it.

The library sits in the package (`lastengine_b200/_lib/`), so a built tree carries it along.
In a fresh checkout the first call compiles it (a line per file on stderr); where the package
folder cannot be written, a per-user folder under the temporary directory is used.  There is
no fallback without it: if it can be neither found nor built, loading raises.

The reference compiles its two .cu files at start-up with NVRTC for the device it finds
(src/gpu.rs:658-690, src/gpu/dense.rs:58-61); here nvcc runs ahead of time, or at first use.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
LIB_NAME = "libleb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _say(msg: str) -> None:
    print(f"[lastengine_b200] {msg}", file=sys.stderr, flush=True)


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()[:16]


def _find_nvcc() -> str:
    for cand in (os.environ.get("LEB200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError(
        "lastengine_b200: the CUDA kernels are not built and nvcc was not found (looked at "
        "$LEB200_NVCC, PATH and /usr/local/cuda/bin/nvcc); there is no path without them")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


def _lib_dirs() -> list[str]:
    dirs = [os.path.join(_PKG, "_lib")]
    dirs.append(os.path.join(tempfile.gettempdir(), f"lastengine_b200-{os.getuid()}", "_lib"))
    return dirs


def _up_to_date(d: str, digest: str) -> bool:
    stamp = os.path.join(d, "build.stamp")
    lib = os.path.join(d, LIB_NAME)
    try:
        with open(stamp) as f:
            return f.read().strip() == digest and os.path.isfile(lib)
    except OSError:
        return False


def _compile(d: str, digest: str, verbose: bool) -> None:
    nvcc = _find_nvcc()
    srcs = _sources()
    objdir = os.path.join(d, "obj")
    os.makedirs(objdir, exist_ok=True)
    t0 = time.time()
    _say(f"building {LIB_NAME} for sm_100a from {len(srcs)} files in {d} (first use; about a minute)")

    def one(i_src):
        i, src = i_src
        obj = os.path.join(objdir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"lastengine_b200: nvcc failed on {src}:\n{p.stdout}\n{p.stderr}")
        _say(f"  compiled {src} ({i + 1}/{len(srcs)}, {time.time() - t0:.0f}s)")
        if verbose and p.stderr:
            sys.stderr.write(p.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(one, enumerate(srcs)))
    tmp = os.path.join(d, f".{LIB_NAME}.{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"lastengine_b200: linking failed:\n{p.stdout}\n{p.stderr}")
    os.replace(tmp, os.path.join(d, LIB_NAME))
    with open(os.path.join(d, "build.stamp"), "w") as f:
        f.write(digest + "\n")
    _say(f"built in {time.time() - t0:.0f}s")


def build(force: bool = False, verbose: bool = False) -> str:
    """Makes sure the library exists and matches the sources; returns its path."""
    digest = _digest()
    if not force:
        for d in _lib_dirs():
            if _up_to_date(d, digest):
                return os.path.join(d, LIB_NAME)
    last_err: Exception | None = None
    for d in _lib_dirs():
        if not _writable_dir(d):
            continue
        lock = open(os.path.join(d, ".lock"), "w")
        try:
            fcntl.flock(lock, fcntl.LOCK_EX)
            if force or not _up_to_date(d, digest):
                _compile(d, digest, verbose)
            return os.path.join(d, LIB_NAME)
        except RuntimeError as e:
            last_err = e
            break
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            lock.close()
    if last_err:
        raise last_err
    raise RuntimeError("lastengine_b200: no writable folder for the kernel library "
                       f"(tried {', '.join(_lib_dirs())})")


_LIB: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = build()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise RuntimeError(f"lastengine_b200: cannot load {path}: {e}") from None
        _LIB.leb_last_error.restype = ctypes.c_char_p
    return _LIB
