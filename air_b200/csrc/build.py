"""Compiles the CUDA sources of this folder for sm_100a into one shared library and loads
it with ctypes.  There is no fallback: without nvcc, or if a source does not compile, the
import fails with the compiler's message.

The library is built at the first call that needs it, into ``_build/`` beside the sources
(or into $AIR_B200_BUILD_DIR, or a per-user temporary folder if the package folder cannot
be written).  A stamp of the sources' contents and the flags decides whether it is rebuilt.
Each translation unit is compiled by its own nvcc process, a few at a time, and a line is
printed for each that starts and ends, so that a first call does not look hung.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# --use_fast_math is never given: expf, rsqrtf and divisions keep their accurate forms.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
LIB_NAME = "libair_b200_kernels.so"

_lib = None


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("air_b200: nvcc was not found (set NVCC or add it to PATH); the CUDA kernels "
                       "cannot be built and there is no other implementation")


def _stamp() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("AIR_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(HERE, "_build")
    if _writable(local):
        return local
    alt = os.path.join(tempfile.gettempdir(), f"air_b200_build_{os.getuid()}")
    os.makedirs(alt, exist_ok=True)
    return alt


def _say(msg: str) -> None:
    print(f"[air_b200 build] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = False) -> str:
    """Builds the library if its stamp is stale; returns its path."""
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp_file = os.path.join(out_dir, "stamp.txt")
    stamp = _stamp()
    if not force and os.path.exists(lib) and os.path.exists(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    nvcc = _nvcc()
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir}")
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
              ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        t = time.time()
        _say(f"  nvcc {src} ...")
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"air_b200: nvcc failed on {src}:\n{p.stdout}")
        if verbose and p.stdout:
            print(p.stdout, file=sys.stderr)
        _say(f"  nvcc {src} done in {time.time() - t:.1f} s")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = lib + f".tmp{os.getpid()}"
    p = subprocess.run([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs + ["-lcudart"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"air_b200: linking {LIB_NAME} failed:\n{p.stdout}")
    os.replace(tmp, lib)
    with open(stamp_file, "w") as f:
        f.write(stamp + "\n")
    _say(f"built {LIB_NAME} in {time.time() - t0:.1f} s")
    return lib


def library() -> ctypes.CDLL:
    """The loaded library (built first if needed)."""
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib
