"""Compile the CUDA library in-tree for B200 (sm_100a).

    python -m flash_colsum_b200.build [--force]

The shared library lands in ``flash_colsum_b200/_lib/`` next to the sources; it is
loaded with ctypes and never installed into site-packages.  nvcc cross-compiles,
so this works on a machine without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libflash_colsum_b200.so")
SOURCES = [os.path.join(CSRC, "flash_colsum_sm100.cu")]
HEADERS = [os.path.join(CSRC, "sm100_ptx.cuh"), os.path.join(CSRC, "schedule.h"),
           os.path.join(CSRC, "colsum_small_q.cuh"), os.path.join(CSRC, "colsum_math.cuh"),
           os.path.join(CSRC, "colsum_single_pass.cuh"), os.path.join(CSRC, "select_topk.cuh"),
           os.path.join(CSRC, "colsum_fused_short.cuh"),
           os.path.join(os.path.dirname(PKG), "include", "flash_colsum_b200.h")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > built for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build if missing or older than its sources; returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    # Several processes may get here at once (one rank per GPU): one of them builds, into a
    # file of its own that is renamed over the library when complete, the others wait for the
    # lock and find the library fresh.  Nobody can open a half-written file.
    import fcntl
    with open(os.path.join(LIB_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():
                return LIB_PATH
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            cmd = [find_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp] + SOURCES
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
            os.replace(tmp, LIB_PATH)
            if verbose:
                print(res.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
