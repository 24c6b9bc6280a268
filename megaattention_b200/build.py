"""Build the sm_100a shared library in-tree with nvcc (no GPU needed to compile)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmegaattn_b200.so")
SOURCES = ["fused_prefill.cu", "cabi.cu", "noalloc.cu"]
HEADERS = ["ptx.cuh", "kparams.h", os.path.join("..", "..", "include", "megaattn_b200.h")]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc/*.cu`` into ``libmegaattn_b200.so`` next to this file."""
    if not force and not _stale():
        return LIB
    # Several processes (one per GPU under torchrun) may get here at once: one builds, into a
    # temporary file that is renamed over the library in one step, the others wait on the
    # lock and find the library fresh.
    import fcntl
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not _stale():
            return LIB
        nvcc = os.environ.get("NVCC", "nvcc")
        tmp = f"{LIB}.{os.getpid()}.tmp"
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
               "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", tmp]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += [os.path.join(CSRC, f) for f in SOURCES]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        os.replace(tmp, LIB)
        if verbose:
            sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
