"""Build the sm_100a shared library in-tree with nvcc (no GPU needed to compile)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmegaattn_b200.so")
# Same sources with -DMA_AUDIT: the scheduler counts every finished unit of work (tests
# assert exactly-once execution with it).  Kept out of the product build because even a
# never-taken branch in the scheduler role shifts the attention loop's code generation
# (measured: +1.2 % on the attention stage).
LIB_AUDIT = os.path.join(HERE, "libmegaattn_b200_audit.so")
SOURCES = ["fused_prefill.cu", "cabi.cu", "noalloc.cu", "residual_rmsnorm.cu", "rope.cu"]
HEADERS = ["ptx.cuh", "kparams.h", os.path.join("..", "..", "include", "megaattn_b200.h")]


def _stale(lib: str = None) -> bool:
    lib = lib or LIB
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, audit: bool = False) -> str:
    """Compile ``csrc/*.cu`` into ``libmegaattn_b200.so`` (or, with ``audit``, into
    ``libmegaattn_b200_audit.so``) next to this file."""
    LIB = LIB_AUDIT if audit else globals()["LIB"]
    if not force and not _stale(LIB):
        return LIB
    # Several processes (one per GPU under torchrun) may get here at once: one builds, into a
    # temporary file that is renamed over the library in one step, the others wait on the
    # lock and find the library fresh.
    import fcntl
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not _stale(LIB):
            return LIB
        nvcc = os.environ.get("NVCC", "nvcc")
        tmp = f"{LIB}.{os.getpid()}.tmp"
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
               "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", tmp]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        if audit:
            cmd += ["-DMA_AUDIT"]
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
    print(build(force=True, audit=True))
