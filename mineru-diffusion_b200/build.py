"""Builds libmdb200.so (sm_100a only) next to this file with nvcc.

Run as ``python mineru-diffusion_b200/build.py`` or call :func:`build`.
nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "libmdb200.cu")
OUT = os.path.join(HERE, "libmdb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-diag-suppress", "550",
]


def _sources() -> list[str]:
    out = [os.path.join(HERE, "..", "include", "mdb200.h")]
    csrc = os.path.join(HERE, "csrc")
    for name in sorted(os.listdir(csrc)):
        if name.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(csrc, name))
    return out


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    return any(os.path.getmtime(p) > built for p in _sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if sources are newer than the binary; returns its path."""
    if not force and not is_stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libmdb200.so cannot be built on this machine")
    cmd = [nvcc, *NVCC_FLAGS]
    if os.environ.get("MDB_TRACE") == "1":      # timeline stamps in the kernels (mdb_set_trace); off: compiled out
        cmd += ["-DMDB_TRACE"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", OUT, SRC]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
