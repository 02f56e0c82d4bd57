"""Ahead-of-time build of libtarafer_b200.so for sm_100a (no JIT at run time).

The reference compiles its kernels with NVRTC when a model is loaded
(crates/core/src/cuda/device.rs:96-122); this library ships compiled sm_100a code instead.
The compile options mirror the reference's NVRTC options (fast math, flush-to-zero,
approximate division and square root, fused multiply-add) so that identical expressions
lower to identical instructions.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libtarafer_b200.so"
SOURCES = [CSRC / "tfr_engine.cu", CSRC / "tfr_gguf.cpp"]
HEADERS = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "tarafer_b200.h"]

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-shared"]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library in-tree if sources are newer than the binary."""
    if not force and not is_stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIB), *map(str, SOURCES)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    env = dict(os.environ)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
