"""Ahead-of-time build of libtarafer_b200.so and its instrumented twin for sm_100a (no JIT at run time).

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
LIB = PKG / "libtarafer_b200.so"            # the product: decode path, loader, operators, read-only taps
AIDS_LIB = PKG / "libtarafer_b200_aids.so"  # the same sources with -DTFR_TEST_AIDS: timeline probes, integer taps, quantiser
SOURCES = [CSRC / "tfr_engine.cu", CSRC / "tfr_gguf.cpp"]
HEADERS = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "tarafer_b200.h"]

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-shared"]


def is_stale() -> bool:
    for lib in (LIB, AIDS_LIB):
        if not lib.exists():
            return True
        t = lib.stat().st_mtime
        if any(p.stat().st_mtime > t for p in SOURCES + HEADERS):
            return True
    return False


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile both libraries in-tree (side by side) if sources are newer than the binaries."""
    if not force and not is_stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    procs = []
    for lib, extra in ((LIB, []), (AIDS_LIB, ["-DTFR_TEST_AIDS"])):
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-o", str(lib), *map(str, SOURCES)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((lib, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=dict(os.environ))))
    for lib, pr in procs:
        out, err = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed for {lib.name}:\n" + out + err)
        if verbose:
            print(err)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
