"""In-tree build of libua_b200.so (sm_100a only) with nvcc.

    python -m universal_attention_triton_b200.build [--verbose]

The shared library is written next to this file so that it travels with the
source tree; there is no JIT cache and no pip install step.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libua_b200.so")
SOURCES = ["ua_api.cu"]
# developer micro-benchmark (stand-alone executable, not loaded by the package): `--tools` builds it next to the library
TOOL_SOURCE = "mma_timing.cu"
TOOL_PATH = os.path.join(PKG_DIR, "mma_timing.bin")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG_DIR), "include", "ua_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB_PATH, "-lcuda"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libua_b200.so")
    return LIB_PATH


def build_tools() -> str:
    """Compile the stand-alone MMA timing micro-benchmark (run it on a B200: ``./mma_timing.bin 256``)."""
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
           os.path.join(CSRC, TOOL_SOURCE), "-o", TOOL_PATH, "-lcuda"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building the MMA timing micro-benchmark")
    return TOOL_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv))
    if "--tools" in sys.argv:
        print(build_tools())
