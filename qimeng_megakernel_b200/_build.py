"""Builds libqmk_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension machinery).

The reference builds one pybind module per model with a Makefile
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/Makefile:21-60);
here there is one shared library with a C ABI for every supported shape.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_PATH = CSRC / "libqmk_b200.so"
SOURCES = ["qmk_api.cu", "qmk_static.cu", "qmk_batch.cu"]
HEADERS = ["qmk_megakernel.cuh", "qmk_kernel.cuh", "qmk_phases.cuh", "qmk_attention.cuh", "qmk_staging.cuh", "qmk_device.cuh",
           "qmk_params.h", "qmk_schedule.h", "qmk_batch_kernel.cuh", "qmk_batch_device.cuh", "qmk_batch_params.h", "qmk_batch_schedule.h", "qmk_batch_host.h", "../../include/qmk_b200.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libqmk_b200.so")
    return cand


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any((CSRC / f).resolve().stat().st_mtime > t for f in SOURCES + HEADERS)


def _compile(out: Path, sources: list[str], defines: list[str], verbose: bool) -> Path:
    cmd = [_nvcc(), *NVCC_FLAGS, *defines, *(["-Xptxas", "-v"] if verbose else []), "-o", str(out),
           *[str(CSRC / s) for s in sources]]
    proc = subprocess.run(cmd, cwd=str(CSRC), capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return out


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    return _compile(LIB_PATH, SOURCES, [], verbose)


if __name__ == "__main__":
    print(build(force=True, verbose=True))
