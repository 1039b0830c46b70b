"""Compile libfvla_b200.so (sm_100a only) next to this file with nvcc.

    python -m flash_vla_b200.build [--force]

The library is built in-tree so that it travels with the source tree; there is no
JIT cache and no fallback: if the file is missing, loading the backend raises.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "libfvla_b200.so"
STAMP = ROOT / "libfvla_b200.so.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [ROOT.parent / "include" / "flash_vla_b200.h"]


def source_digest() -> str:
    h = hashlib.sha256()
    for p in _sources():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> Path:
    """Build the shared library unless an up-to-date one is present. Returns its path.

    `debug=True` builds a separate development library, libfvla_b200_debug.so, with -DFVLA_DEBUG: its
    kernels can record %globaltimer stamps into a buffer registered through fvla_debug_set_timestamps.
    The package never loads that file; the shipped library is built without the flag and contains none
    of that code."""
    lib = ROOT / "libfvla_b200_debug.so" if debug else LIB
    stamp = Path(str(lib) + ".stamp")
    flags = NVCC_FLAGS + (["-DFVLA_DEBUG"] if debug else [])
    digest = source_digest() + ("-debug" if debug else "")
    if not force and lib.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return lib
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *flags, "-o", str(lib)] + [str(p) for p in sorted(CSRC.glob("*.cu"))]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    Path(str(lib).replace(".so", ".ptxas.log")).write_text(proc.stdout + proc.stderr)
    stamp.write_text(digest)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, debug="--debug" in sys.argv))
