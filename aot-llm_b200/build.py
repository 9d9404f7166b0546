"""Builds libaot_cuda.so (the C-ABI library) in-tree with nvcc for sm_100a.

The same command is what a Rust ``build.rs`` would run for the reference's
generated project.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libaot_cuda.so"
SOURCES = [CSRC / "aotcu.cu"]
SYNTH_SRC = HERE / "synth" / "synth.cpp"
SYNTH_LIB = HERE / "libaot_synth.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # Exactness: no implicit a*b+c contraction anywhere (device or host); every fused
    # operation in the sources is an explicit fma.
    "--fmad=false",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-O2",
    "-shared",
]


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return p


STAMP = HERE / "libaot_cuda.so.srchash"


def source_hash() -> str:
    """Hash of everything the library is built from (contents, not timestamps: a copied
    tree does not keep modification times in a useful order)."""
    deps = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))) + \
        [HERE.parent / "include" / "aot_cuda.h"]
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for d in deps:
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def stale() -> bool:
    if not LIB.exists() or not STAMP.exists():
        return True
    return STAMP.read_text().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    # Several ranks of one job may get here together: one builds, the others wait and
    # then find the library fresh. The new file replaces the old one atomically.
    with open(HERE / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not stale():
            return LIB
        tmp = HERE / f".libaot_cuda.{os.getpid()}.so"
        cmd = [nvcc_path(), *NVCC_FLAGS, "-o", str(tmp), *map(str, SOURCES)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(r.stderr)
        if r.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        os.replace(tmp, LIB)
        STAMP.write_text(source_hash() + "\n")
    return LIB


def build_synth(force: bool = False) -> Path:
    """libaot_synth.so: the host-only generator of synthetic weights (tests, benchmarks).
    Plain g++, no CUDA: a process that only needs test data never maps the CUDA library."""
    deps = [SYNTH_SRC, HERE / "synth" / "aot_synth.h", CSRC / "blockmath.cuh"]
    if not force and SYNTH_LIB.exists() and all(SYNTH_LIB.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return SYNTH_LIB
    with open(HERE / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        tmp = HERE / f".libaot_synth.{os.getpid()}.so"
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread", "-o", str(tmp), str(SYNTH_SRC)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
        os.replace(tmp, SYNTH_LIB)
    return SYNTH_LIB


if __name__ == "__main__":
    build_synth(force="--force" in sys.argv)
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
