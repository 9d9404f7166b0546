"""Shared fixtures. GPU tests are marked `gpu` and call through the C-ABI library;
everything else runs on a machine without a GPU."""
from __future__ import annotations

import ctypes as C
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    graft.build()
    return graft.import_package()


@pytest.fixture(scope="session")
def ob(pkg):
    from oracle import binding
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def hostcheck():
    """The library's host/device arithmetic headers compiled as plain C++ (test-only)."""
    d = ROOT / "tests" / "hostcheck"
    so = d / "_hostcheck.so"
    src = d / "hostcheck.cpp"
    deps = [src] + list((ROOT / "aot-llm_b200" / "csrc").glob("*.cuh"))
    if not so.exists() or any(p.stat().st_mtime > so.stat().st_mtime for p in deps):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-o", str(so), str(src),
                        "-lm"], check=True)
    hc = C.CDLL(str(so))
    hc.hc_dot.restype = C.c_float
    hc.hc_dot.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    hc.hc_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]
    hc.hc_expf.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    hc.hc_expf_mismatches.restype = C.c_uint64
    hc.hc_expf_mismatches.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    hc.hc_half.restype = C.c_float
    hc.hc_half.argtypes = [C.c_uint16]
    return hc


@pytest.fixture(scope="session")
def ctx(pkg):
    """One CUDA context for the whole GPU session."""
    c = pkg.Context(0)
    yield c
    c.close()


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bits_equal(got, want, what=""):
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    bad = np.flatnonzero(bits(got).ravel() != bits(want).ravel())
    if bad.size:
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.size} of {got.size} values differ bitwise; first at {i}: "
                             f"{got.ravel()[i]!r} vs {want.ravel()[i]!r}")


class XorShift64:
    """The generator of the reference's kernel tests (crates/aot-kernels/tests/dots.rs:10-21)."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> int:
        s = self.s
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = s
        return s

    def f(self) -> float:
        return np.float32(np.float32(self.next() % 20001) / np.float32(10000.0) - np.float32(1.0))

    def floats(self, n: int, scale: float = 1.0) -> np.ndarray:
        return np.array([self.f() * np.float32(scale) for _ in range(n)], dtype=np.float32)


def make_weights(pkg, kind: int, rows: int, cols: int, seed: int, mode: str = "enc") -> np.ndarray:
    """Rows of `kind`: encoded from uniform floats ("enc") or with field-uniform random
    block content ("uniform", quantized kinds only)."""
    L = pkg.lib
    w = np.empty(rows * L.row_bytes(kind, cols), dtype=np.uint8)
    if mode == "enc" or kind < 3:
        L.check(L.synth().aotcu_synth_tensor(kind, rows, cols, 1.0, 0.0, seed, L.ptr(w)))
    else:
        L.check(L.synth().aotcu_synth_blocks(kind, rows * cols // L.BLOCK[kind], seed, L.ptr(w)))
    return w
