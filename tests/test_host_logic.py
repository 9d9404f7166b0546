"""CPU-side checks: the C-ABI library loads and exports what the header declares, the
golden fixtures pin the oracle, and the library's host/device arithmetic headers agree
with the oracle when compiled as plain C++."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from conftest import ROOT, assert_bits_equal

GOLD = np.load(ROOT / "tests" / "golden" / "dots.npz")
KINDS = ["f32", "f16", "bf16", "q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k"]


def test_library_exports_every_declared_symbol(pkg):
    header = (ROOT / "include" / "aot_cuda.h").read_text()
    declared = set(re.findall(r"\b(aotcu_[a-z0-9_]+)\s*\(", header))
    declared -= {"aotcu_upload_weights"}  # mentioned in a comment only
    lib = pkg.lib.load()
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert declared == set(pkg.lib.SYMBOLS), declared ^ set(pkg.lib.SYMBOLS)
    assert lib.aotcu_version().startswith(b"aot-cuda")
    assert lib.aotcu_row_bytes(6, 2048) == 1152 and lib.aotcu_row_bytes(8, 2048) == 1680


def test_no_device_means_an_error_not_a_fallback(pkg):
    """Without a GPU every compute entry point must fail loudly."""
    import shutil
    if shutil.which("nvidia-smi"):
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = pkg.lib.load().aotcu_init(0, C.byref(h))
    assert rc == pkg.lib.ERR_CUDA
    assert b"no CPU path" in pkg.lib.load().aotcu_last_error()


def test_product_does_not_import_the_oracle():
    for p in (ROOT / "aot-llm_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".h"):
            assert "oracle" not in p.read_text().replace("# only tests", ""), p


@pytest.mark.parametrize("key", sorted({k.rsplit("_", 1)[0] for k in GOLD.files}))
def test_oracle_matches_golden(ob, key):
    kind = KINDS.index("_".join(key.split("_")[:-1]))
    w, x = GOLD[key + "_w"], GOLD[key + "_x"]
    cols, rows = x.size, 4
    rb = ob.row_bytes(kind, cols)
    xq = ob.quantize_act(kind, x)
    assert xq.tobytes() == GOLD[key + "_xq"].tobytes()
    for r in range(rows):
        wr = w[r * rb:(r + 1) * rb].copy()
        assert ob.dot(ob.AVX2_F16C, kind, wr, xq, cols).view(np.uint32) == GOLD[key + "_dot"][r].view(np.uint32)
        assert_bits_equal(ob.dequant_row(kind, wr, cols), GOLD[key + "_deq"][r], key)
        if kind >= 3:
            si, sm = ob.block_sums(kind, wr, xq, cols)
            assert np.array_equal(si, GOLD[key + "_sumi"][r]) and np.array_equal(sm, GOLD[key + "_summ"][r])


@pytest.mark.parametrize("key", sorted({k.rsplit("_", 1)[0] for k in GOLD.files}))
def test_library_arithmetic_matches_golden(pkg, hostcheck, key):
    """The per-block integer sums, f32 operation order and element dequantizers of the
    CUDA sources (compiled for the host) against the fixtures."""
    kind = KINDS.index("_".join(key.split("_")[:-1]))
    w, x = GOLD[key + "_w"], GOLD[key + "_x"]
    cols, rows = x.size, 4
    rb = pkg.lib.row_bytes(kind, cols)
    xq = np.frombuffer(GOLD[key + "_xq"].tobytes(), dtype=np.uint8).copy() if kind >= 3 else x
    nb = max(cols // pkg.lib.BLOCK[kind], 1)
    for r in range(rows):
        wr = w[r * rb:(r + 1) * rb].copy()
        si, sm = np.zeros(nb, np.int32), np.zeros(nb, np.int32)
        got = np.float32(hostcheck.hc_dot(kind, pkg.lib.ptr(wr), pkg.lib.ptr(xq), cols, pkg.lib.ptr(si), pkg.lib.ptr(sm)))
        assert got.view(np.uint32) == GOLD[key + "_dot"][r].view(np.uint32), (key, r)
        if kind >= 3:
            assert np.array_equal(si, GOLD[key + "_sumi"][r])
        if kind in (6, 7):
            assert np.array_equal(sm, GOLD[key + "_summ"][r])
        deq = np.zeros(cols, np.float32)
        hostcheck.hc_dequant_row(kind, pkg.lib.ptr(wr), pkg.lib.ptr(deq), cols)
        assert_bits_equal(deq, GOLD[key + "_deq"][r], key)


def test_half_conversion_all_patterns(hostcheck):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([hostcheck.hc_half(int(v)) for v in h], dtype=np.float32)
    assert ((got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))).all()


def test_expf_matches_libm(hostcheck):
    """The fp64 restatement of expf against this machine's C library: every 61st bit
    pattern of the whole f32 range, every pattern in [-1.5, -0.5] (the softmax core),
    and the two inputs where the non-FMA variant of the algorithm would differ."""
    assert hostcheck.hc_expf_mismatches(0, 0xFFFFFFFF, 61) == 0
    lo, hi = np.float32(-0.5).view(np.uint32), np.float32(-1.5).view(np.uint32)
    assert hostcheck.hc_expf_mismatches(int(lo), int(hi), 1) == 0
    x = np.array([float.fromhex('-0x1.f8cbb2p+5'), float.fromhex('0x1.04845ep+5'), 0.0, -0.0, -104.0, 89.0, -np.inf], dtype=np.float32)
    y = np.zeros_like(x)
    hostcheck.hc_expf(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), x.size)
    libm = C.CDLL("libm.so.6")
    libm.expf.restype = C.c_float
    libm.expf.argtypes = [C.c_float]
    assert_bits_equal(y, np.array([libm.expf(float(v)) for v in x], dtype=np.float32), "expf specials")


def test_expf_table_is_correctly_rounded():
    from decimal import Decimal, getcontext
    import struct
    getcontext().prec = 80
    src = (ROOT / "aot-llm_b200" / "csrc" / "expf_exact.cuh").read_text()
    vals = [int(v, 16) for v in re.findall(r"0x([0-9a-f]{16})ULL", src)][:32]
    for i, v in enumerate(vals):
        d = float(Decimal(2) ** (Decimal(i) / Decimal(32)))
        assert v == (struct.unpack("<Q", struct.pack("<d", d))[0] - (i << 47)) & (2**64 - 1)


def _naive_sum(p):
    s = np.float32(0)
    with np.errstate(over="ignore"):
        for v in p:
            s = np.float32(s + v)
    return s


def test_parallel_sequential_sum_is_exact(hostcheck):
    """The binade-scan evaluation of `s += p[i]` against the scalar loop on inputs built
    to hit ties, subnormals, zeros, single huge terms and overflow."""
    hostcheck.hc_seqsum.restype = C.c_float
    hostcheck.hc_seqsum.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_int)]
    rng = np.random.default_rng(0)
    cases = []
    for n in (1, 2, 7, 64, 65, 200, 2048, 4096):
        cases += [(rng.standard_normal(n) ** 2).astype(np.float32),
                  (rng.standard_normal(n).astype(np.float32) * np.float32(1e-20)) ** 2,
                  rng.integers(0, 5, n).astype(np.float32),
                  rng.integers(0, 1 << 12, n).astype(np.float32) * np.float32(2.0 ** -10),
                  np.exp(-rng.random(n) * 30).astype(np.float32),
                  (2.0 ** rng.integers(-30, 10, n)).astype(np.float32),
                  (rng.standard_normal(n) ** 2).astype(np.float32) * np.float32(1e37),
                  np.zeros(n, dtype=np.float32)]
        for first, rest in ((2.0 ** 24, 0.5), (2.0 ** 24 + 2, 1.0), (2.0 ** 25, 3.0)):
            x = np.full(n, rest, dtype=np.float32)
            x[0] = first
            cases.append(x)
    hostcheck.hc_seqsum_runs.restype = C.c_float
    hostcheck.hc_seqsum_runs.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.POINTER(C.c_int)]
    for n in (300, 2048, 5000):
        # sums that sit on a binade boundary for long stretches, and ties at every step
        cases += [np.full(n, 2.0 ** -3, dtype=np.float32), np.full(n, 1.5, dtype=np.float32),
                  np.concatenate([[np.float32(2.0 ** 20)], np.full(n - 1, 0.5 * 2.0 ** -3, dtype=np.float32)]).astype(np.float32),
                  np.concatenate([(rng.standard_normal(n - 3) ** 2), [np.inf, 1.0, 2.0]]).astype(np.float32),
                  np.concatenate([(rng.standard_normal(n - 3) ** 2), [np.nan, 1.0, 2.0]]).astype(np.float32)]
    for p in cases:
        want = _naive_sum(p)
        for T, head in ((992, 48), (32, 0), (256, 8), (7, 3)):
            got = np.float32(hostcheck.hc_seqsum(p.ctypes.data_as(C.c_void_p), p.size, T, head, None))
            assert got.view(np.uint32) == want.view(np.uint32) or (np.isnan(got) and np.isnan(want)), (p.size, T)
        # the chunked form the device runs, with honest and with deliberately wrong predictions
        for skew in (1.0, 1.0 + 2.0 ** -20, 0.75, 1.5, 0.0, 1e30):
            n_slow = C.c_int(0)
            got = np.float32(hostcheck.hc_seqsum_runs(p.ctypes.data_as(C.c_void_p), p.size, skew, C.byref(n_slow)))
            assert got.view(np.uint32) == want.view(np.uint32) or (np.isnan(got) and np.isnan(want)), (p.size, skew)


def test_sequential_sum_of_squares_takes_the_fast_path(hostcheck):
    """For the sums the decode step evaluates (squares of a normalised row) only a handful of
    chunks fall back to term-by-term adds: the binade crossings and the odd exact tie."""
    hostcheck.hc_seqsum_runs.restype = C.c_float
    hostcheck.hc_seqsum_runs.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.POINTER(C.c_int)]
    rng = np.random.default_rng(5)
    for n in (2048, 4096):
        for _ in range(20):
            p = (rng.standard_normal(n) ** 2).astype(np.float32)
            n_slow = C.c_int(0)
            got = np.float32(hostcheck.hc_seqsum_runs(p.ctypes.data_as(C.c_void_p), p.size, 1.0, C.byref(n_slow)))
            assert got.view(np.uint32) == _naive_sum(p).view(np.uint32)
            assert n_slow.value <= 16, n_slow.value


def test_bench_kind_table_matches_the_library(pkg):
    """bench.py names kinds by the ids of include/aot_cuda.h."""
    import importlib.util
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("bench_mod", Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert [k for k, _ in sorted(bench.KINDS.items(), key=lambda kv: kv[1])] == pkg.lib.KIND_NAMES
    assert bench.METRIC == "decode_tokens_per_s"
