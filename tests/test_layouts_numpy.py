"""An independent statement of the seven GGUF block layouts, written in numpy from the layout
table alone (field offsets and element mappings of crates/aot-kernels/src/quant.rs:300-443),
checked against the oracle's dequant_row on field-uniform random blocks and on encoded rows.
It pins the one part of the oracle that the reference's own tests only check against itself:
the reading of raw weight bytes."""
import numpy as np
import pytest

from conftest import make_weights

F32, F16, BF16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = range(9)


def _f16(b: np.ndarray) -> np.ndarray:
    """Little-endian byte pairs [..., 2] -> float32 (IEEE binary16)."""
    return np.ascontiguousarray(b).view("<f2").astype(np.float32)[..., 0]


def _scale_min_k4(s: np.ndarray):
    """The eight 6-bit (scale, min) pairs packed in 12 bytes, s: [n, 12] uint8 -> two [n, 8] arrays."""
    s = s.astype(np.int32)
    sc, mn = np.zeros((s.shape[0], 8), np.int32), np.zeros((s.shape[0], 8), np.int32)
    for j in range(8):
        if j < 4:
            sc[:, j], mn[:, j] = s[:, j] & 63, s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 15) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    return sc, mn


def dequant(kind: int, raw: np.ndarray, n: int) -> np.ndarray:
    """n weights of one row from its raw bytes, float32, with the reference's operation order."""
    f = np.float32
    if kind == Q4_0:
        b = raw.reshape(-1, 18)
        d = _f16(b[:, 0:2])[:, None]
        q = np.concatenate([b[:, 2:] & 15, b[:, 2:] >> 4], axis=1).astype(np.int32) - 8
        return (q.astype(f) * d).reshape(-1)[:n]
    if kind == Q5_0:
        b = raw.reshape(-1, 22)
        d = _f16(b[:, 0:2])[:, None]
        qh = np.ascontiguousarray(b[:, 2:6]).view("<u4")[:, 0].astype(np.uint64)
        nib = np.concatenate([b[:, 6:] & 15, b[:, 6:] >> 4], axis=1).astype(np.int32)
        bit = ((qh[:, None] >> np.arange(32, dtype=np.uint64)[None, :]) & 1).astype(np.int32)
        return ((nib | (bit << 4)) - 16).astype(f).__mul__(d).reshape(-1)[:n]
    if kind == Q8_0:
        b = raw.reshape(-1, 34)
        d = _f16(b[:, 0:2])[:, None]
        return (b[:, 2:].view(np.int8).astype(f) * d).reshape(-1)[:n]
    if kind in (Q4_K, Q5_K):
        bs = 176 if kind == Q5_K else 144
        b = raw.reshape(-1, bs)
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _scale_min_k4(b[:, 4:16])
        qs = b[:, bs - 128:].astype(np.int32).reshape(-1, 4, 32)      # chunk c, byte l
        q = np.stack([qs & 15, qs >> 4], axis=2).reshape(-1, 8, 32)    # sub-block j = 2c (+1 for the high nibble)
        if kind == Q5_K:
            qh = b[:, 16:48].astype(np.int32)                          # bit j of byte l
            q = q + (((qh[:, None, :] >> np.arange(8)[None, :, None]) & 1) << 4)
        # quant.rs:366-374: (d * sc) * q - dmin * m, all in f32
        dl = (d[:, None] * sc.astype(f)).astype(f)
        ml = (dmin[:, None] * mn.astype(f)).astype(f)
        return ((dl[:, :, None] * q.astype(f)).astype(f) - ml[:, :, None]).astype(f).reshape(-1)[:n]
    if kind == Q6_K:
        b = raw.reshape(-1, 210)
        ql, qh = b[:, 0:128].astype(np.int32), b[:, 128:192].astype(np.int32)
        sc = b[:, 192:208].view(np.int8).astype(np.int32)
        d = _f16(b[:, 208:210])
        out = np.zeros((b.shape[0], 256), f)
        for e in range(256):
            half, r = divmod(e, 128)
            quarter, l = divmod(r, 32)
            lb = ql[:, 64 * half + l + 32 * (quarter & 1)]
            lo = (lb & 15) if quarter < 2 else (lb >> 4)
            hi = (qh[:, 32 * half + l] >> (2 * quarter)) & 3
            q = (lo | (hi << 4)) - 32
            # quant.rs:422-425: d * sc * q, left to right
            out[:, e] = ((d * sc[:, e // 16].astype(f)).astype(f) * q.astype(f)).astype(f)
        return out.reshape(-1)[:n]
    raise ValueError(kind)


@pytest.mark.parametrize("mode", ["enc", "uniform"])
@pytest.mark.parametrize("kind", [Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K])
def test_numpy_layouts_agree_with_the_oracle(pkg, ob, kind, mode):
    rows, cols = 6, 1024
    w = make_weights(pkg, kind, rows, cols, 4242 + kind, mode)
    rb = pkg.lib.row_bytes(kind, cols)
    for r in range(rows):
        row = w[r * rb:(r + 1) * rb].copy()
        want = ob.dequant_row(kind, row, cols)
        got = dequant(kind, row, cols)
        assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32)), (kind, mode, r)


def test_numpy_layouts_float_kinds(pkg, ob):
    x = (np.random.default_rng(1).standard_normal(512) * 3).astype(np.float32)
    for kind, conv in ((F16, lambda b: b.view("<f2").astype(np.float32)),
                       (BF16, lambda b: (b.view("<u2").astype(np.uint32) << 16).view(np.float32)),
                       (F32, lambda b: b.view("<f4"))):
        w = make_weights(pkg, kind, 1, 512, 9)
        assert np.array_equal(conv(w).view(np.uint32), ob.dequant_row(kind, w, 512).view(np.uint32)), kind
