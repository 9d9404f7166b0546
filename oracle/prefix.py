"""CPU restatement of the reference's saved KV cache ("AOTP" blob): test infrastructure
only. The product path is `aotcu_kv_save` / `aotcu_kv_load` of the CUDA library; nothing
outside tests/, the smoke check and the benchmark's CPU arm may import this module.

Follows crates/aot-kernels/src/prefix.rs: layout comment 14-26, `Prefix::parse` 45-69,
`load_into` 88-101, `serialize` 112-141. The reference holds no golden blob for this path;
its own check is the end-to-end property of crates/aot-llm/tests/e2e.rs:797-805 (a run
continued from a saved cache gives the logits of the whole prompt), which the tests repeat
on the oracle's model and on the GPU, next to a header written out by hand from the layout
comment.
"""
from __future__ import annotations

import struct

import numpy as np

MAGIC = b"AOTP"      # prefix.rs:30
VERSION = 2          # prefix.rs:31
HEADER = 24          # prefix.rs:32


def data_offset(n_tokens: int) -> int:
    """Token ids end at HEADER + 4 n; rows start at the next 64-byte boundary (prefix.rs:62, 125-127)."""
    return (HEADER + 4 * n_tokens + 63) // 64 * 64


def serialize(k_cache: np.ndarray, v_cache: np.ndarray, ctx: int, n_layer: int, kv_dim: int, tokens, n_cached: int) -> bytes:
    """prefix.rs:112-141. `k_cache` / `v_cache` are the State's flat caches, layer-major:
    row (layer, position) at (layer * ctx + position) * kv_dim."""
    tokens = [int(t) for t in tokens]
    n = len(tokens)
    n_cached = min(n_cached, n)                                               # prefix.rs:114
    out = bytearray()
    out += MAGIC
    out += struct.pack("<5I", VERSION, n, n_layer, kv_dim, n_cached)          # prefix.rs:117-122
    out += struct.pack(f"<{n}I", *tokens)                                     # prefix.rs:123-125
    out += b"\0" * (data_offset(n) - len(out))                                # prefix.rs:126-128
    k = np.asarray(k_cache, dtype="<f4").reshape(n_layer, ctx, kv_dim)
    v = np.asarray(v_cache, dtype="<f4").reshape(n_layer, ctx, kv_dim)
    for layer in range(n_layer):                                              # prefix.rs:129-138
        out += k[layer, :n_cached].tobytes()
        out += v[layer, :n_cached].tobytes()
    return bytes(out)


class Prefix:
    def __init__(self, tokens, n_cached, n_layer, kv_dim, data):
        self.tokens, self.n_cached, self.n_layer, self.kv_dim, self.data = tokens, n_cached, n_layer, kv_dim, data

    def __len__(self):                      # prefix.rs:72-74
        return len(self.tokens)

    def cached(self) -> int:                # prefix.rs:81-83
        return self.n_cached

    def load_into(self, k_cache: np.ndarray, v_cache: np.ndarray, ctx: int) -> None:
        """prefix.rs:88-101: positions [0, cached) of every layer."""
        rows = self.n_cached * self.kv_dim
        flat = np.frombuffer(self.data, dtype="<f4")
        for layer in range(self.n_layer):
            at = layer * ctx * self.kv_dim
            k_cache[at:at + rows] = flat[(layer * 2) * rows:(layer * 2 + 1) * rows]
            v_cache[at:at + rows] = flat[(layer * 2 + 1) * rows:(layer * 2 + 2) * rows]


def parse(blob: bytes, n_layer: int, kv_dim: int):
    """prefix.rs:45-69: the parsed view, or None when the blob is empty, malformed or of
    another model."""
    if len(blob) < HEADER or blob[:4] != MAGIC:
        return None
    version, n, nl, kv, nc = struct.unpack_from("<5I", blob, 4)
    if version not in (1, VERSION):
        return None
    if version == 1:
        nc = n                                                                # prefix.rs:57
    if nl != n_layer or kv != kv_dim or n == 0 or nc > n:
        return None
    if len(blob) < HEADER + 4 * n:
        return None
    tokens = list(struct.unpack_from(f"<{n}I", blob, HEADER))
    off = data_offset(n)
    need = off + nl * 2 * nc * kv * 4
    if len(blob) < need:
        return None
    return Prefix(tokens, nc, nl, kv, blob[off:need])
