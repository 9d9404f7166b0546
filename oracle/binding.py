"""ctypes binding of the CPU oracle (test infrastructure).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product path never does. The library is built on demand from
the sources next to this file (see ``Makefile``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "liboracle.so"

# Kind order of crates/aot-kernels/src/quant.rs:34-44.
F32, F16, BF16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = range(9)
KIND_NAMES = ["f32", "f16", "bf16", "q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k"]
SCALAR, AVX2, AVX2_F16C = 0, 1, 2

Q8_0_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (32,))])
Q8_K_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (256,)), ("bsums", "<i2", (16,))])
assert Q8_0_DTYPE.itemsize == 36 and Q8_K_DTYPE.itemsize == 292


class Tensor(C.Structure):
    _fields_ = [("kind", C.c_int32), ("present", C.c_int32), ("off", C.c_uint64), ("len", C.c_uint64),
                ("rows", C.c_uint64), ("cols", C.c_uint64)]


class Dims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dim", "hidden", "n_layer", "n_head", "n_kv_head", "head_dim", "rot_dim",
                                          "vocab", "n_ctx_train", "swa_window")] + \
               [(n, C.c_float) for n in ("eps", "rope_base", "rope_scale", "rope_base_local", "rope_scale_local")] + \
               [(n, C.c_int32) for n in ("qkv_bias", "qk_norm", "rope_neox", "post_norms", "gelu", "embd_scale")]


LAYER_TENSORS = ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "gate", "up", "down", "bq", "bk", "bv", "q_norm",
                 "k_norm", "attn_post_norm", "ffn_post_norm")


class Layer(C.Structure):
    _fields_ = [(n, Tensor) for n in LAYER_TENSORS] + [("local_attn", C.c_int32), ("pad_", C.c_int32)]


class ModelHead(C.Structure):
    _fields_ = [("dims", Dims), ("token_embd", Tensor), ("output_norm", Tensor), ("output", Tensor),
                ("rope_freqs", Tensor)]


def build(force: bool = False) -> Path:
    """Compile liboracle.so if it is missing or older than its sources."""
    srcs = list(_HERE.glob("*.cpp")) + list(_HERE.glob("*.h"))
    stale = force or not _LIB_PATH.exists() or any(s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in srcs)
    if stale:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB_PATH))
        vp, sz, f32p = C.c_void_p, C.c_size_t, C.c_void_p
        L.orc_row_bytes.restype = sz
        L.orc_row_bytes.argtypes = [C.c_int, sz]
        L.orc_block_size.restype = sz
        L.orc_type_size.restype = sz
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_quantize_q8_0.argtypes = [vp, sz, vp]
        L.orc_quantize_q8_k.argtypes = [vp, sz, vp]
        L.orc_dequant_row.argtypes = [C.c_int, vp, vp, sz]
        L.orc_dot.restype = C.c_float
        L.orc_dot.argtypes = [C.c_int, C.c_int, vp, vp, sz]
        L.orc_dot_x4.restype = C.c_int
        L.orc_dot_x4.argtypes = [C.c_int, C.c_int, vp, vp, vp, vp, vp, sz, vp]
        L.orc_block_sums.argtypes = [C.c_int, vp, vp, sz, vp, vp]
        L.orc_pool_new.restype = vp
        L.orc_pool_new.argtypes = [C.c_int]
        L.orc_pool_free.argtypes = [vp]
        L.orc_matvec.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, sz, sz]
        L.orc_matvec2.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, vp, vp, sz, sz]
        L.orc_matvec3.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz]
        L.orc_matmul.argtypes = [vp, C.c_int, C.c_int, vp, vp, vp, sz, sz, sz]
        L.orc_rmsnorm.argtypes = [vp, vp, vp, sz, C.c_float]
        L.orc_rope_cos_sin.argtypes = [vp, vp, sz, C.c_float]
        L.orc_rope.argtypes = [vp, sz, sz, sz, vp]
        L.orc_rope_neox.argtypes = [vp, sz, sz, sz, vp]
        L.orc_rmsnorm_heads.argtypes = [vp, vp, sz, sz, C.c_float]
        L.orc_softmax.argtypes = [vp, sz]
        L.orc_silu_mul.argtypes = [vp, vp, sz]
        L.orc_gelu.restype = C.c_float
        L.orc_gelu.argtypes = [C.c_float]
        L.orc_gelu_mul.argtypes = [vp, vp, sz]
        L.orc_add_inplace.argtypes = [vp, vp, sz]
        L.orc_inv_freq.argtypes = [vp, sz, C.c_float, vp]
        L.orc_attention.argtypes = [vp, vp, vp, vp, vp, vp, C.POINTER(Dims), sz, sz, sz, sz]
        L.orc_attention_rows.argtypes = [vp, vp, vp, vp, vp, vp, C.POINTER(Dims), sz, sz, sz, sz, sz]
        L.orc_argmax.restype = C.c_uint32
        L.orc_argmax.argtypes = [vp, sz]
        L.orc_model_new.restype = vp
        L.orc_model_new.argtypes = [C.POINTER(ModelHead), C.POINTER(Layer), vp, sz, sz, sz, C.c_int, C.c_int]
        L.orc_model_free.argtypes = [vp]
        L.orc_forward.restype = C.c_int
        L.orc_forward.argtypes = [vp, C.c_uint32, sz, C.c_int]
        L.orc_forward_batch.restype = C.c_int
        L.orc_forward_batch.argtypes = [vp, vp, sz, sz, C.c_int]
        L.orc_state_buf.restype = C.POINTER(C.c_float)
        L.orc_state_buf.argtypes = [vp, C.c_char_p, C.POINTER(sz)]
        L.orc_state_aqk.restype = vp
        L.orc_state_aqk.argtypes = [vp, C.POINTER(sz)]
        L.orc_state_aq0.restype = vp
        L.orc_state_aq0.argtypes = [vp, C.POINTER(sz)]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def row_bytes(kind: int, n: int) -> int:
    return lib().orc_row_bytes(kind, n)


def activation(kind: int) -> str:
    return "q8_0" if kind in (Q4_0, Q5_0, Q8_0) else "q8_k" if kind in (Q4_K, Q5_K, Q6_K) else "f32"


def detect_table() -> int:
    return lib().orc_detect_table()


def quantize_q8_0(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(x.size // 32, dtype=Q8_0_DTYPE)
    lib().orc_quantize_q8_0(_p(x), x.size, _p(out))
    return out


def quantize_q8_k(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(x.size // 256, dtype=Q8_K_DTYPE)
    lib().orc_quantize_q8_k(_p(x), x.size, _p(out))
    return out


def quantize_act(kind: int, x) -> np.ndarray:
    a = activation(kind)
    return quantize_q8_0(x) if a == "q8_0" else quantize_q8_k(x) if a == "q8_k" else _f32(x)


def dequant_row(kind: int, row: np.ndarray, n: int) -> np.ndarray:
    row = np.ascontiguousarray(row, dtype=np.uint8)
    out = np.zeros(n, dtype=np.float32)
    lib().orc_dequant_row(kind, _p(row), _p(out), n)
    return out


def dot(table: int, kind: int, w: np.ndarray, x: np.ndarray, cols: int) -> np.float32:
    return np.float32(lib().orc_dot(table, kind, _p(w), _p(x), cols))


def dot_x4(table: int, kind: int, w: np.ndarray, xs, cols: int):
    out = np.zeros(4, dtype=np.float32)
    ok = lib().orc_dot_x4(table, kind, _p(w), _p(xs[0]), _p(xs[1]), _p(xs[2]), _p(xs[3]), cols, _p(out))
    return out if ok else None


def block_sums(kind: int, w: np.ndarray, x: np.ndarray, cols: int):
    nb = cols // lib().orc_block_size(kind)
    sumi = np.zeros(nb, dtype=np.int32)
    summ = np.zeros(nb, dtype=np.int32)
    lib().orc_block_sums(kind, _p(w), _p(x), cols, _p(sumi), _p(summ))
    return sumi, summ


class Pool:
    def __init__(self, n_threads: int):
        self.h = lib().orc_pool_new(n_threads)
        self.n = n_threads

    def close(self):
        if self.h:
            lib().orc_pool_free(self.h)
            self.h = None

    def __del__(self):
        self.close()


def matvec(pool: Pool, table: int, kind: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int) -> np.ndarray:
    out = np.zeros(rows, dtype=np.float32)
    lib().orc_matvec(pool.h, table, kind, _p(out), _p(w), _p(x), rows, cols)
    return out


def matvec2(pool, table, kind, wa, wb, x, rows, cols):
    oa = np.zeros(rows, dtype=np.float32)
    ob = np.zeros(rows, dtype=np.float32)
    lib().orc_matvec2(pool.h, table, kind, _p(oa), _p(ob), _p(wa), _p(wb), _p(x), rows, cols)
    return oa, ob


def matvec3(pool, table, kind, ws, x, rows3, cols):
    outs = [np.zeros(r, dtype=np.float32) for r in rows3]
    lib().orc_matvec3(pool.h, table, kind, _p(outs[0]), _p(outs[1]), _p(outs[2]), _p(ws[0]), _p(ws[1]), _p(ws[2]),
                      _p(x), rows3[0], rows3[1], rows3[2], cols)
    return outs


def matmul(pool, table, kind, w, xs, m, rows, cols) -> np.ndarray:
    out = np.zeros(m * rows, dtype=np.float32)
    lib().orc_matmul(pool.h, table, kind, _p(out), _p(w), _p(xs), m, rows, cols)
    return out.reshape(m, rows)


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.zeros_like(x)
    lib().orc_rmsnorm(_p(out), _p(x), _p(w), x.size, eps)
    return out


def rope_cos_sin(inv_freq, pos: float) -> np.ndarray:
    inv_freq = _f32(inv_freq)
    cs = np.zeros(2 * inv_freq.size, dtype=np.float32)
    lib().orc_rope_cos_sin(_p(cs), _p(inv_freq), inv_freq.size, pos)
    return cs


def rope(x, n_heads, head_dim, rot_dim, cs, neox=False) -> np.ndarray:
    x = _f32(x).copy()
    cs = _f32(cs)
    (lib().orc_rope_neox if neox else lib().orc_rope)(_p(x), n_heads, head_dim, rot_dim, _p(cs))
    return x


def rmsnorm_heads(x, w, n_heads, head_dim, eps) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(w)
    lib().orc_rmsnorm_heads(_p(x), _p(w), n_heads, head_dim, eps)
    return x


def softmax(x) -> np.ndarray:
    x = _f32(x).copy()
    lib().orc_softmax(_p(x), x.size)
    return x


def silu_mul(h, up) -> np.ndarray:
    h = _f32(h).copy()
    up = _f32(up)
    lib().orc_silu_mul(_p(h), _p(up), h.size)
    return h


def gelu_mul(h, up) -> np.ndarray:
    h = _f32(h).copy()
    up = _f32(up)
    lib().orc_gelu_mul(_p(h), _p(up), h.size)
    return h


def add_inplace(x, y) -> np.ndarray:
    x = _f32(x).copy()
    y = _f32(y)
    lib().orc_add_inplace(_p(x), _p(y), x.size)
    return x


def inv_freq(rot_dim: int, base: float, freq_factors=None) -> np.ndarray:
    out = np.zeros(rot_dim // 2, dtype=np.float32)
    ff = _f32(freq_factors) if freq_factors is not None else None
    lib().orc_inv_freq(_p(out), rot_dim, base, _p(ff) if ff is not None else None)
    return out


def attention(pool, q, k_cache, v_cache, dims: Dims, ctx, layer, pos, window=0) -> np.ndarray:
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    out = np.zeros(dims.n_head * dims.head_dim, dtype=np.float32)
    scores = np.zeros(max(dims.n_head, pool.n) * ctx, dtype=np.float32)
    lib().orc_attention(pool.h, _p(out), _p(q), _p(k_cache), _p(v_cache), _p(scores), C.byref(dims), ctx, layer,
                        pos, window)
    return out


def attention_rows(pool, q, k_cache, v_cache, dims: Dims, ctx, layer, pos0, m, window=0) -> np.ndarray:
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    out = np.zeros(m * dims.n_head * dims.head_dim, dtype=np.float32)
    scratch = np.zeros(max(dims.n_head, pool.n) * ctx, dtype=np.float32)
    lib().orc_attention_rows(pool.h, _p(out), _p(q), _p(k_cache), _p(v_cache), _p(scratch), C.byref(dims), ctx,
                             layer, pos0, m, window)
    return out


def argmax(x) -> int:
    x = _f32(x)
    return int(lib().orc_argmax(_p(x), x.size))


class Model:
    """The oracle's interpreter of the generated forward pass over a weights blob."""

    def __init__(self, head: ModelHead, layers, weights: np.ndarray, ctx: int, max_batch: int = 1,
                 n_threads: int | None = None, table: int | None = None):
        self.weights = np.ascontiguousarray(weights, dtype=np.uint8)
        self.head = head
        self.layers = (Layer * len(layers))(*layers)
        self.n_threads = n_threads or min(os.cpu_count() or 1, 8)
        self.table = detect_table() if table is None else table
        self.h = lib().orc_model_new(C.byref(head), self.layers, _p(self.weights), self.weights.size, ctx, max_batch,
                                     self.n_threads, self.table)

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def forward(self, token: int, pos: int, want_logits: bool = True) -> int:
        return lib().orc_forward(self.h, token, pos, int(want_logits))

    def forward_batch(self, tokens, pos0: int, want_logits: bool = True) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        return lib().orc_forward_batch(self.h, _p(t), t.size, pos0, int(want_logits))

    def buf(self, name: str) -> np.ndarray:
        n = C.c_size_t(0)
        p = lib().orc_state_buf(self.h, name.encode(), C.byref(n))
        if not p:
            raise KeyError(name)
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def aqk(self) -> np.ndarray:
        n = C.c_size_t(0)
        p = lib().orc_state_aqk(self.h, C.byref(n))
        return np.frombuffer((C.c_char * (n.value * 292)).from_address(p), dtype=Q8_K_DTYPE).copy()

    def logits(self) -> np.ndarray:
        return self.buf("logits")


def model_from_spec(spec, ctx: int, max_batch: int = 1, n_threads: int | None = None, table: int | None = None) -> Model:
    """Build the oracle's model from a synthetic ModelSpec of the package (same tensor
    table, identical struct layout, same weights bytes)."""
    head = ModelHead.from_buffer_copy(bytes(spec.head))
    layers = [Layer.from_buffer_copy(bytes(l)) for l in spec.layers]
    return Model(head, layers, spec.weights, ctx, max_batch, n_threads, table)
