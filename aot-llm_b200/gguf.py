"""GGUF files to the library's tensor table: the header / metadata / tensor-table parser
(crates/aot-gguf/src/lib.rs:156-222, value types 358-387, type table types.rs:46-134), the
model description the code generator derives from it (crates/aot-codegen/src/model.rs:
176-195 architecture switches, 240-279 shape checks, 281-400 `ModelSpec::from_gguf`), and a
version-3 writer (lib.rs:392-455) for tests and for turning a synthetic model into a file.

The tensor data section of a GGUF file is exactly what `aotcu_gpu_new` uploads: tensors at
offsets relative to the aligned start of the section, rows back to back. `load_model(path)`
memory-maps the file and returns a `ModelSpec` whose `weights` is that section.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass, field

import numpy as np

from . import lib as L
from .lib import Dims, Layer, ModelHead, Tensor
from .model import ModelSpec, _absent

GGUF_MAGIC = 0x46554747          # "GGUF" little-endian (lib.rs:21)
DEFAULT_ALIGNMENT = 32           # lib.rs:23

# ggml type id -> (name, elements per block, bytes per block); types.rs:46-134
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144),
    13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74),
    18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50), 20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82),
    23: ("IQ4_XS", 256, 136), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 34: ("TQ1_0", 256, 54), 35: ("TQ2_0", 256, 66),
}
# the nine kinds the runtime executes (model.rs:24-37), ggml id -> library kind
KIND_OF_GGML = {0: L.F32, 1: L.F16, 30: L.BF16, 2: L.Q4_0, 6: L.Q5_0, 8: L.Q8_0, 12: L.Q4_K, 13: L.Q5_K, 14: L.Q6_K}
GGML_OF_KIND = {v: k for k, v in KIND_OF_GGML.items()}


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dims: list          # ggml order: innermost first
    ty: int             # ggml type id
    offset: int         # relative to the data section

    def n_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def n_bytes(self) -> int:
        _, blk, size = GGML_TYPES[self.ty]
        return self.n_elements() // blk * size

    def cols(self) -> int:
        return self.dims[0] if self.dims else 1

    def rows(self) -> int:
        n = 1
        for d in self.dims[1:]:
            n *= d
        return n


@dataclass
class GgufFile:
    version: int
    alignment: int
    metadata: list                      # (key, value) in file order
    tensors: list                       # TensorInfo in file order
    data_offset: int                    # absolute offset of the aligned tensor data section
    _keys: dict = field(default_factory=dict)
    _tensors: dict = field(default_factory=dict)

    def get(self, key, default=None):
        i = self._keys.get(key)
        return default if i is None else self.metadata[i][1]

    def tensor(self, name):
        i = self._tensors.get(name)
        return None if i is None else self.tensors[i]


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, n, what):
        if self.pos + n > len(self.buf):
            raise GgufError(f"unexpected end of data while reading {what} at offset {self.pos}")
        b = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return b

    def num(self, fmt, what):
        return struct.unpack("<" + fmt, self.take(struct.calcsize(fmt), what))[0]

    def string(self, what):
        n = self.num("Q", what)
        start = self.pos
        try:
            return self.take(n, what).decode("utf-8")
        except UnicodeDecodeError:
            raise GgufError(f"invalid UTF-8 in string at offset {start}")

    _SCALARS = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 10: "Q", 11: "q", 12: "d"}

    def value(self, vt, depth=0):
        """lib.rs:358-387"""
        W = "metadata value"
        if vt in self._SCALARS:
            return self.num(self._SCALARS[vt], W)
        if vt == 7:
            return self.num("B", W) != 0
        if vt == 8:
            return self.string(W)
        if vt == 9:
            et = self.num("I", W)
            n = self.num("Q", W)
            if et == 9 and depth > 4:
                raise GgufError("metadata arrays nested too deeply")
            return [self.value(et, depth + 1) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {vt}")


def parse(buf, file_len: int | None = None) -> GgufFile:
    """Header, metadata and tensor descriptors (lib.rs:156-222). `buf` may be a prefix of the
    file; tensor bounds are checked against `file_len`."""
    file_len = len(buf) if file_len is None else file_len
    r = _Reader(buf)
    magic = r.num("I", "magic")
    if magic != GGUF_MAGIC:
        raise GgufError(f"not a GGUF file (magic {magic:#x})")
    version = r.num("I", "version")
    if version not in (2, 3):
        raise GgufError(f"unsupported GGUF version {version}")
    n_tensors = r.num("Q", "tensor count")
    n_kv = r.num("Q", "metadata count")
    metadata, keys = [], {}
    for _ in range(n_kv):
        key = r.string("metadata key")
        vt = r.num("I", "metadata value type")
        keys[key] = len(metadata)
        metadata.append((key, r.value(vt)))
    alignment = DEFAULT_ALIGNMENT
    if "general.alignment" in keys:
        v = metadata[keys["general.alignment"]][1]
        alignment = v if isinstance(v, int) and not isinstance(v, bool) else DEFAULT_ALIGNMENT
    if alignment <= 0 or alignment & (alignment - 1):
        raise GgufError(f"alignment {alignment} is not a power of two")
    tensors, tindex = [], {}
    for _ in range(n_tensors):
        name = r.string("tensor name")
        nd = r.num("I", "tensor n_dims")
        if nd > 4:
            raise GgufError(f"tensor {name} has {nd} dimensions")
        dims = [r.num("Q", "tensor dim") for _ in range(nd)]
        ty = r.num("I", "tensor type")
        if ty not in GGML_TYPES:
            raise GgufError(f"tensor {name} has unknown type id {ty}")
        off = r.num("Q", "tensor offset")
        tindex[name] = len(tensors)
        tensors.append(TensorInfo(name, dims, ty, off))
    data_offset = -(-r.pos // alignment) * alignment
    for t in tensors:
        start = data_offset + t.offset
        if start + t.n_bytes() > file_len:
            raise GgufError(f"tensor {t.name} [{start}, {start + t.n_bytes()}) lies outside the file ({file_len} bytes)")
    return GgufFile(version, alignment, metadata, tensors, data_offset, keys, tindex)


# ---- architecture switches (model.rs:182-194) ---------------------------------------------------
ARCH_FLAGS = {
    "llama": {},
    "qwen2": dict(rope_neox=1, qkv_bias=1),
    "qwen3": dict(rope_neox=1, qk_norm=1),
    "phi3": dict(rope_neox=1, fused_qkv=1, fused_gate_up=1),
    "gemma3": dict(rope_neox=1, qk_norm=1, embd_scale=1, post_norms=1, gelu=1, swa_pattern=6),
}


def _tensor_spec(t: TensorInfo) -> Tensor:
    """model.rs:241-248"""
    if t.ty not in KIND_OF_GGML:
        raise GgufError(f"tensor {t.name} uses unsupported type {GGML_TYPES[t.ty][0]}; supported: f32, f16, bf16, q4_0, q5_0, "
                        "q8_0, q4_K, q5_K, q6_K")
    kind = KIND_OF_GGML[t.ty]
    cols = t.cols()
    if cols % GGML_TYPES[t.ty][1]:
        raise GgufError(f"tensor {t.name}: inner dimension {cols} is not a multiple of the {GGML_TYPES[t.ty][0]} block size")
    return Tensor(kind=kind, present=1, off=t.offset, len=t.n_bytes(), rows=t.rows(), cols=cols)


def _rows_view(t: Tensor, row0: int, rows: int) -> Tensor:
    """model.rs:260-263: rows of a fused matrix as a tensor of their own (Phi-3)."""
    rb = t.len // t.rows
    return Tensor(kind=t.kind, present=1, off=t.off + row0 * rb, len=rows * rb, rows=rows, cols=t.cols)


def model_spec(g: GgufFile, weights: np.ndarray, name: str = "gguf") -> ModelSpec:
    """`ModelSpec::from_gguf` (model.rs:281-400) for the library's tensor table. `weights` is
    the file's tensor data section (bytes from `g.data_offset` on)."""
    arch = g.get("general.architecture")
    if not isinstance(arch, str):
        raise GgufError("general.architecture is missing")
    if arch not in ARCH_FLAGS:
        raise GgufError(f'unsupported architecture "{arch}": supported are ' + ", ".join(f'"{a}"' for a in ARCH_FLAGS))
    fl = dict(rope_neox=0, qkv_bias=0, qk_norm=0, fused_qkv=0, fused_gate_up=0, embd_scale=0, post_norms=0, gelu=0, swa_pattern=0)
    fl.update(ARCH_FLAGS[arch])
    if g.tensor("rope_factors_long.weight") or g.tensor("rope_factors_short.weight"):
        raise GgufError("this model uses LongRoPE scaling (rope_factors_long/short), which is not supported")
    k = lambda s: f"{arch}.{s}"

    def need(key):
        v = g.get(k(key))
        if v is None or isinstance(v, (str, list)):
            raise GgufError(f"metadata key {k(key)} is missing")
        return int(v)

    def num(key, default):
        v = g.get(k(key))
        return default if v is None or isinstance(v, (str, list)) else v

    dim, hidden, n_layer, n_head = need("embedding_length"), need("feed_forward_length"), need("block_count"), need("attention.head_count")
    n_kv_head = int(num("attention.head_count_kv", n_head))
    head_dim = int(num("attention.key_length", dim // n_head))
    rot_dim = int(num("rope.dimension_count", head_dim))
    eps = float(num("attention.layer_norm_rms_epsilon", 1e-5))
    rope_base = float(num("rope.freq_base", 10000.0))
    n_ctx_train = int(num("context_length", 2048))
    rope_scale = 1.0
    st = g.get(k("rope.scaling.type"))
    if isinstance(st, str) and st == "linear":
        rope_scale = float(num("rope.scaling.factor", 1.0))
    if n_head % n_kv_head:
        raise GgufError(f"head_count {n_head} is not a multiple of head_count_kv {n_kv_head}")
    swa_window = need("attention.sliding_window") if fl["swa_pattern"] else 0
    if rot_dim > head_dim or rot_dim % 2:
        raise GgufError(f"invalid rope dimension count {rot_dim} for head_dim {head_dim}")
    toks = g.get("tokenizer.ggml.tokens")
    vocab = len(toks) if isinstance(toks, list) else need("vocab_size")
    qd, kvd = n_head * head_dim, n_kv_head * head_dim
    tensors = {}

    def req(tname):
        t = g.tensor(tname)
        if t is None:
            raise GgufError(f"tensor {tname} is missing")
        return t

    def matrix(tname, rows, cols):
        t = req(tname)
        s = _tensor_spec(t)
        if s.rows != rows or s.cols != cols:
            raise GgufError(f"tensor {tname}: expected shape [{cols} x {rows}] (ggml order), found {t.dims}")
        tensors[tname] = s
        return s

    def vector(tname, n):
        t = req(tname)
        s = _tensor_spec(t)
        if s.kind != L.F32:
            raise GgufError(f"tensor {tname}: norm weights must be f32")
        if t.n_elements() != n:
            raise GgufError(f"tensor {tname}: expected {n} elements, found {t.n_elements()}")
        s = Tensor(kind=L.F32, present=1, off=s.off, len=s.len, rows=1, cols=n)
        tensors[tname] = s
        return s

    token_embd = matrix("token_embd.weight", vocab, dim)
    output_norm = vector("output_norm.weight", dim)
    output = matrix("output.weight", vocab, dim) if g.tensor("output.weight") else _absent()
    rope_freqs = _absent()
    if g.tensor("rope_freqs.weight"):
        t = g.tensor("rope_freqs.weight")
        if t.ty != 0 or t.n_elements() != rot_dim // 2:
            raise GgufError(f"rope_freqs.weight must be f32[{rot_dim // 2}]")
        rope_freqs = vector("rope_freqs.weight", rot_dim // 2)
    layers = []
    for i in range(n_layer):
        p = lambda s: f"blk.{i}.{s}.weight"
        b = lambda s: f"blk.{i}.{s}.bias"
        l = Layer()
        l.attn_norm = vector(p("attn_norm"), dim)
        if fl["fused_qkv"]:
            qkv = matrix(p("attn_qkv"), qd + 2 * kvd, dim)
            l.wq, l.wk, l.wv = _rows_view(qkv, 0, qd), _rows_view(qkv, qd, kvd), _rows_view(qkv, qd + kvd, kvd)
        else:
            l.wq, l.wk, l.wv = matrix(p("attn_q"), qd, dim), matrix(p("attn_k"), kvd, dim), matrix(p("attn_v"), kvd, dim)
        l.wo = matrix(p("attn_output"), dim, qd)
        l.ffn_norm = vector(p("ffn_norm"), dim)
        if fl["fused_gate_up"]:
            gu = matrix(p("ffn_up"), 2 * hidden, dim)
            l.gate, l.up = _rows_view(gu, 0, hidden), _rows_view(gu, hidden, hidden)
        else:
            l.gate, l.up = matrix(p("ffn_gate"), hidden, dim), matrix(p("ffn_up"), hidden, dim)
        l.down = matrix(p("ffn_down"), dim, hidden)
        if fl["qkv_bias"]:
            l.bq, l.bk, l.bv = vector(b("attn_q"), qd), vector(b("attn_k"), kvd), vector(b("attn_v"), kvd)
        if fl["qk_norm"]:
            l.q_norm, l.k_norm = vector(p("attn_q_norm"), head_dim), vector(p("attn_k_norm"), head_dim)
        if fl["post_norms"]:
            l.attn_post_norm, l.ffn_post_norm = vector(p("post_attention_norm"), dim), vector(p("post_ffw_norm"), dim)
        l.local_attn = int(fl["swa_pattern"] > 0 and (i + 1) % fl["swa_pattern"] != 0)
        layers.append(l)
    dims = Dims(dim=dim, hidden=hidden, n_layer=n_layer, n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim, rot_dim=rot_dim,
                vocab=vocab, n_ctx_train=n_ctx_train, swa_window=swa_window, eps=eps, rope_base=rope_base, rope_scale=rope_scale,
                rope_base_local=10000.0, rope_scale_local=1.0, qkv_bias=fl["qkv_bias"], qk_norm=fl["qk_norm"],
                rope_neox=fl["rope_neox"], post_norms=fl["post_norms"], gelu=fl["gelu"], embd_scale=fl["embd_scale"])
    head = ModelHead(dims=dims, token_embd=token_embd, output_norm=output_norm, output=output, rope_freqs=rope_freqs)
    return ModelSpec(name=name, head=head, layers=layers, weights=weights, tensors=tensors)


def load_model(path: str) -> ModelSpec:
    """Memory-maps a GGUF file; the returned spec's `weights` is a view of the tensor section."""
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    g = parse(mm, len(mm))
    weights = np.frombuffer(mm, dtype=np.uint8, offset=g.data_offset)
    name = g.get("general.name")
    return model_spec(g, weights, name if isinstance(name, str) else path)


# ---- writer (lib.rs:392-455) ---------------------------------------------------------------------
def _w_string(out: bytearray, s: str):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _value_type(v) -> int:
    if isinstance(v, bool):
        return 7
    if isinstance(v, int):
        return 4 if 0 <= v < 2 ** 32 else (10 if v >= 0 else 11)
    if isinstance(v, float):
        return 6
    if isinstance(v, str):
        return 8
    if isinstance(v, (list, tuple)):
        return 9
    raise TypeError(f"no GGUF value type for {type(v).__name__}")


def _w_value(out: bytearray, v, with_type: bool, vt: int | None = None):
    vt = _value_type(v) if vt is None else vt
    if with_type:
        out += struct.pack("<I", vt)
    if vt == 9:
        et = _value_type(v[0]) if len(v) else 4
        out += struct.pack("<IQ", et, len(v))
        for e in v:
            _w_value(out, e, False, et)
    elif vt == 8:
        _w_string(out, v)
    elif vt == 7:
        out += struct.pack("<B", int(v))
    else:
        out += struct.pack("<" + _Reader._SCALARS[vt], v)


def write(metadata, tensors, alignment: int = DEFAULT_ALIGNMENT) -> bytes:
    """A version-3 file from `metadata` = [(key, value)] and `tensors` = [(name, dims in ggml
    order, ggml type id, bytes)]."""
    out = bytearray(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata)))
    for key, v in metadata:
        _w_string(out, key)
        _w_value(out, v, True)
    off = 0
    for name, dims, ty, data in tensors:
        n = 1
        for d in dims:
            n *= d
        _, blk, size = GGML_TYPES[ty]
        if n // blk * size != len(data):
            raise ValueError(f"tensor {name}: data size mismatch")
        _w_string(out, name)
        out += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)
        off = -(-(off + len(data)) // alignment) * alignment
    out += b"\0" * (-len(out) % alignment)
    for _, _, _, data in tensors:
        out += bytes(data)
        out += b"\0" * (-len(out) % alignment)
    return bytes(out)


def spec_to_gguf(spec: ModelSpec, arch: str) -> bytes:
    """A synthetic model as a GGUF file of architecture `arch` (tests; also a way to hand a
    synthetic model to the reference's own compiler)."""
    d = spec.head.dims
    md = [("general.architecture", arch), ("general.name", spec.name), ("general.alignment", DEFAULT_ALIGNMENT),
          (f"{arch}.embedding_length", d.dim), (f"{arch}.feed_forward_length", d.hidden), (f"{arch}.block_count", d.n_layer),
          (f"{arch}.attention.head_count", d.n_head), (f"{arch}.attention.head_count_kv", d.n_kv_head),
          (f"{arch}.attention.key_length", d.head_dim), (f"{arch}.rope.dimension_count", d.rot_dim),
          (f"{arch}.attention.layer_norm_rms_epsilon", float(d.eps)), (f"{arch}.rope.freq_base", float(d.rope_base)),
          (f"{arch}.context_length", d.n_ctx_train), (f"{arch}.vocab_size", d.vocab)]
    if d.swa_window:
        md.append((f"{arch}.attention.sliding_window", d.swa_window))
    if d.rope_scale != 1.0:
        md += [(f"{arch}.rope.scaling.type", "linear"), (f"{arch}.rope.scaling.factor", float(d.rope_scale))]
    ts = []
    for name, t in spec.tensors.items():
        data = spec.weights[t.off:t.off + t.len]
        dims = [t.cols] if t.rows == 1 and t.kind == L.F32 else [t.cols, t.rows]
        ts.append((name, dims, GGML_OF_KIND[t.kind], data.tobytes()))
    return write(md, ts)
