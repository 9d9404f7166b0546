"""Synthetic models: the tensor table the reference's generator would emit as
`DIMS` / `LAYERS` (crates/aot-codegen/src/emit.rs:399-454) plus a GGUF-style data
section (tensors at 32-byte aligned offsets, rows back to back) filled with
seeded random weights encoded by the library's block encoders.

Real model files cannot be fetched where this runs; these stand in for them with
the same shapes, tensor kinds and value ranges.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import numpy as np

from . import lib as L
from .lib import (BF16, F16, F32, Q4_0, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, Dims, Layer, ModelHead, Tensor, check, ptr,
                  row_bytes)

ALIGN = 32  # GGUF tensor alignment (crates/aot-gguf/src/lib.rs:23)


@dataclass
class ModelSpec:
    name: str
    head: ModelHead
    layers: list
    weights: np.ndarray  # uint8 data section
    tensors: dict = field(default_factory=dict)  # name -> Tensor

    @property
    def dims(self) -> Dims:
        return self.head.dims

    def weight_bytes_per_token(self) -> int:
        """Bytes of weights one decode step reads: every layer matrix and norm, the output
        head and its norm, and one embedding row."""
        d = self.head.dims
        total = 0
        for name, t in self.tensors.items():
            if name == "token_embd.weight":
                tied = not self.head.output.present
                total += row_bytes(t.kind, t.cols) + (t.len if tied else 0)
            else:
                total += t.len
        return total

    def kv_bytes_per_position(self) -> int:
        d = self.head.dims
        return 2 * d.n_layer * d.n_kv_head * d.head_dim * 4


class _Builder:
    def __init__(self, seed: int):
        self.seed = seed
        self.chunks = []
        self.off = 0
        self.n = 0
        self.tensors = {}

    def add(self, name: str, kind: int, rows: int, cols: int, amp: float, offset: float = 0.0) -> Tensor:
        pad = (-self.off) % ALIGN
        if pad:
            self.chunks.append(np.zeros(pad, dtype=np.uint8))
            self.off += pad
        nbytes = rows * row_bytes(kind, cols)
        buf = np.empty(nbytes, dtype=np.uint8)
        self.n += 1
        check(L.synth().aotcu_synth_tensor(kind, rows, cols, amp, offset, self.seed * 1000003 + self.n, ptr(buf)))
        t = Tensor(kind=kind, present=1, off=self.off, len=nbytes, rows=rows, cols=cols)
        self.chunks.append(buf)
        self.off += nbytes
        self.tensors[name] = t
        return t

    def blob(self) -> np.ndarray:
        return np.concatenate(self.chunks) if self.chunks else np.zeros(0, dtype=np.uint8)


def _absent() -> Tensor:
    return Tensor(kind=0, present=0, off=0, len=0, rows=0, cols=0)


def build(name: str, *, dim: int, hidden: int, n_layer: int, n_head: int, n_kv_head: int, head_dim: int, vocab: int,
          rope_base: float = 10000.0, eps: float = 1e-5, qk_norm: bool = False, rope_neox: bool = False,
          qkv_bias: bool = False, n_ctx_train: int = 2048, rot_dim: int | None = None, seed: int = 0x5EED,
          kinds=None, tied_output: bool = False, gelu: bool = False, post_norms: bool = False, embd_scale: bool = False,
          swa_window: int = 0, swa_pattern: int = 0, rope_base_local: float = 10000.0, rope_scale: float = 1.0,
          rope_freqs: bool = False) -> ModelSpec:
    """`kinds(layer_index, tensor_name) -> kind` picks the weight format per matrix;
    tensor_name in {token_embd, output, wq, wk, wv, wo, gate, up, down}.
    The Gemma switches: `gelu` (GeGLU gating), `post_norms` (a norm after attention and after
    the FFN), `embd_scale` (embedding scaled by sqrt(dim)), `swa_window` with `swa_pattern`
    (every layer whose index + 1 is not a multiple of the pattern attends to a sliding
    window and uses the local RoPE base). `rope_scale` is the linear position divisor,
    `rope_freqs` adds the per-frequency divisors tensor of Llama 3 files (rope_freqs.weight)."""
    kinds = kinds or q4_k_m_mix
    b = _Builder(seed)
    qd, kvd = n_head * head_dim, n_kv_head * head_dim
    amp = lambda cols: math.sqrt(3.0 / cols)
    token_embd = b.add("token_embd.weight", kinds(-1, "token_embd"), vocab, dim, 1.0)
    layers = []
    for i in range(n_layer):
        l = Layer()
        l.attn_norm = b.add(f"blk.{i}.attn_norm.weight", F32, 1, dim, 0.5, 1.0)
        l.wq = b.add(f"blk.{i}.attn_q.weight", kinds(i, "wq"), qd, dim, amp(dim))
        l.wk = b.add(f"blk.{i}.attn_k.weight", kinds(i, "wk"), kvd, dim, amp(dim))
        l.wv = b.add(f"blk.{i}.attn_v.weight", kinds(i, "wv"), kvd, dim, amp(dim))
        l.wo = b.add(f"blk.{i}.attn_output.weight", kinds(i, "wo"), dim, qd, amp(qd))
        l.ffn_norm = b.add(f"blk.{i}.ffn_norm.weight", F32, 1, dim, 0.5, 1.0)
        l.gate = b.add(f"blk.{i}.ffn_gate.weight", kinds(i, "gate"), hidden, dim, amp(dim))
        l.up = b.add(f"blk.{i}.ffn_up.weight", kinds(i, "up"), hidden, dim, amp(dim))
        l.down = b.add(f"blk.{i}.ffn_down.weight", kinds(i, "down"), dim, hidden, amp(hidden))
        if qkv_bias:
            l.bq = b.add(f"blk.{i}.attn_q.bias", F32, 1, qd, 0.1)
            l.bk = b.add(f"blk.{i}.attn_k.bias", F32, 1, kvd, 0.1)
            l.bv = b.add(f"blk.{i}.attn_v.bias", F32, 1, kvd, 0.1)
        if qk_norm:
            l.q_norm = b.add(f"blk.{i}.attn_q_norm.weight", F32, 1, head_dim, 0.5, 1.0)
            l.k_norm = b.add(f"blk.{i}.attn_k_norm.weight", F32, 1, head_dim, 0.5, 1.0)
        if post_norms:
            l.attn_post_norm = b.add(f"blk.{i}.post_attention_norm.weight", F32, 1, dim, 0.5, 1.0)
            l.ffn_post_norm = b.add(f"blk.{i}.post_ffw_norm.weight", F32, 1, dim, 0.5, 1.0)
        l.local_attn = int(swa_window > 0 and swa_pattern > 0 and (i + 1) % swa_pattern != 0)
        layers.append(l)
    output_norm = b.add("output_norm.weight", F32, 1, dim, 0.5, 1.0)
    output = _absent() if tied_output else b.add("output.weight", kinds(-1, "output"), vocab, dim, amp(dim))
    dims = Dims(dim=dim, hidden=hidden, n_layer=n_layer, n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim,
                rot_dim=rot_dim or head_dim, vocab=vocab, n_ctx_train=n_ctx_train, swa_window=swa_window, eps=eps,
                rope_base=rope_base, rope_scale=rope_scale, rope_base_local=rope_base_local, rope_scale_local=1.0,
                qkv_bias=int(qkv_bias), qk_norm=int(qk_norm), rope_neox=int(rope_neox), post_norms=int(post_norms),
                gelu=int(gelu), embd_scale=int(embd_scale))
    ff = b.add("rope_freqs.weight", F32, 1, (rot_dim or head_dim) // 2, 3.5, 4.5) if rope_freqs else _absent()
    head = ModelHead(dims=dims, token_embd=token_embd, output_norm=output_norm, output=output, rope_freqs=ff)
    return ModelSpec(name=name, head=head, layers=layers, weights=b.blob(), tensors=b.tensors)


def q4_k_m_mix(layer: int, tensor: str) -> int:
    """The Q4_K_M recipe: Q4_K for most matrices, Q6_K for the output head and for
    attn_v / ffn_down on every other layer."""
    if tensor == "output":
        return Q6_K
    if tensor in ("wv", "down") and layer % 2 == 0:
        return Q6_K
    return Q4_K


def tinyllama(seed: int = 0x5EED, n_layer: int = 22) -> ModelSpec:
    return build("tinyllama-1.1b-shape-q4_k_m", dim=2048, hidden=5632, n_layer=n_layer, n_head=32, n_kv_head=4,
                 head_dim=64, vocab=32000, rope_base=10000.0, eps=1e-5, seed=seed)


def qwen3_8b(seed: int = 0x5EED, n_layer: int = 36) -> ModelSpec:
    return build("qwen3-8b-shape-q4_k_m", dim=4096, hidden=12288, n_layer=n_layer, n_head=32, n_kv_head=8,
                 head_dim=128, vocab=151936, rope_base=1e6, eps=1e-6, qk_norm=True, rope_neox=True,
                 n_ctx_train=40960, seed=seed)


ALL_KINDS = [Q4_K, Q6_K, Q5_K, Q8_0, Q4_0, Q5_0, F16, BF16, F32]


def tiny(arch: str = "llama", seed: int = 11, n_layer: int = 3, kinds=None, dim: int = 256, hidden: int = 512,
         vocab: int = 384) -> ModelSpec:
    """dim-256 models exercising every weight kind (the shape of the reference's e2e
    fixtures, crates/aot-llm/tests/e2e.rs:25-26, 427-458)."""
    order = ["wq", "wk", "wv", "wo", "gate", "up", "down"]

    def spread(layer, tensor):
        if tensor == "token_embd":
            return Q4_K
        if tensor == "output":
            return Q6_K
        return ALL_KINDS[(layer * 7 + order.index(tensor)) % len(ALL_KINDS)]

    kw = dict(dim=dim, hidden=hidden, n_layer=n_layer, n_head=8, n_kv_head=2, head_dim=32, vocab=vocab, seed=seed,
              kinds=kinds or spread, n_ctx_train=512)
    if arch == "qwen3":
        kw.update(qk_norm=True, rope_neox=True, rope_base=1e6, eps=1e-6)
    elif arch == "qwen2":
        kw.update(qkv_bias=True, rope_neox=True, rope_base=1e6, eps=1e-6)
    elif arch == "gemma":
        # Gemma 3 shape: GeGLU, post-norms, scaled embedding, q/k norm, NEOX RoPE, five
        # sliding-window layers (local RoPE base) per global one -- here every third is global
        kw.update(gelu=True, post_norms=True, embd_scale=True, qk_norm=True, rope_neox=True, rope_base=1e6, eps=1e-6,
                  swa_window=16, swa_pattern=3, tied_output=True)
    return build(f"tiny-{arch}", **kw)
