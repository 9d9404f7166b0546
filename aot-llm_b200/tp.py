"""Tensor-parallel decode: row-sharding a model over the GPUs of one box.

The split (one rank per GPU):

* attention: query heads and KV heads are dealt out in contiguous groups, so `attn_q`,
  `attn_k`, `attn_v` lose rows (column-parallel); `attn_output` keeps every row but only the
  columns of this rank's heads (row-parallel) and yields a partial sum;
* FFN: `ffn_gate` / `ffn_up` lose rows, `ffn_down` keeps the matching columns and yields a
  partial sum;
* the output head loses rows: rank r keeps vocabulary rows [r * vocab / world, (r + 1) * vocab /
  world). Each rank finds the best logit of its slice and the ranks exchange {logit, id}
  (the greedy choice is the first maximum of the whole vector, as on one device); the whole
  logits vector is gathered only when the host asks for it. A tied head (the token embedding
  doubles as the output matrix) or a vocabulary that does not divide stays replicated;
* norms and the token embedding are replicated.

Column slices are cut on 256-weight super-block boundaries (32-weight blocks for the Q8_0
family, single weights for float kinds), so every block of a shard is byte-identical to
the block of the full matrix and per-block integer dot products do not change. The two
partial sums per layer are added across ranks by an all-reduce inside the library
(`aotcu_tp_attach`). Only the order of the f32 additions over blocks differs from the
single-device path.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import lib as L
from .lib import Dims, Layer, ModelHead, Tensor, check, row_bytes
from .model import ALIGN, ModelSpec, _absent

_BLOCK = {L.F32: 1, L.F16: 1, L.BF16: 1, L.Q4_0: 32, L.Q5_0: 32, L.Q8_0: 32, L.Q4_K: 256, L.Q5_K: 256, L.Q6_K: 256}


def check_shardable(dims: Dims, world: int, kinds) -> None:
    """Raises ValueError unless heads, FFN rows and the column slices divide evenly."""
    if world < 1:
        raise ValueError("world must be at least 1")
    if dims.n_head % world or dims.n_kv_head % world:
        raise ValueError(f"{dims.n_head} query / {dims.n_kv_head} KV heads do not split {world} ways")
    if dims.hidden % world:
        raise ValueError(f"FFN width {dims.hidden} does not split {world} ways")
    qd = dims.n_head * dims.head_dim
    for name, cols in (("attn_output", qd), ("ffn_down", dims.hidden)):
        blk = max(_BLOCK[k] for k in kinds[name])
        if (cols // world) % blk or cols % world:
            raise ValueError(f"{name}: {cols} columns do not split {world} ways on {blk}-weight block boundaries")
    for name, rows in (("ffn_gate", dims.hidden),):
        # the gate/up rows of a rank must be the rows whose ffn_down columns it keeps
        if rows % world:
            raise ValueError(f"{name}: {rows} rows do not split {world} ways")


class _Blob:
    def __init__(self):
        self.chunks, self.off = [], 0

    def add(self, data: np.ndarray, kind: int, rows: int, cols: int) -> Tensor:
        pad = (-self.off) % ALIGN
        if pad:
            self.chunks.append(np.zeros(pad, dtype=np.uint8))
            self.off += pad
        t = Tensor(kind=kind, present=1, off=self.off, len=data.nbytes, rows=rows, cols=cols)
        self.chunks.append(np.ascontiguousarray(data))
        self.off += data.nbytes
        return t

    def blob(self) -> np.ndarray:
        return np.concatenate(self.chunks) if self.chunks else np.zeros(0, dtype=np.uint8)


def _bytes_of(spec: ModelSpec, t: Tensor) -> np.ndarray:
    return spec.weights[t.off:t.off + t.len]


def slice_rows(spec: ModelSpec, t: Tensor, r0: int, r1: int):
    rb = row_bytes(t.kind, t.cols)
    return _bytes_of(spec, t)[r0 * rb:r1 * rb], r1 - r0, t.cols


def slice_cols(spec: ModelSpec, t: Tensor, c0: int, c1: int):
    """Columns [c0, c1) of every row; c0 and c1 must fall on block boundaries of the kind."""
    blk = _BLOCK[t.kind]
    if c0 % blk or c1 % blk:
        raise ValueError("column slice off a block boundary")
    rb = row_bytes(t.kind, t.cols)
    bs = rb * blk // t.cols  # bytes per block
    data = _bytes_of(spec, t).reshape(t.rows, rb)[:, c0 // blk * bs:c1 // blk * bs]
    return np.ascontiguousarray(data).reshape(-1), t.rows, c1 - c0


def shard_spec(spec: ModelSpec, rank: int, world: int, shard_head: bool = True) -> ModelSpec:
    """The model one rank of `world` holds. world == 1 returns the spec unchanged.
    `shard_head=False` keeps the whole output head on every rank."""
    if world == 1:
        return spec
    if not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    d = spec.head.dims
    kinds = {"attn_output": [l.wo.kind for l in spec.layers], "ffn_down": [l.down.kind for l in spec.layers]}
    check_shardable(d, world, kinds)
    if d.post_norms or d.swa_window:
        raise ValueError("post-norm / sliding-window models are not sharded")
    hd = d.head_dim
    nh, nkv, hid = d.n_head // world, d.n_kv_head // world, d.hidden // world
    b = _Blob()
    tensors = {}

    def put(name, data, kind, rows, cols):
        t = b.add(data, kind, rows, cols)
        tensors[name] = t
        return t

    def whole(name, t):
        return put(name, _bytes_of(spec, t), t.kind, t.rows, t.cols) if t.present else _absent()

    token_embd = whole("token_embd.weight", spec.head.token_embd)
    layers = []
    for i, l in enumerate(spec.layers):
        n = Layer()
        n.attn_norm = whole(f"blk.{i}.attn_norm.weight", l.attn_norm)
        n.wq = put(f"blk.{i}.attn_q.weight", *slice_rows(spec, l.wq, rank * nh * hd, (rank + 1) * nh * hd)[:1], l.wq.kind, nh * hd, l.wq.cols)
        n.wk = put(f"blk.{i}.attn_k.weight", *slice_rows(spec, l.wk, rank * nkv * hd, (rank + 1) * nkv * hd)[:1], l.wk.kind, nkv * hd, l.wk.cols)
        n.wv = put(f"blk.{i}.attn_v.weight", *slice_rows(spec, l.wv, rank * nkv * hd, (rank + 1) * nkv * hd)[:1], l.wv.kind, nkv * hd, l.wv.cols)
        data, rows, cols = slice_cols(spec, l.wo, rank * nh * hd, (rank + 1) * nh * hd)
        n.wo = put(f"blk.{i}.attn_output.weight", data, l.wo.kind, rows, cols)
        n.ffn_norm = whole(f"blk.{i}.ffn_norm.weight", l.ffn_norm)
        n.gate = put(f"blk.{i}.ffn_gate.weight", *slice_rows(spec, l.gate, rank * hid, (rank + 1) * hid)[:1], l.gate.kind, hid, l.gate.cols)
        n.up = put(f"blk.{i}.ffn_up.weight", *slice_rows(spec, l.up, rank * hid, (rank + 1) * hid)[:1], l.up.kind, hid, l.up.cols)
        data, rows, cols = slice_cols(spec, l.down, rank * hid, (rank + 1) * hid)
        n.down = put(f"blk.{i}.ffn_down.weight", data, l.down.kind, rows, cols)
        if d.qkv_bias:
            n.bq = put(f"blk.{i}.attn_q.bias", *slice_cols(spec, l.bq, rank * nh * hd, (rank + 1) * nh * hd)[:1], L.F32, 1, nh * hd)
            n.bk = put(f"blk.{i}.attn_k.bias", *slice_cols(spec, l.bk, rank * nkv * hd, (rank + 1) * nkv * hd)[:1], L.F32, 1, nkv * hd)
            n.bv = put(f"blk.{i}.attn_v.bias", *slice_cols(spec, l.bv, rank * nkv * hd, (rank + 1) * nkv * hd)[:1], L.F32, 1, nkv * hd)
        if d.qk_norm:
            n.q_norm = whole(f"blk.{i}.attn_q_norm.weight", l.q_norm)
            n.k_norm = whole(f"blk.{i}.attn_k_norm.weight", l.k_norm)
        n.local_attn = l.local_attn
        layers.append(n)
    output_norm = whole("output_norm.weight", spec.head.output_norm)
    out_t = spec.head.output
    if out_t.present and shard_head and d.vocab % world == 0:
        per = d.vocab // world
        output = put("output.weight", slice_rows(spec, out_t, rank * per, (rank + 1) * per)[0], out_t.kind, per, out_t.cols)
    else:
        output = whole("output.weight", out_t)
    nd = Dims()
    C.memmove(C.byref(nd), C.byref(d), C.sizeof(Dims))
    nd.n_head, nd.n_kv_head, nd.hidden = nh, nkv, hid
    head = ModelHead(dims=nd, token_embd=token_embd, output_norm=output_norm, output=output,
                     rope_freqs=whole("rope_freqs.weight", spec.head.rope_freqs))
    return ModelSpec(name=f"{spec.name}[{rank}/{world}]", head=head, layers=layers, weights=b.blob(), tensors=tensors)


def nccl_library_path() -> str:
    """The NCCL shared object that ships with the installed torch (the one its NCCL backend
    loads), else the loader's default."""
    try:
        import nvidia.nccl  # type: ignore
        for base in nvidia.nccl.__path__:
            p = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except Exception:
        pass
    return "libnccl.so.2"


def unique_id(nccl_library: str | None = None) -> bytes:
    buf = (C.c_uint8 * 128)()
    check(L.load().aotcu_tp_unique_id((nccl_library or nccl_library_path()).encode(), buf))
    return bytes(buf)


def inbox_handle(gpu) -> bytes:
    """This rank's inbox for the other ranks' partial rows, as a 64-byte CUDA IPC handle."""
    buf = (C.c_uint8 * 64)()
    check(L.load().aotcu_tp_inbox_handle(gpu.h, buf))
    return bytes(buf)


def attach(gpu, rank: int, world: int, uid: bytes, nccl_library: str | None = None, peer_handles: bytes | None = None) -> None:
    """Collective: every rank calls it with the same 128-byte id (from `unique_id` on one rank).
    `peer_handles` = the ranks' inbox handles in rank order (world x 64 bytes) keeps the decode
    step's exchange inside the one-kernel step; None sends every exchange through NCCL."""
    if len(uid) != 128:
        raise ValueError("the id is 128 bytes")
    buf = (C.c_uint8 * 128).from_buffer_copy(uid)
    ph = None
    if peer_handles is not None:
        if len(peer_handles) != 64 * world:
            raise ValueError("peer_handles holds 64 bytes per rank")
        ph = (C.c_uint8 * len(peer_handles)).from_buffer_copy(peer_handles)
    check(L.load().aotcu_tp_attach(gpu.h, (nccl_library or nccl_library_path()).encode(), rank, world, buf, ph))


def gather_handles(ranks, mine: bytes) -> bytes:
    """All ranks' 64-byte handles in rank order, through the process group."""
    if ranks.info.world == 1:
        return mine
    import torch
    import torch.distributed as dist
    dev = ranks._device
    t = torch.tensor(list(mine), dtype=torch.uint8, device=dev)
    outs = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in range(ranks.info.world)]
    dist.all_gather(outs, t)
    return b"".join(bytes(o.cpu().tolist()) for o in outs)


def join(gpu, ranks, fused: bool = True, nccl_library: str | None = None) -> None:
    """The whole hand-shake for one rank: id from rank 0, inbox handles from everyone, attach."""
    info = ranks.info
    uid = exchange_id(ranks, lambda: unique_id(nccl_library))
    handles = gather_handles(ranks, inbox_handle(gpu)) if fused and info.world > 1 else None
    attach(gpu, info.rank, info.world, uid, nccl_library, handles)


def exchange_id(ranks, make_id) -> bytes:
    """Rank 0 makes the id; the others get it through the process group (any backend)."""
    if ranks.info.world == 1:
        return make_id()
    import torch
    import torch.distributed as dist
    dev = ranks._device
    t = torch.zeros(128, dtype=torch.uint8, device=dev)
    if ranks.info.rank == 0:
        t = torch.tensor(list(make_id()), dtype=torch.uint8, device=dev)
    dist.broadcast(t, src=0)
    return bytes(t.cpu().tolist())
