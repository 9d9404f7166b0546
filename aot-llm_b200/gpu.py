"""Host-side mirror of the reference's runtime interface for the hot path.

Names follow crates/aot-kernels: the kernel functions (`matvec_q4_k`, `matmul_*`,
`quantize_q8_k`, `rmsnorm`, `rope`, `attention`, ...) and the GPU backend slot
(`Gpu` with `BufId`s, crates/aot-kernels/src/metal.rs:205-229, 361-813). Everything
here is a thin call into the C-ABI library; there is no computation in Python.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import lib as L
from .lib import BUF, Dims, Layer, ModelHead, Tensor, check, ptr


class DeviceBuffer:
    """A device allocation owned by a Context (padded at the end, see aotcu_malloc)."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(L.load().aotcu_malloc(ctx.h, max(self.nbytes, 1), C.byref(p)))
        self.ptr = p.value

    def free(self):
        if self.ptr and self.ctx.h:
            L.load().aotcu_dev_free(self.ctx.h, C.c_void_p(self.ptr))
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def at(self, byte_offset: int) -> int:
        return self.ptr + byte_offset

    def upload(self, host: np.ndarray, byte_offset: int = 0):
        host = np.ascontiguousarray(host)
        assert byte_offset + host.nbytes <= self.nbytes
        check(L.load().aotcu_h2d(self.ctx.h, C.c_void_p(self.ptr + byte_offset), ptr(host), host.nbytes))
        return self

    def download(self, dtype, count: int, byte_offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        assert byte_offset + out.nbytes <= self.nbytes
        check(L.load().aotcu_d2h(self.ctx.h, ptr(out), C.c_void_p(self.ptr + byte_offset), out.nbytes))
        return out


class Context:
    """One CUDA device + stream (aotcu_ctx); the role `Pool` plays in the reference's
    kernel signatures."""

    def __init__(self, device: int = 0):
        self.h = None
        h = C.c_void_p()
        check(L.load().aotcu_init(device, C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if self.h:
            # the library frees the context's Gpus with it; drop their handles first
            for g in list(getattr(self, "_gpus", ())):
                g.close()
            L.load().aotcu_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        check(L.load().aotcu_sync(self.h))

    def timer_start(self):
        check(L.load().aotcu_timer_start(self.h))

    def timer_stop(self) -> float:
        ms = C.c_float(0)
        check(L.load().aotcu_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def device_status(self):
        check(L.load().aotcu_device_status(self.h))

    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def to_device(self, host: np.ndarray) -> DeviceBuffer:
        host = np.ascontiguousarray(host)
        return DeviceBuffer(self, host.nbytes).upload(host)

    # ---- quant.rs --------------------------------------------------------------------
    def quantize_q8_0(self, x: DeviceBuffer, n: int, out: DeviceBuffer):
        check(L.load().aotcu_quantize_q8_0(self.h, x.ptr, n, out.ptr))

    def quantize_q8_k(self, x: DeviceBuffer, n: int, out: DeviceBuffer):
        check(L.load().aotcu_quantize_q8_k(self.h, x.ptr, n, out.ptr))

    def dequant_rows(self, kind: int, table: DeviceBuffer, row_ids: DeviceBuffer, n_rows: int, cols: int,
                     out: DeviceBuffer):
        check(L.load().aotcu_dequant_rows(self.h, kind, table.ptr, row_ids.ptr, n_rows, cols, out.ptr))

    # ---- matvec.rs -------------------------------------------------------------------
    def matvec(self, kind: int, out, w, x, rows: int, cols: int):
        fn = getattr(L.load(), "aotcu_matvec_" + L.KIND_NAMES[kind])
        check(fn(self.h, _dp(out), _dp(w), _dp(x), rows, cols))

    def matvec2(self, kind: int, out_a, out_b, w_a, w_b, x, rows: int, cols: int):
        check(L.load().aotcu_matvec2(self.h, kind, _dp(out_a), _dp(out_b), _dp(w_a), _dp(w_b), _dp(x), rows, cols))

    def matvec3(self, kinds, outs, ws, x, rows3, cols: int):
        k = (C.c_int * 3)(*kinds)
        o = (C.c_void_p * 3)(*[_dp(b) for b in outs])
        w = (C.c_void_p * 3)(*[_dp(b) for b in ws])
        r = (C.c_size_t * 3)(*rows3)
        check(L.load().aotcu_matvec3(self.h, k, o, w, _dp(x), r, cols))

    def matmul(self, kind: int, out, w, xs, m: int, rows: int, cols: int):
        check(L.load().aotcu_matmul(self.h, kind, _dp(out), _dp(w), _dp(xs), m, rows, cols))

    def matmul2(self, kind: int, out_a, out_b, w_a, w_b, xs, m: int, rows: int, cols: int):
        check(L.load().aotcu_matmul2(self.h, kind, _dp(out_a), _dp(out_b), _dp(w_a), _dp(w_b), _dp(xs), m, rows, cols))

    def bench_matmul(self, kind: int, out, w, copy_stride: int, n_copies: int, xs, m: int, rows: int, cols: int,
                     iters: int) -> float:
        """Average milliseconds per launch of the (m x cols) by (rows x cols) product, timed on the
        device over `iters` back-to-back launches that rotate through `n_copies` copies of `w`."""
        ms = C.c_float(0.0)
        check(L.load().aotcu_bench_matmul(self.h, kind, _dp(out), _dp(w), copy_stride, n_copies, _dp(xs), m, rows, cols,
                                          iters, C.byref(ms)))
        return float(ms.value)

    def matvec_k_static(self, kind: int, out, w, x_f32, rows: int, cols: int):
        """K-quant product of an f32 device vector through the library's built-in activation
        area: no device allocation anywhere on this call path (see include/aot_cuda.h)."""
        check(L.load().aotcu_matvec_k_static(self.h, kind, _dp(out), _dp(w), _dp(x_f32), rows, cols))

    def block_sums_of(self, kernel: int, kind: int, w, x, m: int, rows: int, cols: int, sumi, summ):
        """Integer block sums as production kernel `kernel` forms them (0 streaming row product, 1 tcgen05)."""
        check(L.load().aotcu_block_sums_of(self.h, kernel, kind, _dp(w), _dp(x), m, rows, cols, _dp(sumi), _dp(summ)))

    def block_sums(self, kind: int, w, x, rows: int, cols: int, sumi, summ=None):
        check(L.load().aotcu_block_sums(self.h, kind, _dp(w), _dp(x), rows, cols, _dp(sumi),
                                        _dp(summ) if summ is not None else None))

    # ---- ops.rs / sampler.rs ------------------------------------------------------------
    def rmsnorm(self, out, x, w, n: int, m: int, eps: float):
        check(L.load().aotcu_rmsnorm(self.h, _dp(out), _dp(x), _dp(w), n, m, eps))

    def rmsnorm_heads(self, x, w, n_heads: int, head_dim: int, eps: float):
        check(L.load().aotcu_rmsnorm_heads(self.h, _dp(x), _dp(w), n_heads, head_dim, eps))

    def rope(self, x, m: int, n_heads: int, head_dim: int, rot_dim: int, cs, neox: bool = False):
        check(L.load().aotcu_rope(self.h, _dp(x), m, n_heads, head_dim, rot_dim, _dp(cs), int(neox)))

    def silu_mul(self, h, up, n: int):
        check(L.load().aotcu_silu_mul(self.h, _dp(h), _dp(up), n))

    def gelu_mul(self, h, up, n: int):
        check(L.load().aotcu_gelu_mul(self.h, _dp(h), _dp(up), n))

    def add_inplace(self, x, y, n: int):
        check(L.load().aotcu_add_inplace(self.h, _dp(x), _dp(y), n))

    def add_bias_rows(self, x, b, n: int, m: int):
        check(L.load().aotcu_add_bias_rows(self.h, _dp(x), _dp(b), n, m))

    def scale_inplace(self, x, s: float, n: int):
        check(L.load().aotcu_scale_inplace(self.h, _dp(x), s, n))

    def attention(self, out, q, k_cache, v_cache, n_head, n_kv_head, head_dim, ctx_len, pos0, m, window=0):
        check(L.load().aotcu_attention(self.h, _dp(out), _dp(q), _dp(k_cache), _dp(v_cache), n_head, n_kv_head,
                                       head_dim, ctx_len, pos0, m, window))

    def argmax(self, x, n: int, out_token):
        check(L.load().aotcu_argmax(self.h, _dp(x), n, _dp(out_token)))

    # ---- host-buffer conveniences (upload, run, download) --------------------------------------
    def host_quantize(self, act: str, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        dx = self.to_device(x)
        if act == "q8_k":
            out = self.alloc(x.size // 256 * 292)
            self.quantize_q8_k(dx, x.size, out)
            return out.download(L.Q8_K_DTYPE, x.size // 256)
        out = self.alloc(x.size // 32 * 36)
        self.quantize_q8_0(dx, x.size, out)
        return out.download(L.Q8_0_DTYPE, x.size // 32)

    def host_matmul(self, kind: int, w: np.ndarray, x_f32: np.ndarray, m: int, rows: int, cols: int) -> np.ndarray:
        """Quantize `m` host activation rows as the kind requires and multiply; every copy
        crosses PCIe, which is what an end-to-end caller with host buffers pays."""
        dw = self.to_device(np.ascontiguousarray(w, dtype=np.uint8))
        x_f32 = np.ascontiguousarray(x_f32, dtype=np.float32).reshape(m, cols)
        dx = self.to_device(x_f32)
        act = L.activation(kind)
        if act == "q8_k":
            xq = self.alloc(m * cols // 256 * 292)
            self.quantize_q8_k(dx, m * cols, xq)
        elif act == "q8_0":
            xq = self.alloc(m * cols // 32 * 36)
            self.quantize_q8_0(dx, m * cols, xq)
        else:
            xq = dx
        out = self.alloc(m * rows * 4)
        self.matmul(kind, out, dw, xq, m, rows, cols)
        return out.download(np.float32, m * rows).reshape(m, rows)


def _dp(b):
    if b is None:
        return C.c_void_p(None)
    if isinstance(b, DeviceBuffer):
        return C.c_void_p(b.ptr)
    if isinstance(b, int):
        return C.c_void_p(b)
    return b


class Gpu:
    """The GPU backend object the generated `forward_gpu` drives in the reference
    (`Gpu::new/begin/finish/rmsnorm/mv/mv3/matmul/gate_up/rope_ex/attention`,
    crates/aot-kernels/src/metal.rs:361-813), over CUDA. Weights are uploaded once;
    State buffers and the KV cache live in HBM."""

    def __init__(self, ctx: Context, head: ModelHead, layers, weights: np.ndarray, n_ctx: int, max_batch: int = 1):
        self.ctx = ctx
        self.head = head
        self.layers = (Layer * len(layers))(*layers)
        self.n_ctx = n_ctx
        self.max_batch = max_batch
        weights = np.ascontiguousarray(weights, dtype=np.uint8)
        self.h = None
        h = C.c_void_p()
        check(L.load().aotcu_gpu_new(ctx.h, C.byref(head), self.layers, ptr(weights), weights.size, n_ctx, max_batch,
                                     C.byref(h)))
        self.h = h
        if not hasattr(ctx, "_gpus"):
            ctx._gpus = weakref.WeakSet()
        ctx._gpus.add(self)

    def close(self):
        if self.h:
            if self.ctx.h:
                L.load().aotcu_gpu_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- buffers
    def buf_len(self, name: str) -> int:
        p, n = C.c_void_p(), C.c_size_t()
        check(L.load().aotcu_gpu_buf(self.h, BUF[name], C.byref(p), C.byref(n)))
        return n.value

    def buf_ptr(self, name: str) -> int:
        p, n = C.c_void_p(), C.c_size_t()
        check(L.load().aotcu_gpu_buf(self.h, BUF[name], C.byref(p), C.byref(n)))
        return p.value

    def read(self, name: str, n: int | None = None, offset: int = 0) -> np.ndarray:
        n = self.buf_len(name) - offset if n is None else n
        out = np.empty(n, dtype=np.float32)
        check(L.load().aotcu_gpu_read(self.h, BUF[name], offset, ptr(out), n))
        return out

    def write(self, name: str, data: np.ndarray, offset: int = 0):
        data = np.ascontiguousarray(data, dtype=np.float32)
        check(L.load().aotcu_gpu_write(self.h, BUF[name], offset, ptr(data), data.size))

    # -- operator level (metal.rs)
    def begin(self):
        check(L.load().aotcu_gpu_begin(self.h))

    def finish(self):
        check(L.load().aotcu_gpu_finish(self.h))

    def rmsnorm(self, dst: str, src: str, w: Tensor, n: int, m: int, eps: float, dst_off=0, src_off=0,
                accumulate=False):
        check(L.load().aotcu_gpu_rmsnorm(self.h, BUF[dst], dst_off, BUF[src], src_off, C.byref(w), n, m, eps,
                                         int(accumulate)))

    def matmul(self, dst: str, w: Tensor, src: str, m: int = 1, accumulate=False, dst_off=0, src_off=0):
        check(L.load().aotcu_gpu_matmul(self.h, BUF[dst], dst_off, C.byref(w), BUF[src], src_off, m, int(accumulate)))

    mv = matmul

    def mv3(self, dsts, ws, src: str, m: int = 1, dst_offs=(0, 0, 0)):
        d = (C.c_int * 3)(*[BUF[x] for x in dsts])
        o = (C.c_size_t * 3)(*dst_offs)
        w = (C.POINTER(Tensor) * 3)(*[C.pointer(t) for t in ws])
        check(L.load().aotcu_gpu_mv3(self.h, d, o, w, BUF[src], m))

    def gate_up(self, dst: str, gate: Tensor, up: Tensor, src: str, m: int = 1):
        check(L.load().aotcu_gpu_gate_up(self.h, BUF[dst], C.byref(gate), C.byref(up), BUF[src], m))

    def qk_post(self, layer: int, pos0: int, m: int = 1):
        check(L.load().aotcu_gpu_qk_post(self.h, layer, pos0, m))

    def attention(self, dst: str, q: str, layer: int, pos0: int, m: int = 1, window: int = 0):
        check(L.load().aotcu_gpu_attention(self.h, BUF[dst], BUF[q], layer, pos0, m, window))

    # -- step level (emit.rs forward / forward_batch)
    def forward(self, token: int, pos: int, want_logits: bool = True):
        check(L.load().aotcu_forward(self.h, token, pos, int(want_logits)))

    def forward_batch(self, tokens, pos0: int, want_logits: bool = True):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        check(L.load().aotcu_forward_batch(self.h, ptr(t), t.size, pos0, int(want_logits)))

    def logits(self) -> np.ndarray:
        out = np.empty(self.head.dims.vocab, dtype=np.float32)
        check(L.load().aotcu_logits(self.h, ptr(out)))
        return out

    def generate(self, token: int, pos: int, n_steps: int):
        """Greedy decode on the device; returns (ids, device milliseconds)."""
        out = np.zeros(n_steps, dtype=np.uint32)
        ms = C.c_float(0)
        check(L.load().aotcu_generate(self.h, token, pos, n_steps, ptr(out), C.byref(ms)))
        return out, ms.value

    def gemv_sweep(self, iters: int = 20):
        """(ms per sweep, launches per sweep, algorithmic bytes per sweep) of the decode
        step's matrix products alone."""
        ms, n, b = C.c_float(0), C.c_uint64(0), C.c_uint64(0)
        check(L.load().aotcu_bench_gemv_sweep(self.h, iters, C.byref(ms), C.byref(n), C.byref(b)))
        return ms.value, n.value, b.value

    def profile_step(self, token: int, pos: int, cta: int = 0) -> np.ndarray:
        out = np.zeros(32, dtype=np.uint64)
        check(L.load().aotcu_gpu_profile_step(self.h, token, pos, cta, ptr(out)))
        return out

    def timeline_step(self, token: int, pos: int, layer: int) -> np.ndarray:
        """[n_cta, 16] device-timer nanoseconds at which each CTA left each phase of `layer`."""
        out = np.zeros(16 * 256, dtype=np.uint64)
        n = C.c_int(0)
        check(L.load().aotcu_gpu_timeline_step(self.h, token, pos, layer, ptr(out), C.byref(n)))
        return out.reshape(256, 16)[: n.value]

    def kv_save(self, tokens, n_cached: int) -> bytes:
        """The "AOTP" v2 blob of `tokens` and the cache rows of their first `n_cached`
        positions (prefix::serialize, crates/aot-kernels/src/prefix.rs:112-141)."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        size = L.load().aotcu_kv_blob_size(self.h, toks.size, n_cached)
        out = np.empty(size, dtype=np.uint8)
        n = C.c_size_t(0)
        check(L.load().aotcu_kv_save(self.h, ptr(toks), toks.size, n_cached, ptr(out), out.size, C.byref(n)))
        return out[: n.value].tobytes()

    def kv_load(self, blob: bytes):
        """Restores a saved cache into positions [0, n_cached) and returns (tokens, n_cached)
        (Prefix::parse + load_into, prefix.rs:45-103). Raises AotCudaError for a blob that is
        not a cache of this model."""
        raw = np.frombuffer(blob, dtype=np.uint8)
        cap = max(1, (len(blob) - 24) // 4)
        toks = np.zeros(cap, dtype=np.uint32)
        n, nc = C.c_size_t(0), C.c_size_t(0)
        check(L.load().aotcu_kv_load(self.h, ptr(raw), raw.size, ptr(toks), toks.size, C.byref(n), C.byref(nc)))
        return toks[: n.value].tolist(), nc.value

    def dispatches(self) -> int:
        return L.load().aotcu_gpu_dispatches(self.h)

    def set_option(self, name: str, value: int) -> int:
        """Sets a tuning switch; query names ("mega_available") return their value."""
        return check(L.load().aotcu_gpu_set_option(self.h, name.encode(), value))
