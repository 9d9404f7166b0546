"""ctypes binding of libaot_cuda.so, the C-ABI library declared in include/aot_cuda.h.

This is the same binding shape as the reference's Python example over its C API
(examples/python/aot_llm.py): load the shared object, declare argument types,
raise on a negative status with the library's thread-local error message.
There is no fallback: if the shared object is missing it is built with nvcc, and
if that fails the import raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

HERE = Path(__file__).resolve().parent

# Kind order of crates/aot-kernels/src/quant.rs:34-44.
F32, F16, BF16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = range(9)
KIND_NAMES = ["f32", "f16", "bf16", "q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k"]
BLOCK = [1, 1, 1, 32, 32, 32, 256, 256, 256]
TYPE_SIZE = [4, 2, 2, 18, 22, 34, 144, 176, 210]

# BufId order of crates/aot-kernels/src/metal.rs:205-229.
BUF_NAMES = ["X", "Xb", "Xb2", "Q", "K", "V", "Hb", "Hb2", "Logits", "KCache", "VCache", "RopeCs", "Bx", "Bxb",
             "Bxb2", "Bq", "Bk", "Bv", "Bhb", "Bhb2", "BropeCs", "RopeCsLocal", "BropeCsLocal"]
BUF = {n: i for i, n in enumerate(BUF_NAMES)}

Q8_0_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (32,))])
Q8_K_DTYPE = np.dtype([("d", "<f4"), ("qs", "i1", (256,)), ("bsums", "<i2", (16,))])


def row_bytes(kind: int, cols: int) -> int:
    return cols // BLOCK[kind] * TYPE_SIZE[kind]


def activation(kind: int) -> str:
    return "q8_0" if kind in (Q4_0, Q5_0, Q8_0) else "q8_k" if kind in (Q4_K, Q5_K, Q6_K) else "f32"


class Tensor(C.Structure):
    _fields_ = [("kind", C.c_int32), ("present", C.c_int32), ("off", C.c_uint64), ("len", C.c_uint64),
                ("rows", C.c_uint64), ("cols", C.c_uint64)]


DIM_INT_FIELDS = ("dim", "hidden", "n_layer", "n_head", "n_kv_head", "head_dim", "rot_dim", "vocab", "n_ctx_train",
                  "swa_window")
DIM_FLOAT_FIELDS = ("eps", "rope_base", "rope_scale", "rope_base_local", "rope_scale_local")
DIM_FLAG_FIELDS = ("qkv_bias", "qk_norm", "rope_neox", "post_norms", "gelu", "embd_scale")


class Dims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in DIM_INT_FIELDS] + [(n, C.c_float) for n in DIM_FLOAT_FIELDS] + \
               [(n, C.c_int32) for n in DIM_FLAG_FIELDS]


LAYER_TENSORS = ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "gate", "up", "down", "bq", "bk", "bv", "q_norm",
                 "k_norm", "attn_post_norm", "ffn_post_norm")


class Layer(C.Structure):
    _fields_ = [(n, Tensor) for n in LAYER_TENSORS] + [("local_attn", C.c_int32), ("pad_", C.c_int32)]


class ModelHead(C.Structure):
    _fields_ = [("dims", Dims), ("token_embd", Tensor), ("output_norm", Tensor), ("output", Tensor),
                ("rope_freqs", Tensor)]


class AotCudaError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"aotcu status {status}: {msg}")
        self.status = status


ERR_BAD_ARG, ERR_CUDA, ERR_TIMEOUT, ERR_NCCL, ERR_UNSUPPORTED = -1, -2, -3, -4, -5

# Every symbol include/aot_cuda.h declares: name -> (restype, argtypes). Tests check the
# shared object exports exactly these.
_vp, _sz, _i, _f, _u32 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint32
_pp = C.POINTER(C.c_void_p)
_MV = [_vp, _vp, _vp, _vp, _sz, _sz]
SYMBOLS = {
    "aotcu_last_error": (C.c_char_p, []),
    "aotcu_version": (C.c_char_p, []),
    "aotcu_init": (_i, [_i, _pp]),
    "aotcu_free": (None, [_vp]),
    "aotcu_sync": (_i, [_vp]),
    "aotcu_malloc": (_i, [_vp, _sz, _pp]),
    "aotcu_dev_free": (_i, [_vp, _vp]),
    "aotcu_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "aotcu_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "aotcu_device_status": (_i, [_vp]),
    "aotcu_timer_start": (_i, [_vp]),
    "aotcu_timer_stop": (_i, [_vp, C.POINTER(_f)]),
    "aotcu_quantize_q8_0": (_i, [_vp, _vp, _sz, _vp]),
    "aotcu_quantize_q8_k": (_i, [_vp, _vp, _sz, _vp]),
    "aotcu_dequant_rows": (_i, [_vp, _i, _vp, _vp, _sz, _sz, _vp]),
    "aotcu_matvec": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _sz]),
    "aotcu_matvec_q4_0": (_i, _MV), "aotcu_matvec_q5_0": (_i, _MV), "aotcu_matvec_q8_0": (_i, _MV),
    "aotcu_matvec_q4_k": (_i, _MV), "aotcu_matvec_q5_k": (_i, _MV), "aotcu_matvec_q6_k": (_i, _MV),
    "aotcu_matvec_f16": (_i, _MV), "aotcu_matvec_bf16": (_i, _MV), "aotcu_matvec_f32": (_i, _MV),
    "aotcu_matvec2": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _sz]),
    "aotcu_matvec3": (_i, [_vp, C.POINTER(_i), _pp, _pp, _vp, C.POINTER(_sz), _sz]),
    "aotcu_matmul": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _sz, _sz]),
    "aotcu_matmul2": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "aotcu_matvec_k_static": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _sz]),
    "aotcu_block_sums": (_i, [_vp, _i, _vp, _vp, _sz, _sz, _vp, _vp]),
    "aotcu_block_sums_of": (_i, [_vp, _i, _i, _vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "aotcu_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _f]),
    "aotcu_rmsnorm_heads": (_i, [_vp, _vp, _vp, _sz, _sz, _f]),
    "aotcu_rope": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _vp, _i]),
    "aotcu_silu_mul": (_i, [_vp, _vp, _vp, _sz]),
    "aotcu_gelu_mul": (_i, [_vp, _vp, _vp, _sz]),
    "aotcu_add_inplace": (_i, [_vp, _vp, _vp, _sz]),
    "aotcu_add_bias_rows": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "aotcu_scale_inplace": (_i, [_vp, _vp, _f, _sz]),
    "aotcu_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz]),
    "aotcu_argmax": (_i, [_vp, _vp, _sz, _vp]),
    "aotcu_gpu_new": (_i, [_vp, C.POINTER(ModelHead), C.POINTER(Layer), _vp, _sz, _sz, _sz, _pp]),
    "aotcu_gpu_free": (None, [_vp]),
    "aotcu_gpu_buf": (_i, [_vp, _i, _pp, C.POINTER(_sz)]),
    "aotcu_gpu_read": (_i, [_vp, _i, _sz, _vp, _sz]),
    "aotcu_gpu_write": (_i, [_vp, _i, _sz, _vp, _sz]),
    "aotcu_gpu_begin": (_i, [_vp]),
    "aotcu_gpu_finish": (_i, [_vp]),
    "aotcu_gpu_rmsnorm": (_i, [_vp, _i, _sz, _i, _sz, C.POINTER(Tensor), _sz, _sz, _f, _i]),
    "aotcu_gpu_matmul": (_i, [_vp, _i, _sz, C.POINTER(Tensor), _i, _sz, _sz, _i]),
    "aotcu_gpu_mv3": (_i, [_vp, C.POINTER(_i), C.POINTER(_sz), C.POINTER(C.POINTER(Tensor)), _i, _sz]),
    "aotcu_gpu_gate_up": (_i, [_vp, _i, C.POINTER(Tensor), C.POINTER(Tensor), _i, _sz]),
    "aotcu_gpu_qk_post": (_i, [_vp, _sz, _sz, _sz]),
    "aotcu_gpu_attention": (_i, [_vp, _i, _i, _sz, _sz, _sz, _sz]),
    "aotcu_forward": (_i, [_vp, _u32, _sz, _i]),
    "aotcu_forward_batch": (_i, [_vp, _vp, _sz, _sz, _i]),
    "aotcu_logits": (_i, [_vp, _vp]),
    "aotcu_generate": (_i, [_vp, _u32, _sz, _sz, _vp, C.POINTER(_f)]),
    "aotcu_kv_blob_size": (_sz, [_vp, _sz, _sz]),
    "aotcu_kv_save": (_i, [_vp, _vp, _sz, _sz, _vp, _sz, C.POINTER(_sz)]),
    "aotcu_kv_load": (_i, [_vp, _vp, _sz, _vp, _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "aotcu_gpu_dispatches": (C.c_uint64, [_vp]),
    "aotcu_gpu_set_option": (_i, [_vp, C.c_char_p, _i]),
    "aotcu_bench_gemv_sweep": (_i, [_vp, _i, C.POINTER(_f), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "aotcu_tp_unique_id": (_i, [C.c_char_p, _vp]),
    "aotcu_tp_inbox_handle": (_i, [_vp, _vp]),
    "aotcu_tp_attach": (_i, [_vp, C.c_char_p, _i, _i, _vp, _vp]),
    "aotcu_bench_matmul": (_i, [_vp, _i, _vp, _vp, _sz, _sz, _vp, _sz, _sz, _sz, _i, C.POINTER(_f)]),
    "aotcu_gpu_profile_step": (_i, [_vp, _u32, _sz, _i, _vp]),
    "aotcu_gpu_timeline_step": (_i, [_vp, _u32, _sz, _i, _vp, _vp]),
    "aotcu_row_bytes": (_sz, [_i, _sz]),
}

# Host-only generator of synthetic weights (libaot_synth.so), separate from the CUDA library.
SYNTH_SYMBOLS = {
    "aotcu_synth_quantize_row": (_i, [_i, _vp, _sz, _vp]),
    "aotcu_synth_tensor": (_i, [_i, _sz, _sz, _f, _f, C.c_uint64, _vp]),
    "aotcu_synth_blocks": (_i, [_i, _sz, C.c_uint64, _vp]),
}

_lib = None
_synth = None


def synth() -> C.CDLL:
    """Load (building first if needed) libaot_synth.so."""
    global _synth
    if _synth is None:
        L = C.CDLL(str(_build.build_synth()))
        for name, (res, args) in SYNTH_SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _synth = L
    return _synth


def load() -> C.CDLL:
    """Load (building first if needed) libaot_cuda.so. Raises if it cannot be had."""
    global _lib
    if _lib is None:
        path = _build.build()
        L = C.CDLL(str(path))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> int:
    if status is not None and status < 0:
        raise AotCudaError(status, load().aotcu_last_error().decode(errors="replace"))
    return status


def ptr(a) -> C.c_void_p:
    if a is None:
        return C.c_void_p(None)
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    if isinstance(a, int):
        return C.c_void_p(a)
    return a
