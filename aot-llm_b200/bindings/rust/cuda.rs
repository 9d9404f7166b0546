//! CUDA backend for generated aot-llm projects: `src/rt/cuda.rs`.
//!
//! The counterpart of `rt/metal.rs` for NVIDIA GPUs. It binds `libaot_cuda.so` (declared in
//! `include/aot_cuda.h`) at the step level: the whole generated forward pass runs on the
//! device, so `forward_gpu` / `forward_batch_gpu` of the generated `model.rs` shrink to one
//! call each (see `emit_cuda_forwards.rs` for the generator side). Results are bit-identical
//! to the CPU path (`forward` / `forward_batch`), including the logits the sampler reads.
//!
//! This file is written against the reference's runtime types (`rt::state::{Dims, Tensor,
//! State}`, `rt::quant::Kind`); it has not been compiled where it was written (no Rust
//! toolchain there). The C side of every declaration below is exercised by the C client in
//! `bindings/c/client.c` and by the ctypes binding of the test-suite.

use std::ffi::CStr;
use std::os::raw::{c_char, c_int};

use super::quant::Kind;
use super::state::{Dims, State, Tensor};

// ---- C ABI (include/aot_cuda.h) -------------------------------------------------------------

#[repr(C)]
#[derive(Clone, Copy)]
pub struct AotcuTensor {
    pub kind: i32,
    pub present: i32,
    pub off: u64,
    pub len: u64,
    pub rows: u64,
    pub cols: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct AotcuDims {
    pub dim: i32,
    pub hidden: i32,
    pub n_layer: i32,
    pub n_head: i32,
    pub n_kv_head: i32,
    pub head_dim: i32,
    pub rot_dim: i32,
    pub vocab: i32,
    pub n_ctx_train: i32,
    pub swa_window: i32,
    pub eps: f32,
    pub rope_base: f32,
    pub rope_scale: f32,
    pub rope_base_local: f32,
    pub rope_scale_local: f32,
    pub qkv_bias: i32,
    pub qk_norm: i32,
    pub rope_neox: i32,
    pub post_norms: i32,
    pub gelu: i32,
    pub embd_scale: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct AotcuLayer {
    pub attn_norm: AotcuTensor,
    pub wq: AotcuTensor,
    pub wk: AotcuTensor,
    pub wv: AotcuTensor,
    pub wo: AotcuTensor,
    pub ffn_norm: AotcuTensor,
    pub gate: AotcuTensor,
    pub up: AotcuTensor,
    pub down: AotcuTensor,
    pub bq: AotcuTensor,
    pub bk: AotcuTensor,
    pub bv: AotcuTensor,
    pub q_norm: AotcuTensor,
    pub k_norm: AotcuTensor,
    pub attn_post_norm: AotcuTensor,
    pub ffn_post_norm: AotcuTensor,
    pub local_attn: i32,
    pub pad_: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct AotcuModelHead {
    pub dims: AotcuDims,
    pub token_embd: AotcuTensor,
    pub output_norm: AotcuTensor,
    pub output: AotcuTensor,
    pub rope_freqs: AotcuTensor,
}

#[repr(C)]
pub struct AotcuCtx {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct AotcuGpu {
    _opaque: [u8; 0],
}

#[link(name = "aot_cuda")]
extern "C" {
    fn aotcu_last_error() -> *const c_char;
    fn aotcu_init(device: c_int, out: *mut *mut AotcuCtx) -> c_int;
    fn aotcu_free(ctx: *mut AotcuCtx);
    fn aotcu_gpu_new(
        ctx: *mut AotcuCtx,
        head: *const AotcuModelHead,
        layers: *const AotcuLayer,
        weights: *const u8,
        weights_len: usize,
        n_ctx: usize,
        max_batch: usize,
        out: *mut *mut AotcuGpu,
    ) -> c_int;
    fn aotcu_gpu_free(g: *mut AotcuGpu);
    fn aotcu_forward(g: *mut AotcuGpu, token: u32, pos: usize, want_logits: c_int) -> c_int;
    fn aotcu_forward_batch(g: *mut AotcuGpu, tokens: *const u32, n: usize, pos0: usize, want_logits: c_int) -> c_int;
    fn aotcu_logits(g: *mut AotcuGpu, host_dst: *mut f32) -> c_int;
    fn aotcu_generate(g: *mut AotcuGpu, token: u32, pos: usize, n_steps: usize, out_tokens: *mut u32, elapsed_ms: *mut f32) -> c_int;
    fn aotcu_kv_blob_size(g: *const AotcuGpu, n_tokens: usize, n_cached: usize) -> usize;
    fn aotcu_kv_save(g: *mut AotcuGpu, tokens: *const u32, n_tokens: usize, n_cached: usize, out: *mut u8, out_cap: usize, out_len: *mut usize) -> c_int;
    fn aotcu_kv_load(g: *mut AotcuGpu, blob: *const u8, blob_len: usize, tokens_out: *mut u32, tokens_cap: usize, n_tokens: *mut usize, n_cached: *mut usize) -> c_int;
    fn aotcu_gpu_dispatches(g: *mut AotcuGpu) -> u64;
}

fn last_error() -> String {
    // SAFETY: the library returns a NUL-terminated thread-local string, never NULL.
    unsafe { CStr::from_ptr(aotcu_last_error()) }.to_string_lossy().into_owned()
}

fn check(rc: c_int) -> Result<(), String> {
    if rc == 0 {
        Ok(())
    } else {
        Err(format!("aot_cuda: {} (status {rc})", last_error()))
    }
}

// ---- description of the model ---------------------------------------------------------------

/// Tensor kinds in the order of `rt::quant::Kind` (quant.rs:34-44), which is the order of the
/// library's `kind` field.
pub const fn kind_id(k: Kind) -> i32 {
    match k {
        Kind::F32 => 0,
        Kind::F16 => 1,
        Kind::BF16 => 2,
        Kind::Q4_0 => 3,
        Kind::Q5_0 => 4,
        Kind::Q8_0 => 5,
        Kind::Q4_K => 6,
        Kind::Q5_K => 7,
        Kind::Q6_K => 8,
    }
}

pub const ABSENT: AotcuTensor = AotcuTensor { kind: 0, present: 0, off: 0, len: 0, rows: 0, cols: 0 };

/// `rt::state::Tensor` without its name (state.rs:165-180).
pub const fn tensor(t: &Tensor) -> AotcuTensor {
    AotcuTensor { kind: kind_id(t.kind), present: 1, off: t.off as u64, len: t.len as u64, rows: t.rows as u64, cols: t.cols as u64 }
}

pub const fn tensor_opt(t: Option<&Tensor>) -> AotcuTensor {
    match t {
        Some(t) => tensor(t),
        None => ABSENT,
    }
}

/// The generator's per-architecture switches (`ArchFlags`, crates/aot-codegen/src/model.rs),
/// which `Dims` does not carry; `emit_cuda_forwards` writes them next to `DIMS`.
#[derive(Clone, Copy)]
pub struct CudaFlags {
    pub qkv_bias: bool,
    pub qk_norm: bool,
    pub rope_neox: bool,
    pub post_norms: bool,
    pub gelu: bool,
    pub embd_scale: bool,
}

pub const fn dims(d: &Dims, f: &CudaFlags) -> AotcuDims {
    AotcuDims {
        dim: d.dim as i32,
        hidden: d.hidden as i32,
        n_layer: d.n_layer as i32,
        n_head: d.n_head as i32,
        n_kv_head: d.n_kv_head as i32,
        head_dim: d.head_dim as i32,
        rot_dim: d.rot_dim as i32,
        vocab: d.vocab as i32,
        n_ctx_train: d.n_ctx_train as i32,
        swa_window: d.swa_window as i32,
        eps: d.eps,
        rope_base: d.rope_base,
        rope_scale: d.rope_scale,
        rope_base_local: d.rope_base_local,
        rope_scale_local: d.rope_scale_local,
        qkv_bias: f.qkv_bias as i32,
        qk_norm: f.qk_norm as i32,
        rope_neox: f.rope_neox as i32,
        post_norms: f.post_norms as i32,
        gelu: f.gelu as i32,
        embd_scale: f.embd_scale as i32,
    }
}

// ---- the backend ----------------------------------------------------------------------------

/// Device-resident model and State: the CUDA counterpart of `metal::Gpu` (metal.rs:331-360).
pub struct Gpu {
    ctx: *mut AotcuCtx,
    gpu: *mut AotcuGpu,
    vocab: usize,
}

// One evaluation at a time per context, as the runtime already guarantees (capi.rs:180-181).
unsafe impl Send for Gpu {}

impl Gpu {
    /// `Gpu::new` (metal.rs:366): uploads the tensor section once and allocates the device
    /// State for `state.ctx` positions and prompt batches of `max_batch` tokens. `head` and
    /// `layers` are the `CUDA_HEAD` / `CUDA_LAYERS` statics of the generated `model.rs`.
    pub fn new(weights: &'static [u8], state: &State, max_batch: usize, head: &AotcuModelHead, layers: &[AotcuLayer]) -> Result<Gpu, String> {
        if layers.len() != head.dims.n_layer as usize {
            return Err(format!("{} layer records for {} layers", layers.len(), head.dims.n_layer));
        }
        let device = std::env::var("AOT_CUDA_DEVICE").ok().and_then(|v| v.parse::<c_int>().ok()).unwrap_or(0);
        let mut ctx: *mut AotcuCtx = std::ptr::null_mut();
        // SAFETY: plain C calls; every out-pointer is valid for the duration of its call.
        check(unsafe { aotcu_init(device, &mut ctx) })?;
        let mut gpu: *mut AotcuGpu = std::ptr::null_mut();
        let rc = unsafe { aotcu_gpu_new(ctx, head, layers.as_ptr(), weights.as_ptr(), weights.len(), state.ctx, max_batch.max(1), &mut gpu) };
        if rc != 0 {
            let e = last_error();
            unsafe { aotcu_free(ctx) };
            return Err(format!("aot_cuda: {e} (status {rc})"));
        }
        Ok(Gpu { ctx, gpu, vocab: head.dims.vocab as usize })
    }

    /// One decoding step (what `forward_gpu` of emit.rs:529-641 does op by op): the logits,
    /// when wanted, land in `logits` (`s.logits`) for the sampler.
    pub fn forward(&mut self, token: u32, pos: usize, want_logits: bool, logits: &mut [f32]) {
        // the reference's forward asserts its arguments (emit.rs:467-468); the library
        // reports the same conditions as errors
        check(unsafe { aotcu_forward(self.gpu, token, pos, want_logits as c_int) }).unwrap_or_else(|e| panic!("{e}"));
        if want_logits {
            self.read_logits(logits);
        }
    }

    /// One prompt batch (`forward_batch_gpu`, emit.rs:643-705).
    pub fn forward_batch(&mut self, tokens: &[u32], pos0: usize, want_logits: bool, logits: &mut [f32]) {
        check(unsafe { aotcu_forward_batch(self.gpu, tokens.as_ptr(), tokens.len(), pos0, want_logits as c_int) }).unwrap_or_else(|e| panic!("{e}"));
        if want_logits {
            self.read_logits(logits);
        }
    }

    fn read_logits(&mut self, logits: &mut [f32]) {
        assert!(logits.len() >= self.vocab, "logits buffer shorter than the vocabulary");
        check(unsafe { aotcu_logits(self.gpu, logits.as_mut_ptr()) }).unwrap_or_else(|e| panic!("{e}"));
    }

    /// Greedy decoding kept on the device (the loop of app.rs:553-610 with `argmax`,
    /// sampler.rs:99-109): `out.len()` tokens starting from `token` at `pos`.
    pub fn generate_greedy(&mut self, token: u32, pos: usize, out: &mut [u32]) -> Result<f32, String> {
        let mut ms = 0f32;
        check(unsafe { aotcu_generate(self.gpu, token, pos, out.len(), out.as_mut_ptr(), &mut ms) })?;
        Ok(ms)
    }

    /// `prefix::serialize` on the device cache (prefix.rs:112-141): `--save-kv`, `aot_ctx_save`.
    pub fn kv_save(&mut self, tokens: &[u32], n_cached: usize) -> Result<Vec<u8>, String> {
        let cap = unsafe { aotcu_kv_blob_size(self.gpu, tokens.len(), n_cached) };
        let mut blob = vec![0u8; cap];
        let mut len = 0usize;
        check(unsafe { aotcu_kv_save(self.gpu, tokens.as_ptr(), tokens.len(), n_cached, blob.as_mut_ptr(), cap, &mut len) })?;
        blob.truncate(len);
        Ok(blob)
    }

    /// `Prefix::parse` + `load_into` (prefix.rs:45-103): the tokens of the blob and how many of
    /// them have cache rows, or an error when the blob is not a cache of this model.
    pub fn kv_load(&mut self, blob: &[u8]) -> Result<(Vec<u32>, usize), String> {
        let cap = blob.len().saturating_sub(24) / 4;
        let mut tokens = vec![0u32; cap.max(1)];
        let (mut n, mut cached) = (0usize, 0usize);
        check(unsafe { aotcu_kv_load(self.gpu, blob.as_ptr(), blob.len(), tokens.as_mut_ptr(), tokens.len(), &mut n, &mut cached) })?;
        tokens.truncate(n);
        Ok((tokens, cached))
    }

    /// Kernels launched so far (`Gpu::dispatches`, metal.rs:352-356).
    pub fn dispatches(&mut self) -> u64 {
        unsafe { aotcu_gpu_dispatches(self.gpu) }
    }
}

impl Drop for Gpu {
    fn drop(&mut self) {
        // SAFETY: handles came from aotcu_gpu_new / aotcu_init and are dropped once.
        unsafe {
            aotcu_gpu_free(self.gpu);
            aotcu_free(self.ctx);
        }
    }
}
