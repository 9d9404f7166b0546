//! Generator side of the CUDA backend: a function for `crates/aot-codegen/src/emit.rs`,
//! called from `emit_model_rs` where `emit_gpu_forwards` is called for Metal
//! (emit.rs:529-705) when the project is compiled with `--gpu cuda`. It writes into
//! `model.rs`
//!   * `CUDA_HEAD` / `CUDA_LAYERS`: the tensor table as the library's C structs, built from
//!     the constants `emit_model_rs` has already written (`DIMS`, `TOKEN_EMBD`, `OUTPUT_NORM`,
//!     `OUTPUT`, `ROPE_FREQS`, `LAYERS`; emit.rs:399-454);
//!   * `forward_gpu` / `forward_batch_gpu` with the signatures `app.rs:275-289` calls.
//! Where the Metal variant emits one `g.<operator>(...)` line per operation, the CUDA one
//! emits a single step call: the library interprets the same tensor table on the device.
//! Not compiled where it was written (no Rust toolchain there).
//!
//! Other places a maintainer touches (no code copied here, only the spots):
//!   * `GpuBackend` (emit.rs:81-92): add `Cuda`; the CLI's `--gpu` parser
//!     (crates/aot-llm/src/main.rs:163-176): accept `cuda`;
//!   * `rt_sources.rs:6-26`: add `cuda.rs` to the files copied into `src/rt/`, and copy
//!     `csrc/`, `include/` and `build.rs` into the project when the backend is CUDA;
//!   * `app.rs:263-271` (`gpu_new`): `#[cfg(feature = "cuda")]` variant calling
//!     `cuda::Gpu::new(weights, state, BATCH, &model::CUDA_HEAD, &model::CUDA_LAYERS)`;
//!   * `app.rs:458-471, 629-640` and `capi.rs:518-545`: when the CUDA `Gpu` is active, route
//!     `--save-kv` / `--load-kv` / `aot_ctx_save` / `aot_ctx_load` through `Gpu::kv_save` /
//!     `Gpu::kv_load` (the cache lives on the device).
use std::fmt::Write;

use crate::model::{LayerSpec, ModelSpec};

fn opt_field(l: &LayerSpec, present: bool, field: &str, index: usize) -> String {
    let _ = l;
    if present {
        format!("tensor(&LAYERS[{index}].{field})")
    } else {
        "ABSENT".to_string()
    }
}

/// Appends the CUDA statics and the two GPU entry points to the text of `model.rs`.
pub fn emit_cuda_forwards(o: &mut String, spec: &ModelSpec) {
    let f = &spec.flags;
    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(o, "use crate::rt::cuda::{{dims, tensor, tensor_opt, AotcuLayer, AotcuModelHead, CudaFlags, Gpu, ABSENT}};\n").unwrap();
    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(
        o,
        "pub const CUDA_FLAGS: CudaFlags = CudaFlags {{ qkv_bias: {}, qk_norm: {}, rope_neox: {}, post_norms: {}, gelu: {}, embd_scale: {} }};",
        f.qkv_bias, f.qk_norm, f.rope_neox, f.post_norms, f.gelu, f.embd_scale
    )
    .unwrap();
    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(o, "pub static CUDA_HEAD: AotcuModelHead = AotcuModelHead {{").unwrap();
    writeln!(o, "    dims: dims(&DIMS, &CUDA_FLAGS),").unwrap();
    writeln!(o, "    token_embd: tensor(&TOKEN_EMBD),").unwrap();
    writeln!(o, "    output_norm: tensor(&OUTPUT_NORM),").unwrap();
    // a tied head is described as absent: the library then reads the embedding matrix
    match &spec.output {
        Some(_) => writeln!(o, "    output: tensor(&OUTPUT),").unwrap(),
        None => writeln!(o, "    output: ABSENT,").unwrap(),
    }
    writeln!(o, "    rope_freqs: tensor_opt(ROPE_FREQS.as_ref()),").unwrap();
    writeln!(o, "}};\n").unwrap();

    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(o, "pub static CUDA_LAYERS: [AotcuLayer; {}] = [", spec.layers.len()).unwrap();
    for (i, l) in spec.layers.iter().enumerate() {
        writeln!(o, "    AotcuLayer {{").unwrap();
        for field in ["attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "gate", "up", "down"] {
            writeln!(o, "        {field}: tensor(&LAYERS[{i}].{field}),").unwrap();
        }
        for field in ["bq", "bk", "bv"] {
            writeln!(o, "        {field}: {},", opt_field(l, f.qkv_bias, field, i)).unwrap();
        }
        for field in ["q_norm", "k_norm"] {
            writeln!(o, "        {field}: {},", opt_field(l, f.qk_norm, field, i)).unwrap();
        }
        for field in ["attn_post_norm", "ffn_post_norm"] {
            writeln!(o, "        {field}: {},", opt_field(l, f.post_norms, field, i)).unwrap();
        }
        writeln!(o, "        local_attn: {},", l.local_attn as i32).unwrap();
        writeln!(o, "        pad_: 0,").unwrap();
        writeln!(o, "    }},").unwrap();
    }
    writeln!(o, "];\n").unwrap();

    writeln!(o, "/// One decoding step on the CUDA device; logits (when wanted) end up in `s.logits`.").unwrap();
    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(o, "pub fn forward_gpu(s: &mut State, _w: &Weights, g: &mut Gpu, token: u32, pos: usize, want_logits: bool) {{").unwrap();
    writeln!(o, "    g.forward(token, pos, want_logits, &mut s.logits);").unwrap();
    writeln!(o, "}}\n").unwrap();
    writeln!(o, "/// One prompt batch on the CUDA device.").unwrap();
    writeln!(o, "#[cfg(feature = \"cuda\")]").unwrap();
    writeln!(o, "pub fn forward_batch_gpu(s: &mut State, _w: &Weights, g: &mut Gpu, tokens: &[u32], pos0: usize, want_logits: bool) {{").unwrap();
    writeln!(o, "    g.forward_batch(tokens, pos0, want_logits, &mut s.logits);").unwrap();
    writeln!(o, "}}").unwrap();
}
