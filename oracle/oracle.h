// CPU oracle for the quantized forward-pass hot path of aot-llm.
//
// TEST INFRASTRUCTURE ONLY. This library is a behavioural restatement (new
// code, same arithmetic and the same operation order) of the reference's CPU
// kernels in crates/aot-kernels/src/{quant,matvec,simd_avx2,ops,sampler}.rs and
// of the forward pass that crates/aot-codegen/src/emit.rs generates. It exists
// to check the CUDA library and to serve as the timed CPU baseline; nothing in
// the product path may call it.
//
// Parity pin: the reference is Rust and cannot be compiled where this was
// written, so the restatement is pinned against the known answers and the
// invariants held by the reference's own unit and integration tests (f16
// conversions, rmsnorm/rope/attention small cases, x4 == singles bitwise,
// matmul == matvec bitwise, SIMD-vs-scalar tolerances) and against an
// independent float forward pass written in numpy.
//
// Everything must be compiled with -ffp-contract=off: Rust never contracts
// a*b+c, and the only fused operations of the x86 path are its explicit
// _mm256_fmadd_ps calls.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Kind order follows `enum Kind` in crates/aot-kernels/src/quant.rs:34-44.
enum orc_kind {
  ORC_F32 = 0,
  ORC_F16 = 1,
  ORC_BF16 = 2,
  ORC_Q4_0 = 3,
  ORC_Q5_0 = 4,
  ORC_Q8_0 = 5,
  ORC_Q4_K = 6,
  ORC_Q5_K = 7,
  ORC_Q6_K = 8,
};

// Kernel tables of crates/aot-kernels/src/matvec.rs:221-237 and
// simd_avx2.rs:536-571.
enum orc_table { ORC_SCALAR = 0, ORC_AVX2 = 1, ORC_AVX2_F16C = 2 };

// Activation blocks, crates/aot-kernels/src/quant.rs:194-216 (repr(C)).
typedef struct {
  float d;
  int8_t qs[32];
} orc_block_q8_0;  // 36 bytes

typedef struct {
  float d;
  int8_t qs[256];
  int16_t bsums[16];
} orc_block_q8_k;  // 292 bytes

// crates/aot-kernels/src/state.rs:165-180 (Tensor) without the name.
typedef struct {
  int32_t kind;
  int32_t present;  // 0 for an optional tensor that the model does not have
  uint64_t off, len, rows, cols;
} orc_tensor;

// crates/aot-kernels/src/state.rs:126-161 (Dims) plus the architecture flags of
// crates/aot-codegen/src/model.rs (qkv bias, per-head q/k norm, NEOX RoPE,
// Gemma post-norms, GeGLU, embedding scale).
typedef struct {
  int32_t dim, hidden, n_layer, n_head, n_kv_head, head_dim, rot_dim, vocab, n_ctx_train;
  int32_t swa_window;
  float eps, rope_base, rope_scale, rope_base_local, rope_scale_local;
  int32_t qkv_bias, qk_norm, rope_neox, post_norms, gelu, embd_scale;
} orc_dims;

typedef struct {
  orc_tensor attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down;
  orc_tensor bq, bk, bv, q_norm, k_norm, attn_post_norm, ffn_post_norm;
  int32_t local_attn;
  int32_t pad_;
} orc_layer;

typedef struct {
  orc_dims dims;
  orc_tensor token_embd, output_norm, output, rope_freqs;
} orc_model_head;

// ---- quant.rs -------------------------------------------------------------
size_t orc_block_size(int kind);
size_t orc_type_size(int kind);
size_t orc_row_bytes(int kind, size_t n);
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float f);
void orc_quantize_q8_0(const float* x, size_t n, orc_block_q8_0* out);
void orc_quantize_q8_k(const float* x, size_t n, orc_block_q8_k* out);
void orc_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m);
void orc_dequant_row(int kind, const uint8_t* row, float* out, size_t n);

// ---- matvec.rs / simd_avx2.rs ----------------------------------------------
// 1 when this CPU can run `table`.
int orc_table_supported(int table);
// The table `detect_kernels` (matvec.rs:240-257) picks on this CPU.
int orc_detect_table(void);
// One dot product; `x` is orc_block_q8_0[], orc_block_q8_k[] or float[]
// according to the kind's activation format.
float orc_dot(int table, int kind, const uint8_t* w, const void* x, size_t cols);
// 1x4 micro-kernel; returns 0 (and leaves `out` alone) when the table has none
// for this kind.
int orc_dot_x4(int table, int kind, const uint8_t* w, const void* x0, const void* x1, const void* x2,
               const void* x3, size_t cols, float out[4]);
// Integer part of one K-quant / 32-block dot: per block b, sumi[b] and (for
// Q4_K/Q5_K) summ[b] as the reference forms them. For Q6_K sumi is the signed
// sum (equal to the unsigned sum minus 32*bias of the AVX2 form). For
// Q4_0/Q5_0/Q8_0 sumi[b] is the 32-element integer dot.
void orc_block_sums(int kind, const uint8_t* w, const void* x, size_t cols, int32_t* sumi, int32_t* summ);

typedef struct orc_pool orc_pool;
orc_pool* orc_pool_new(int n_threads);
void orc_pool_free(orc_pool* p);
int orc_pool_threads(const orc_pool* p);

void orc_matvec(orc_pool* p, int table, int kind, float* out, const uint8_t* w, const void* x, size_t rows,
                size_t cols);
void orc_matvec2(orc_pool* p, int table, int kind, float* out_a, float* out_b, const uint8_t* w_a,
                 const uint8_t* w_b, const void* x, size_t rows, size_t cols);
void orc_matvec3(orc_pool* p, int table, int kind, float* o0, float* o1, float* o2, const uint8_t* w0,
                 const uint8_t* w1, const uint8_t* w2, const void* x, size_t r0, size_t r1, size_t r2,
                 size_t cols);
void orc_matmul(orc_pool* p, int table, int kind, float* out, const uint8_t* w, const void* xs, size_t m,
                size_t rows, size_t cols);

// ---- ops.rs / sampler.rs ----------------------------------------------------
void orc_rmsnorm(float* out, const float* x, const float* w, size_t n, float eps);
void orc_rope_cos_sin(float* cs, const float* inv_freq, size_t half, float pos);
void orc_rope(float* x, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs);
void orc_rope_neox(float* x, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs);
void orc_rmsnorm_heads(float* x, const float* w, size_t n_heads, size_t head_dim, float eps);
void orc_softmax(float* x, size_t n);
void orc_silu_mul(float* h, const float* up, size_t n);
float orc_gelu(float v);
void orc_set_tanh_mode(int correctly_rounded);
void orc_gelu_mul(float* h, const float* up, size_t n);
void orc_add_inplace(float* x, const float* y, size_t n);
void orc_inv_freq(float* out, size_t rot_dim, float base, const float* freq_factors);
void orc_attention(orc_pool* p, float* out, const float* q, const float* k_cache, const float* v_cache,
                   float* scores, const orc_dims* d, size_t ctx, size_t layer, size_t pos, size_t window);
void orc_attention_rows(orc_pool* p, float* out, const float* q, const float* k_cache, const float* v_cache,
                        float* scratch, const orc_dims* d, size_t ctx, size_t layer, size_t pos0, size_t m,
                        size_t window);
uint32_t orc_argmax(const float* x, size_t n);

// ---- generated forward pass (emit.rs) ---------------------------------------
typedef struct orc_model orc_model;
// `weights` must stay valid for the life of the model (it is not copied).
orc_model* orc_model_new(const orc_model_head* head, const orc_layer* layers, const uint8_t* weights,
                         size_t weights_len, size_t ctx, size_t max_batch, int n_threads, int table);
void orc_model_free(orc_model* m);
// forward / forward_batch of emit.rs:466-516. Return 0, or -1 on the bounds
// violations the generated code asserts.
int orc_forward(orc_model* m, uint32_t token, size_t pos, int want_logits);
int orc_forward_batch(orc_model* m, const uint32_t* tokens, size_t n, size_t pos0, int want_logits);
// Named State buffers ("x","xb","xb2","q","k","v","hb","hb2","logits",
// "k_cache","v_cache","bx",...) for intermediate comparisons; NULL if unknown.
float* orc_state_buf(orc_model* m, const char* name, size_t* len);
// Quantized activations after the last quantize call (aqk / aq0).
const void* orc_state_aqk(orc_model* m, size_t* n_blocks);
const void* orc_state_aq0(orc_model* m, size_t* n_blocks);

#ifdef __cplusplus
}
#endif
