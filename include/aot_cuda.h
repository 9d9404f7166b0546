/* aot_cuda.h - C ABI of the B200 (sm_100a) backend for aot-llm's quantized
 * forward-pass hot path.
 *
 * The reference (p10node/aot-llm) is an ahead-of-time compiler whose generated
 * `model.rs` calls the kernel surface of crates/aot-kernels by name. This
 * library provides that surface on the GPU behind plain C entry points so a
 * thin Rust `extern "C"` block (or any FFI) can bind it:
 *
 *   1. kernel level  - `aotcu_matvec_* / aotcu_matmul_* / aotcu_quantize_* /
 *      aotcu_rmsnorm / aotcu_rope / aotcu_attention ...` on DEVICE pointers:
 *      one entry point per function of crates/aot-kernels/src/{matvec,quant,
 *      ops}.rs, same argument meaning;
 *   2. backend level - `aotcu_gpu_*`: the operator API the generated
 *      `forward_gpu` drives (crates/aot-kernels/src/metal.rs `Gpu`, `BufId`,
 *      `MvOpts`), on buffer ids of a device-resident State;
 *   3. step level    - `aotcu_forward / aotcu_forward_batch / aotcu_generate`:
 *      the generated forward()/forward_batch() of crates/aot-codegen/src/emit.rs
 *      466-516, interpreted from a tensor table, replayed as a CUDA graph.
 *
 * Conventions: every function returns 0 on success or a negative aotcu_status;
 * `aotcu_last_error()` returns a thread-local message (same contract as
 * `aot_last_error`, crates/aot-codegen/src/aot_llm.h:61-62). Nothing aborts or
 * traps. One host thread at a time per context. All device pointers must come
 * from the context's device. There is no CPU fallback: without a CUDA device
 * every compute entry point fails with AOTCU_ERR_CUDA.
 *
 * Numerics: integer block sums are exact; f32 results are bit-identical to the
 * reference's x86 AVX2(+F16C) kernel table (crates/aot-kernels/src/simd_avx2.rs)
 * and to its sequential f32 operators (ops.rs) on the same inputs.
 */
#ifndef AOT_CUDA_H
#define AOT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  AOTCU_OK = 0,
  AOTCU_ERR_BAD_ARG = -1,  /* the asserts of matvec.rs:301-302, 480-482; emit.rs:467-468, 493-494 */
  AOTCU_ERR_CUDA = -2,     /* a CUDA runtime call failed (or no device) */
  AOTCU_ERR_TIMEOUT = -3,  /* a bounded device-side wait expired */
  AOTCU_ERR_NCCL = -4,
  AOTCU_ERR_UNSUPPORTED = -5
} aotcu_status;

/* Weight element kinds, order of `enum Kind` (crates/aot-kernels/src/quant.rs:34-44). */
typedef enum {
  AOTCU_F32 = 0, AOTCU_F16 = 1, AOTCU_BF16 = 2, AOTCU_Q4_0 = 3, AOTCU_Q5_0 = 4,
  AOTCU_Q8_0 = 5, AOTCU_Q4_K = 6, AOTCU_Q5_K = 7, AOTCU_Q6_K = 8
} aotcu_kind;

/* Activation blocks exactly as the reference lays them out (quant.rs:194-216). */
typedef struct { float d; int8_t qs[32]; } aotcu_block_q8_0;                     /* 36 bytes */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } aotcu_block_q8_k; /* 292 bytes */

typedef struct aotcu_ctx aotcu_ctx;

const char* aotcu_last_error(void);
/* Library version string; never fails. */
const char* aotcu_version(void);

/* ---- context ------------------------------------------------------------ */
/* Opens CUDA device `device` (replaces Pool::new + Gpu::new's device setup,
 * crates/aot-kernels/src/metal.rs:366). */
int aotcu_init(int device, aotcu_ctx** out);
/* Also frees every aotcu_gpu created on the context that is still alive (their handles
 * become invalid): a Gpu does not outlive its context. */
void aotcu_free(aotcu_ctx* ctx);
int aotcu_sync(aotcu_ctx* ctx);
/* Device memory helpers so a foreign-language host needs no CUDA binding. */
int aotcu_malloc(aotcu_ctx* ctx, size_t bytes, void** dev_ptr);
int aotcu_dev_free(aotcu_ctx* ctx, void* dev_ptr);
int aotcu_h2d(aotcu_ctx* ctx, void* dev_dst, const void* host_src, size_t bytes);
int aotcu_d2h(aotcu_ctx* ctx, void* host_dst, const void* dev_src, size_t bytes);
/* Device-side stopwatch on the context's stream (CUDA events): everything enqueued
 * between start and stop, including the gaps the host leaves, is timed. */
int aotcu_timer_start(aotcu_ctx* ctx);
int aotcu_timer_stop(aotcu_ctx* ctx, float* elapsed_ms);
/* Reads and clears the device error word (bounded waits that expired, ...). */
int aotcu_device_status(aotcu_ctx* ctx);

/* ---- kernel level: quant.rs --------------------------------------------- */
/* quantize_q8_0 (quant.rs:231-245) / quantize_q8_k (quant.rs:248-283) over `n`
 * floats (rows back to back); `out` receives n/32 resp. n/256 blocks. */
int aotcu_quantize_q8_0(aotcu_ctx* ctx, const float* x, size_t n, aotcu_block_q8_0* out);
int aotcu_quantize_q8_k(aotcu_ctx* ctx, const float* x, size_t n, aotcu_block_q8_k* out);
/* dequant_row_<kind> (quant.rs:300-443): `n_rows` rows of `cols` elements,
 * row `row_ids[i]` of the table -> out[i*cols ..]. row_ids on the device. */
int aotcu_dequant_rows(aotcu_ctx* ctx, int kind, const uint8_t* table, const int32_t* row_ids, size_t n_rows,
                       size_t cols, float* out);

/* ---- kernel level: matvec.rs -------------------------------------------- */
/* matvec_<kind> (matvec.rs:358-401): out[r] = dot(W[r], x), r < rows. `x` is
 * aotcu_block_q8_0[cols/32] for Q4_0/Q5_0/Q8_0, aotcu_block_q8_k[cols/256] for
 * Q4_K/Q5_K/Q6_K and float[cols] for F32/F16/BF16. W is the raw GGUF tensor
 * (row r at r*row_bytes); it must be 16-byte aligned for Q4_K/Q5_K, 4 for F32,
 * 2 otherwise, and readable for 64 bytes past its end (aotcu_malloc and
 * aotcu_upload_weights pad). */
int aotcu_matvec(aotcu_ctx* ctx, int kind, float* out, const uint8_t* w, const void* x, size_t rows, size_t cols);
int aotcu_matvec_q4_0(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_0* x, size_t rows, size_t cols);
int aotcu_matvec_q5_0(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_0* x, size_t rows, size_t cols);
int aotcu_matvec_q8_0(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_0* x, size_t rows, size_t cols);
int aotcu_matvec_q4_k(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_k* x, size_t rows, size_t cols);
int aotcu_matvec_q5_k(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_k* x, size_t rows, size_t cols);
int aotcu_matvec_q6_k(aotcu_ctx* ctx, float* out, const uint8_t* w, const aotcu_block_q8_k* x, size_t rows, size_t cols);
int aotcu_matvec_f16(aotcu_ctx* ctx, float* out, const uint8_t* w, const float* x, size_t rows, size_t cols);
int aotcu_matvec_bf16(aotcu_ctx* ctx, float* out, const uint8_t* w, const float* x, size_t rows, size_t cols);
int aotcu_matvec_f32(aotcu_ctx* ctx, float* out, const uint8_t* w, const float* x, size_t rows, size_t cols);
/* matvec2_q8_k_input / matvec2_q8_0_input (matvec.rs:407-439): gate and up rows
 * in one launch; both matrices have `kind` and `rows`. */
int aotcu_matvec2(aotcu_ctx* ctx, int kind, float* out_a, float* out_b, const uint8_t* w_a, const uint8_t* w_b,
                  const void* x, size_t rows, size_t cols);
/* matvec3_q8_k_input / matvec3_q8_0_input (matvec.rs:323-355): q, k, v over the
 * concatenated row space. Kinds may differ as long as they share the activation
 * format (the reference requires equal kinds; this is a superset). */
int aotcu_matvec3(aotcu_ctx* ctx, const int kinds[3], float* const outs[3], const uint8_t* const ws[3], const void* x,
                  const size_t rows[3], size_t cols);
/* matmul_<kind> (matvec.rs:524-546): out[i*rows + r] = dot(W[r], X[i]), i < m.
 * `xs` holds the m activation vectors back to back (token-major). Bitwise equal
 * to m calls of aotcu_matvec. */
int aotcu_matmul(aotcu_ctx* ctx, int kind, float* out, const uint8_t* w, const void* xs, size_t m, size_t rows,
                 size_t cols);
/* matmul2_q8_k_input / matmul2_q8_0_input (matvec.rs:571-583): two matrices of equal shape
 * and kind against the same m activation vectors (ffn_gate and ffn_up of a prompt chunk);
 * out_x[i*rows + r] as aotcu_matmul. */
int aotcu_matmul2(aotcu_ctx* ctx, int kind, float* out_a, float* out_b, const uint8_t* w_a, const uint8_t* w_b,
                  const void* xs, size_t m, size_t rows, size_t cols);
/* No counterpart in the reference (its CPU kernels borrow `State.aqk`, which the caller
 * owns). out[r] = dot(W[r], quantize_q8_k(x)) for a K-quant matrix (kind Q4_K, Q5_K or
 * Q6_K) and an f32 device vector x, bit-identical to aotcu_quantize_q8_k followed by
 * aotcu_matvec, for callers that must not allocate: a serving process that sized its
 * device memory once at start-up (weights, KV cache) and forbids or cannot afford later
 * cudaMalloc calls - they may fail when HBM is fully committed, and they stall every
 * stream of the device while they run. The quantized copy of x lives in a 19,456-byte
 * array built into the library's device image (held by every GPU that loads the
 * library, until exit), so this call uses no allocator at all.
 *   - cols must be a multiple of 256 and at most 16384; larger vectors are rejected with
 *     AOTCU_ERR_BAD_ARG (use the two-call route with your own buffer).
 *   - The first call on each device looks the array's address up
 *     (cudaGetSymbolAddress); make that first call before any stream capture begins.
 *   - All calls on a device share the one array: two calls whose kernels can overlap
 *     on the GPU (different contexts or streams) race on it. Calls through one context
 *     are ordered by its stream and are safe. Nothing in the array needs clearing
 *     between calls: each call rewrites every block it reads.
 *     The first call on a device looks up the array's address and caches it without a
 *     lock: make that first call from one host thread (two threads racing there would
 *     store the same value, but nothing promises that to stay harmless). */
int aotcu_matvec_k_static(aotcu_ctx* ctx, int kind, float* out, const uint8_t* w, const float* x, size_t rows,
                          size_t cols);
/* Parity export: the integers of one matvec before any float arithmetic.
 * sumi[r*nb + b] (and summ for Q4_K/Q5_K, else untouched) per (row, block), as
 * matvec.rs:89-103 / 146-163 / 38-43 form them. Device pointers. */
int aotcu_block_sums(aotcu_ctx* ctx, int kind, const uint8_t* w, const void* x, size_t rows, size_t cols,
                     int32_t* sumi, int32_t* summ);
/* The same integers as the production kernels form them, written by the kernels themselves
 * while they compute the product: kernel 0 = the streaming single-row product
 * (aotcu_matvec_* of a K-quant; m = 1; sumi[r*nb + b]), kernel 1 = the tcgen05 prompt product
 * (Q4_K / Q5_K, m <= 64; sumi[(t*rows + r)*nb + b]). x: reference-layout BlockQ8_K rows.
 * For Q6_K summ is left untouched. Device pointers. */
int aotcu_block_sums_of(aotcu_ctx* ctx, int kernel, int kind, const uint8_t* w, const void* x, size_t m, size_t rows,
                        size_t cols, int32_t* sumi, int32_t* summ);

/* ---- kernel level: ops.rs / sampler.rs ---------------------------------- */
/* rmsnorm_rows (ops.rs:7-18, 358-363): m rows of n. out may alias x. */
int aotcu_rmsnorm(aotcu_ctx* ctx, float* out, const float* x, const float* w, size_t n, size_t m, float eps);
/* rmsnorm_heads (ops.rs:74-87), in place, n_heads heads of head_dim. */
int aotcu_rmsnorm_heads(aotcu_ctx* ctx, float* x, const float* w, size_t n_heads, size_t head_dim, float eps);
/* rope_rows / rope_neox_rows (ops.rs:40-70, 375-388): m rows of n_heads*head_dim,
 * row i rotated with cs[i*rot_dim ..] (interleaved cos, sin). */
int aotcu_rope(aotcu_ctx* ctx, float* x, size_t m, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs,
               int neox);
int aotcu_silu_mul(aotcu_ctx* ctx, float* h, const float* up, size_t n);   /* ops.rs:115-120 */
/* h = gelu(h) * up, tanh approximation (ops.rs:122-134). tanh is the correctly rounded f32
 * value; the reference takes it from the platform's libm, which may differ by one ulp. */
int aotcu_gelu_mul(aotcu_ctx* ctx, float* h, const float* up, size_t n);
int aotcu_add_inplace(aotcu_ctx* ctx, float* x, const float* y, size_t n); /* ops.rs:144-148 */
int aotcu_add_bias_rows(aotcu_ctx* ctx, float* x, const float* b, size_t n, size_t m); /* ops.rs:90-95 */
int aotcu_scale_inplace(aotcu_ctx* ctx, float* x, float s, size_t n);      /* ops.rs:137-141 */
/* attention_rows (ops.rs:517-556; attention of 185-218 is m == 1): caches are
 * the layer's ctx x kv_dim slices. window == 0 attends to everything. */
int aotcu_attention(aotcu_ctx* ctx, float* out, const float* q, const float* k_cache, const float* v_cache,
                    size_t n_head, size_t n_kv_head, size_t head_dim, size_t ctx_len, size_t pos0, size_t m,
                    size_t window);
/* argmax (sampler.rs:99-109): first maximum; result written to *out_token (device). */
int aotcu_argmax(aotcu_ctx* ctx, const float* x, size_t n, int32_t* out_token);

/* ---- model description (what the generator emits as DIMS / LAYERS) ------- */
/* crates/aot-kernels/src/state.rs:165-180 */
typedef struct {
  int32_t kind;
  int32_t present;
  uint64_t off, len, rows, cols;
} aotcu_tensor;

/* crates/aot-kernels/src/state.rs:126-161 plus the ModelFlags of
 * crates/aot-codegen/src/model.rs. */
typedef struct {
  int32_t dim, hidden, n_layer, n_head, n_kv_head, head_dim, rot_dim, vocab, n_ctx_train;
  int32_t swa_window;
  float eps, rope_base, rope_scale, rope_base_local, rope_scale_local;
  int32_t qkv_bias, qk_norm, rope_neox, post_norms, gelu, embd_scale;
} aotcu_dims;

typedef struct {
  aotcu_tensor attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down;
  aotcu_tensor bq, bk, bv, q_norm, k_norm, attn_post_norm, ffn_post_norm;
  int32_t local_attn;
  int32_t pad_;
} aotcu_layer;

typedef struct {
  aotcu_dims dims;
  aotcu_tensor token_embd, output_norm, output, rope_freqs;
} aotcu_model_head;

/* ---- backend level: the `Gpu` of crates/aot-kernels/src/metal.rs --------- */
/* Buffer ids, order of `enum BufId` (metal.rs:205-229). */
typedef enum {
  AOTCU_BUF_X = 0, AOTCU_BUF_XB, AOTCU_BUF_XB2, AOTCU_BUF_Q, AOTCU_BUF_K, AOTCU_BUF_V, AOTCU_BUF_HB,
  AOTCU_BUF_HB2, AOTCU_BUF_LOGITS, AOTCU_BUF_KCACHE, AOTCU_BUF_VCACHE, AOTCU_BUF_ROPECS, AOTCU_BUF_BX,
  AOTCU_BUF_BXB, AOTCU_BUF_BXB2, AOTCU_BUF_BQ, AOTCU_BUF_BK, AOTCU_BUF_BV, AOTCU_BUF_BHB, AOTCU_BUF_BHB2,
  AOTCU_BUF_BROPECS, AOTCU_BUF_ROPECS_LOCAL, AOTCU_BUF_BROPECS_LOCAL, AOTCU_N_BUFS
} aotcu_buf;

typedef struct aotcu_gpu aotcu_gpu;

/* Gpu::new (metal.rs:366): uploads the GGUF tensor section to HBM once (no copy
 * is kept on the host side), allocates the device State (state.rs:304-355) for
 * a context of `n_ctx` tokens and prompt batches of up to `max_batch`, and
 * precomputes the RoPE (cos, sin) rows of every position with the host libm
 * exactly as ops.rs:28-34 / state.rs:308-319 do per step. */
int aotcu_gpu_new(aotcu_ctx* ctx, const aotcu_model_head* head, const aotcu_layer* layers, const uint8_t* weights,
                  size_t weights_len, size_t n_ctx, size_t max_batch, aotcu_gpu** out);
void aotcu_gpu_free(aotcu_gpu* g);
/* Device address and element count of a State buffer. */
int aotcu_gpu_buf(aotcu_gpu* g, int buf, float** dev_ptr, size_t* n_floats);
/* Copy floats between a State buffer and host memory (offset in elements). */
int aotcu_gpu_read(aotcu_gpu* g, int buf, size_t offset, float* host_dst, size_t n);
int aotcu_gpu_write(aotcu_gpu* g, int buf, size_t offset, const float* host_src, size_t n);
/* Gpu::begin / Gpu::finish (metal.rs:494-521): finish waits for the stream and
 * reports device-side errors. */
int aotcu_gpu_begin(aotcu_gpu* g);
int aotcu_gpu_finish(aotcu_gpu* g);
/* Gpu::rmsnorm (metal.rs:563-574): dst = rmsnorm(src) * w over m rows of n;
 * accumulate adds into dst (Gpu::rmsnorm_add). The normalised rows are also
 * quantized for the products that follow. */
int aotcu_gpu_rmsnorm(aotcu_gpu* g, int dst, size_t dst_off, int src, size_t src_off, const aotcu_tensor* w, size_t n,
                      size_t m, float eps, int accumulate);
/* Gpu::mv / Gpu::matmul (metal.rs:622-657, 712-724): dst (+)= W . src for m rows. */
int aotcu_gpu_matmul(aotcu_gpu* g, int dst, size_t dst_off, const aotcu_tensor* w, int src, size_t src_off, size_t m,
                     int accumulate);
/* Gpu::mv3 (metal.rs:666-709): q, k, v products of one input in one launch. */
int aotcu_gpu_mv3(aotcu_gpu* g, const int dst[3], const size_t dst_off[3], const aotcu_tensor* const w[3], int src,
                  size_t m);
/* Gpu::gate_up (metal.rs:735-747): dst = act(G . src) * (U . src); Hb2 keeps U . src. */
int aotcu_gpu_gate_up(aotcu_gpu* g, int dst, const aotcu_tensor* gate, const aotcu_tensor* up, int src, size_t m);
/* Per-head q/k norm + RoPE + KV store of layer `layer` for m tokens at pos0
 * (Gpu::rmsnorm_at + Gpu::rope_ex, metal.rs:758-769, plus store_kv). */
int aotcu_gpu_qk_post(aotcu_gpu* g, size_t layer, size_t pos0, size_t m);
/* Gpu::attention (metal.rs:774-797). */
int aotcu_gpu_attention(aotcu_gpu* g, int dst, int q, size_t layer, size_t pos0, size_t m, size_t window);

/* ---- step level ----------------------------------------------------------- */
/* forward (emit.rs:466-486). With want_logits the vocabulary logits are left in
 * the Logits buffer, and a copy comes back into pinned host memory with the step's
 * one wait, from which the next aotcu_logits is served. Returns when the step is done. */
int aotcu_forward(aotcu_gpu* g, uint32_t token, size_t pos, int want_logits);
/* forward_batch (emit.rs:491-516): `n` tokens (1..max_batch) at pos0... */
int aotcu_forward_batch(aotcu_gpu* g, const uint32_t* tokens, size_t n, size_t pos0, int want_logits);
/* Copies the logits of the last step to host memory (vocab floats). */
int aotcu_logits(aotcu_gpu* g, float* host_dst);
/* Greedy decoding entirely on the device: starting from `token` at `pos`, runs
 * `n_steps` forward passes, each followed by argmax (sampler.rs:99-109) whose
 * result feeds the next step; writes the n_steps generated ids to `out_tokens`
 * (host). `elapsed_ms`, if not NULL, receives the device time of the loop. */
int aotcu_generate(aotcu_gpu* g, uint32_t token, size_t pos, size_t n_steps, uint32_t* out_tokens, float* elapsed_ms);
/* ---- saved KV cache ("AOTP" blob, crates/aot-kernels/src/prefix.rs:14-26) -------------
 * Little-endian: "AOTP", version 2, n_tokens, n_layer, kv_dim, n_cached (six u32), the
 * token ids, zero padding to a 64-byte boundary, then per layer the K rows
 * f32[n_cached * kv_dim] followed by the V rows. The first n_cached tokens have cache rows;
 * the rest must be evaluated by the caller (prefix.rs:24-26).
 *
 * aotcu_kv_blob_size: bytes aotcu_kv_save writes for these counts (prefix.rs:112-141).
 * aotcu_kv_save: serialises `tokens` and the cache rows of positions [0, n_cached) of this
 *   Gpu into `out` (host memory, `out_cap` bytes); n_cached is clamped to n_tokens as the
 *   reference does (prefix.rs:114) and must not exceed the context. Replaces
 *   prefix::serialize (callers: app.rs:489, 631-640, capi.rs:518-523).
 * aotcu_kv_load: parses a version 1 or 2 blob, checks it against this model (n_layer,
 *   kv_dim, n_tokens > 0, n_cached <= n_tokens, length: prefix.rs:45-69) and that the cached
 *   rows fit the context, copies the rows into the device cache (positions [0, n_cached))
 *   and returns the token ids (up to tokens_cap of them), their count and n_cached. A blob
 *   that is not a cache of this model fails with AOTCU_ERR_BAD_ARG and changes nothing
 *   (Prefix::parse returning None). Replaces Prefix::parse + load_into (callers:
 *   app.rs:458-471, capi.rs:526-545). */
size_t aotcu_kv_blob_size(const aotcu_gpu* g, size_t n_tokens, size_t n_cached);
int aotcu_kv_save(aotcu_gpu* g, const uint32_t* tokens, size_t n_tokens, size_t n_cached, uint8_t* out, size_t out_cap,
                  size_t* out_len);
int aotcu_kv_load(aotcu_gpu* g, const uint8_t* blob, size_t blob_len, uint32_t* tokens_out, size_t tokens_cap,
                  size_t* n_tokens, size_t* n_cached);
/* Number of kernels launched by this Gpu since creation (Gpu.dispatches, metal.rs:352-356). */
uint64_t aotcu_gpu_dispatches(aotcu_gpu* g);
/* Tuning switches (the role of AOT_GPU_MV_ROWS, metal.rs:368): name = "graph"
 * (replay decode steps as a CUDA graph, default 1), "pdl" (programmatic dependent
 * launch between kernels, default 1), "mega" (run decode steps as the one-kernel step
 * when the model allows it, default 1). Query: "mega_available" returns 1 when the model
 * can use the one-kernel step, else 0 (the value argument is ignored). */
int aotcu_gpu_set_option(aotcu_gpu* g, const char* name, int value);

/* Tensor parallel decode (no counterpart in the reference, which runs on one device): each
 * rank creates an aotcu_gpu from its shard of the model (query/KV heads and FFN rows split
 * across ranks; attn_output and ffn_down split by columns on 256-weight boundaries) and
 * joins a group. Inside the forward pass the ranks' partial attn_output and ffn_down rows
 * are summed with an NCCL all-reduce on the context's stream before they join the residual
 * stream. `nccl_library` names the NCCL shared object to load (NULL: "libnccl.so.2" from
 * the loader path). One rank calls aotcu_tp_unique_id and hands the 128 bytes to all
 * ranks by its own means; every rank then calls aotcu_tp_attach (collective). Sums across
 * ranks change the order of f32 additions: results match the single-device path to
 * rounding (1e-3 relative at the logits), not bit for bit.
 *
 * Decode steps of models the one-kernel step covers can keep the exchange inside that kernel:
 * every rank first calls aotcu_tp_inbox_handle (allocates its inbox for the other ranks'
 * partial rows and returns its 64-byte CUDA IPC handle), the host gathers the handles of all
 * ranks in rank order (world x 64 bytes) and passes them to aotcu_tp_attach as
 * `peer_handles`. Each GPU then writes its partial rows straight into the peers' inboxes over
 * NVLink and adds the world's partials in rank order. With peer_handles == NULL every
 * exchange goes through NCCL. At most 8 ranks, one process per GPU, all on one box. */
int aotcu_tp_unique_id(const char* nccl_library, uint8_t out_id[128]);
int aotcu_tp_inbox_handle(aotcu_gpu* g, uint8_t out_handle[64]);
int aotcu_tp_attach(aotcu_gpu* g, const char* nccl_library, int rank, int world, const uint8_t id[128],
                    const uint8_t* peer_handles);

/* Benchmark helper (no counterpart in the reference; its per-op figures come from
 * `bench_ops`, crates/aot-kernels/tests/metal.rs:456-641): times only the matrix
 * products of one decode step, back to back, and reports milliseconds per sweep,
 * kernel launches per sweep and the algorithmic bytes (weights + x + y) they move. */
int aotcu_bench_gemv_sweep(aotcu_gpu* g, int iters, float* ms_per_sweep, uint64_t* launches_per_sweep,
                           uint64_t* bytes_per_sweep);

/* Benchmark helper (the role of the per-kind `bench_ops` table of the reference,
 * crates/aot-kernels/tests/metal.rs:456-641): launches the product of `m` activation rows
 * (m = 1: aotcu_matvec, m > 1: aotcu_matmul) `iters` times back to back inside one pair of
 * CUDA events and returns the average milliseconds per launch. `w` holds `n_copies` copies
 * of the matrix, `copy_stride` bytes apart; launch i uses copy i % n_copies, so that with
 * n_copies * matrix bytes above the L2 size every launch streams its weights from HBM. */
int aotcu_bench_matmul(aotcu_ctx* ctx, int kind, float* out, const uint8_t* w, size_t copy_stride, size_t n_copies,
                       const void* xs, size_t m, size_t rows, size_t cols, int iters, float* ms_per_launch);

/* Tuning aid for the one-kernel decode step (no counterpart in the reference): runs
 * one step and returns the SM cycles CTA `cta` spent in each of its 16 phases
 * (slots 16..31: sub-phases of the first norm and of attention). */
int aotcu_gpu_profile_step(aotcu_gpu* g, uint32_t token, size_t pos, int cta, uint64_t out[32]);
/* The same step with a global timestamp per CTA at each phase boundary of one layer:
   out[cta * 16 + k] = nanoseconds (device global timer) at which CTA `cta` left phase k
   of layer `layer` (k as in aotcu_gpu_profile_step; unused slots stay 0). `n_cta`
   receives the grid size; out must hold 16 * 256 values. Shows which CTAs the others
   wait for. */
int aotcu_gpu_timeline_step(aotcu_gpu* g, uint32_t token, size_t pos, int layer, uint64_t* out, int* n_cta);

size_t aotcu_row_bytes(int kind, size_t cols);

#ifdef __cplusplus
}
#endif
#endif /* AOT_CUDA_H */
