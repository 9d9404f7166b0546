// Oracle (test infrastructure): the non-matmul operators of a transformer
// block. Restates crates/aot-kernels/src/ops.rs, the RoPE frequency table of
// crates/aot-kernels/src/state.rs:308-319 and argmax of
// crates/aot-kernels/src/sampler.rs:99-109. All reductions are the
// reference's sequential f32 loops; exp/sin/cos/pow/tanh/sqrt are the
// platform libm, which is what the reference's std calls resolve to.
#include <math.h>

#include "oracle_internal.h"

// ops.rs:160-166
static inline float dotf(const float* a, const float* b, size_t n) {
  float s = 0.0f;
  for (size_t i = 0; i < n; i++) s += a[i] * b[i];
  return s;
}

// ops.rs:171-177
static inline size_t window_start(size_t pos, size_t window) {
  return (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
}

extern "C" {

// ops.rs:7-18
void orc_rmsnorm(float* out, const float* x, const float* w, size_t n, float eps) {
  float ss = 0.0f;
  for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
  float r = 1.0f / sqrtf(ss / (float)n + eps);
  for (size_t i = 0; i < n; i++) out[i] = x[i] * r * w[i];
}

// ops.rs:28-34
__attribute__((noinline)) void orc_rope_cos_sin(float* cs, const float* inv_freq, size_t half, float pos) {
  for (size_t i = 0; i < half; i++) {
    float a = pos * inv_freq[i];
    cs[2 * i] = cosf(a);
    cs[2 * i + 1] = sinf(a);
  }
}

// ops.rs:40-52
void orc_rope(float* x, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs) {
  for (size_t h = 0; h < n_heads; h++) {
    float* v = x + h * head_dim;
    for (size_t i = 0; i < rot_dim / 2; i++) {
      float c = cs[2 * i], s = cs[2 * i + 1];
      float x0 = v[2 * i], x1 = v[2 * i + 1];
      v[2 * i] = x0 * c - x1 * s;
      v[2 * i + 1] = x0 * s + x1 * c;
    }
  }
}

// ops.rs:57-70
void orc_rope_neox(float* x, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs) {
  size_t half = rot_dim / 2;
  for (size_t h = 0; h < n_heads; h++) {
    float* v = x + h * head_dim;
    for (size_t i = 0; i < half; i++) {
      float c = cs[2 * i], s = cs[2 * i + 1];
      float x0 = v[i], x1 = v[i + half];
      v[i] = x0 * c - x1 * s;
      v[i + half] = x0 * s + x1 * c;
    }
  }
}

// ops.rs:74-87
void orc_rmsnorm_heads(float* x, const float* w, size_t n_heads, size_t head_dim, float eps) {
  for (size_t h = 0; h < n_heads; h++) {
    float* v = x + h * head_dim;
    float ss = 0.0f;
    for (size_t i = 0; i < head_dim; i++) ss += v[i] * v[i];
    float r = 1.0f / sqrtf(ss / (float)head_dim + eps);
    for (size_t i = 0; i < head_dim; i++) v[i] = v[i] * r * w[i];
  }
}

// ops.rs:98-112
void orc_softmax(float* x, size_t n) {
  float mx = -INFINITY;
  for (size_t i = 0; i < n; i++) mx = fmaxf(mx, x[i]);
  float sum = 0.0f;
  for (size_t i = 0; i < n; i++) {
    x[i] = expf(x[i] - mx);
    sum += x[i];
  }
  float inv = 1.0f / sum;
  for (size_t i = 0; i < n; i++) x[i] *= inv;
}

// ops.rs:115-120
void orc_silu_mul(float* h, const float* up, size_t n) {
  for (size_t i = 0; i < n; i++) {
    float v = h[i];
    h[i] = v / (1.0f + expf(-v)) * up[i];
  }
}

// ops.rs:124-127; the constant is FRAC_2_SQRT_PI / SQRT_2 evaluated in f32. Rust's f32::tanh
// is the platform libm's tanhf, so the reference's own result depends on that library
// (glibc before 2.41 is not correctly rounded). Mode 0 calls this host's tanhf as the
// reference would here; mode 1 rounds the double-precision tanh once, which is the value
// a correctly rounded libm returns and the one the CUDA library computes.
static int g_tanh_mode = 0;
void orc_set_tanh_mode(int correctly_rounded) { g_tanh_mode = correctly_rounded; }
float orc_gelu(float v) {
  const float k = 1.1283791670955126f / 1.4142135623730951f;
  const float a = k * (v + 0.044715f * v * v * v);
  const float t = g_tanh_mode ? (float)tanh((double)a) : tanhf(a);
  return 0.5f * v * (1.0f + t);
}

// ops.rs:130-134
void orc_gelu_mul(float* h, const float* up, size_t n) {
  for (size_t i = 0; i < n; i++) h[i] = orc_gelu(h[i]) * up[i];
}

// ops.rs:144-148
void orc_add_inplace(float* x, const float* y, size_t n) {
  for (size_t i = 0; i < n; i++) x[i] += y[i];
}

// state.rs:308-319
void orc_inv_freq(float* out, size_t rot_dim, float base, const float* freq_factors) {
  for (size_t i = 0; i < rot_dim / 2; i++) {
    float f = powf(base, -(2.0f * (float)i) / (float)rot_dim);
    if (freq_factors) f /= freq_factors[i];
    out[i] = f;
  }
}

// ops.rs:185-218
void orc_attention(orc_pool* p, float* out, const float* q, const float* k_cache, const float* v_cache,
                   float* scores, const orc_dims* d, size_t ctx, size_t layer, size_t pos, size_t window) {
  size_t hd = (size_t)d->head_dim, kv = (size_t)d->n_kv_head * hd, gqa = (size_t)(d->n_head / d->n_kv_head);
  float scale = 1.0f / sqrtf((float)hd);
  size_t base = layer * ctx * kv, n = pos + 1, t0 = window_start(pos, window);
  orc_pool_run(p, [&](int tid, int nth) {
    size_t a, b;
    orc_split((size_t)d->n_head, tid, nth, &a, &b);
    for (size_t h = a; h < b; h++) {
      size_t kvh = h / gqa;
      const float* qh = q + h * hd;
      float* s = scores + h * ctx;
      for (size_t t = t0; t < n; t++) s[t - t0] = dotf(qh, k_cache + base + t * kv + kvh * hd, hd) * scale;
      orc_softmax(s, n - t0);
      float* oh = out + h * hd;
      for (size_t i = 0; i < hd; i++) oh[i] = 0.0f;
      for (size_t t = t0; t < n; t++) {
        float w = s[t - t0];
        const float* vt = v_cache + base + t * kv + kvh * hd;
        for (size_t i = 0; i < hd; i++) oh[i] += w * vt[i];
      }
    }
  });
}

// ops.rs:517-556: work items are (row, head) pairs, one scratch row per thread.
void orc_attention_rows(orc_pool* p, float* out, const float* q, const float* k_cache, const float* v_cache,
                        float* scratch, const orc_dims* d, size_t ctx, size_t layer, size_t pos0, size_t m,
                        size_t window) {
  size_t hd = (size_t)d->head_dim, kv = (size_t)d->n_kv_head * hd, qd = (size_t)d->n_head * hd;
  size_t gqa = (size_t)(d->n_head / d->n_kv_head), nh = (size_t)d->n_head;
  float scale = 1.0f / sqrtf((float)hd);
  size_t base = layer * ctx * kv;
  orc_pool_run(p, [&](int tid, int nth) {
    float* s = scratch + (size_t)tid * ctx;
    size_t a, b;
    orc_split(m * nh, tid, nth, &a, &b);
    for (size_t task = a; task < b; task++) {
      size_t i = task / nh, h = task % nh, kvh = h / gqa;
      size_t n = pos0 + i + 1, t0 = window_start(pos0 + i, window);
      const float* qh = q + i * qd + h * hd;
      for (size_t t = t0; t < n; t++) s[t - t0] = dotf(qh, k_cache + base + t * kv + kvh * hd, hd) * scale;
      orc_softmax(s, n - t0);
      float* oh = out + i * qd + h * hd;
      for (size_t j = 0; j < hd; j++) oh[j] = 0.0f;
      for (size_t t = t0; t < n; t++) {
        float w = s[t - t0];
        const float* vt = v_cache + base + t * kv + kvh * hd;
        for (size_t j = 0; j < hd; j++) oh[j] += w * vt[j];
      }
    }
  });
}

// sampler.rs:99-109: the first maximum wins; NaN never does.
uint32_t orc_argmax(const float* x, size_t n) {
  size_t best = 0;
  float bv = -INFINITY;
  for (size_t i = 0; i < n; i++) {
    if (x[i] > bv) {
      bv = x[i];
      best = i;
    }
  }
  return (uint32_t)best;
}

}  // extern "C"
