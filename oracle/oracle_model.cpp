// Oracle (test infrastructure): the per-layer unrolled forward pass that
// crates/aot-codegen/src/emit.rs generates (emit_layer 243-333, emit_layer_batch
// 167-237, forward / forward_batch 466-516), interpreted here from a tensor
// table instead of being emitted as source, over buffers laid out like
// crates/aot-kernels/src/state.rs:251-361.
#include <math.h>
#include <string.h>

#include <string>
#include <vector>

#include "oracle_internal.h"

struct orc_model {
  orc_model_head head;
  std::vector<orc_layer> layers;
  const uint8_t* w = nullptr;
  size_t w_len = 0;
  size_t ctx = 0, max_batch = 1;
  int table = 0;
  orc_pool* pool = nullptr;
  // State
  std::vector<float> x, xb, xb2, q, k, v, hb, hb2, logits, scores, k_cache, v_cache;
  std::vector<float> inv_freq, rope_cs, inv_freq_local, rope_cs_local;
  std::vector<float> bx, bxb, bxb2, bq, bk, bv, bhb, bhb2, brope_cs, brope_cs_local;
  std::vector<orc_block_q8_0> aq0, baq0;
  std::vector<orc_block_q8_k> aqk, baqk;
};

static const float* f32s(const orc_model* m, const orc_tensor& t) { return (const float*)(m->w + t.off); }
static const uint8_t* bytes(const orc_model* m, const orc_tensor& t) { return m->w + t.off; }

// emit.rs:131-139: one quantize call per distinct activation format, Q8_0 first
// (BTreeSet order F32 < Q8_0 < Q8_K).
static void quantize_for(orc_model* m, const float* src, size_t n, const int* kinds, int nk) {
  bool q0 = false, qk = false;
  for (int i = 0; i < nk; i++) {
    int a = orc_activation(kinds[i]);
    q0 |= a == ORC_ACT_Q8_0;
    qk |= a == ORC_ACT_Q8_K;
  }
  if (q0) {
    m->aq0.resize(n / 32);
    orc_quantize_q8_0(src, n, m->aq0.data());
  }
  if (qk) {
    m->aqk.resize(n / 256);
    orc_quantize_q8_k(src, n, m->aqk.data());
  }
}

// ops.rs:466-501 only spread the same per-block arithmetic over the pool.
static void quantize_rows_for(orc_model* m, const float* src, size_t n_total, const int* kinds, int nk) {
  bool q0 = false, qk = false;
  for (int i = 0; i < nk; i++) {
    int a = orc_activation(kinds[i]);
    q0 |= a == ORC_ACT_Q8_0;
    qk |= a == ORC_ACT_Q8_K;
  }
  if (q0) {
    m->baq0.resize(n_total / 32);
    orc_block_q8_0* o = m->baq0.data();
    orc_pool_run_chunks(m->pool, n_total / 32, 32,
                        [&](size_t a, size_t b) { orc_quantize_q8_0(src + a * 32, (b - a) * 32, o + a); });
  }
  if (qk) {
    m->baqk.resize(n_total / 256);
    orc_block_q8_k* o = m->baqk.data();
    orc_pool_run_chunks(m->pool, n_total / 256, 4,
                        [&](size_t a, size_t b) { orc_quantize_q8_k(src + a * 256, (b - a) * 256, o + a); });
  }
}

static const void* act_ptr(const orc_model* m, int kind, const float* src) {
  int a = orc_activation(kind);
  if (a == ORC_ACT_Q8_0) return m->aq0.data();
  if (a == ORC_ACT_Q8_K) return m->aqk.data();
  return src;
}

static const void* bact_ptr(const orc_model* m, int kind, const float* src) {
  int a = orc_activation(kind);
  if (a == ORC_ACT_Q8_0) return m->baq0.data();
  if (a == ORC_ACT_Q8_K) return m->baqk.data();
  return src;
}

static void mv(orc_model* m, const orc_tensor& t, float* dst, const float* src) {
  orc_matvec(m->pool, m->table, t.kind, dst, bytes(m, t), act_ptr(m, t.kind, src), t.rows, t.cols);
}

static void mm(orc_model* m, const orc_tensor& t, float* dst, const float* src, size_t n) {
  orc_matmul(m->pool, m->table, t.kind, dst, bytes(m, t), bact_ptr(m, t.kind, src), n, t.rows, t.cols);
}

// emit.rs:243-333
static void layer_decode(orc_model* m, size_t li, size_t pos) {
  const orc_layer& l = m->layers[li];
  const orc_dims& d = m->head.dims;
  size_t dim = d.dim, qd = (size_t)d.n_head * d.head_dim, kvd = (size_t)d.n_kv_head * d.head_dim;
  const float* cs = l.local_attn ? m->rope_cs_local.data() : m->rope_cs.data();
  size_t window = l.local_attn ? (size_t)d.swa_window : 0;

  orc_rmsnorm(m->xb.data(), m->x.data(), f32s(m, l.attn_norm), dim, d.eps);
  int kq[3] = {l.wq.kind, l.wk.kind, l.wv.kind};
  quantize_for(m, m->xb.data(), dim, kq, 3);
  bool same = l.wq.kind == l.wk.kind && l.wk.kind == l.wv.kind && orc_activation(l.wq.kind) != ORC_ACT_F32;
  if (same) {
    orc_matvec3(m->pool, m->table, l.wq.kind, m->q.data(), m->k.data(), m->v.data(), bytes(m, l.wq),
                bytes(m, l.wk), bytes(m, l.wv), act_ptr(m, l.wq.kind, m->xb.data()), l.wq.rows, l.wk.rows,
                l.wv.rows, l.wq.cols);
  } else {
    mv(m, l.wq, m->q.data(), m->xb.data());
    mv(m, l.wk, m->k.data(), m->xb.data());
    mv(m, l.wv, m->v.data(), m->xb.data());
  }
  if (d.qkv_bias) {
    orc_add_inplace(m->q.data(), f32s(m, l.bq), qd);
    orc_add_inplace(m->k.data(), f32s(m, l.bk), kvd);
    orc_add_inplace(m->v.data(), f32s(m, l.bv), kvd);
  }
  if (d.qk_norm) {
    orc_rmsnorm_heads(m->q.data(), f32s(m, l.q_norm), d.n_head, d.head_dim, d.eps);
    orc_rmsnorm_heads(m->k.data(), f32s(m, l.k_norm), d.n_kv_head, d.head_dim, d.eps);
  }
  if (d.rope_neox) {
    orc_rope_neox(m->q.data(), d.n_head, d.head_dim, d.rot_dim, cs);
    orc_rope_neox(m->k.data(), d.n_kv_head, d.head_dim, d.rot_dim, cs);
  } else {
    orc_rope(m->q.data(), d.n_head, d.head_dim, d.rot_dim, cs);
    orc_rope(m->k.data(), d.n_kv_head, d.head_dim, d.rot_dim, cs);
  }
  // ops.rs:152-157
  size_t at = (li * m->ctx + pos) * kvd;
  memcpy(&m->k_cache[at], m->k.data(), kvd * 4);
  memcpy(&m->v_cache[at], m->v.data(), kvd * 4);
  orc_attention(m->pool, m->xb.data(), m->q.data(), m->k_cache.data(), m->v_cache.data(), m->scores.data(), &d,
                m->ctx, li, pos, window);
  int ko[1] = {l.wo.kind};
  quantize_for(m, m->xb.data(), qd, ko, 1);
  mv(m, l.wo, m->xb2.data(), m->xb.data());
  if (d.post_norms) {
    orc_rmsnorm(m->xb.data(), m->xb2.data(), f32s(m, l.attn_post_norm), dim, d.eps);
    orc_add_inplace(m->x.data(), m->xb.data(), dim);
  } else {
    orc_add_inplace(m->x.data(), m->xb2.data(), dim);
  }

  orc_rmsnorm(m->xb.data(), m->x.data(), f32s(m, l.ffn_norm), dim, d.eps);
  int kg[2] = {l.gate.kind, l.up.kind};
  quantize_for(m, m->xb.data(), dim, kg, 2);
  bool fused = l.gate.kind == l.up.kind && orc_activation(l.gate.kind) != ORC_ACT_F32;
  if (fused) {
    orc_matvec2(m->pool, m->table, l.gate.kind, m->hb.data(), m->hb2.data(), bytes(m, l.gate), bytes(m, l.up),
                act_ptr(m, l.gate.kind, m->xb.data()), l.gate.rows, l.gate.cols);
  } else {
    mv(m, l.gate, m->hb.data(), m->xb.data());
    mv(m, l.up, m->hb2.data(), m->xb.data());
  }
  if (d.gelu) {
    orc_gelu_mul(m->hb.data(), m->hb2.data(), d.hidden);
  } else {
    orc_silu_mul(m->hb.data(), m->hb2.data(), d.hidden);
  }
  int kd[1] = {l.down.kind};
  quantize_for(m, m->hb.data(), d.hidden, kd, 1);
  mv(m, l.down, m->xb2.data(), m->hb.data());
  if (d.post_norms) {
    orc_rmsnorm(m->xb.data(), m->xb2.data(), f32s(m, l.ffn_post_norm), dim, d.eps);
    orc_add_inplace(m->x.data(), m->xb.data(), dim);
  } else {
    orc_add_inplace(m->x.data(), m->xb2.data(), dim);
  }
}

// emit.rs:167-237
static void layer_batch(orc_model* m, size_t li, size_t pos0, size_t n) {
  const orc_layer& l = m->layers[li];
  const orc_dims& d = m->head.dims;
  size_t dim = d.dim, hidden = d.hidden, qd = (size_t)d.n_head * d.head_dim, kvd = (size_t)d.n_kv_head * d.head_dim;
  size_t xbw = dim > qd ? dim : qd;
  (void)xbw;
  const float* cs = l.local_attn ? m->brope_cs_local.data() : m->brope_cs.data();
  size_t window = l.local_attn ? (size_t)d.swa_window : 0;
  size_t rot = d.rot_dim;

  for (size_t i = 0; i < n; i++)
    orc_rmsnorm(&m->bxb[i * dim], &m->bx[i * dim], f32s(m, l.attn_norm), dim, d.eps);
  int kq[3] = {l.wq.kind, l.wk.kind, l.wv.kind};
  quantize_rows_for(m, m->bxb.data(), n * dim, kq, 3);
  mm(m, l.wq, m->bq.data(), m->bxb.data(), n);
  mm(m, l.wk, m->bk.data(), m->bxb.data(), n);
  mm(m, l.wv, m->bv.data(), m->bxb.data(), n);
  if (d.qkv_bias) {
    for (size_t i = 0; i < n; i++) {
      orc_add_inplace(&m->bq[i * qd], f32s(m, l.bq), qd);
      orc_add_inplace(&m->bk[i * kvd], f32s(m, l.bk), kvd);
      orc_add_inplace(&m->bv[i * kvd], f32s(m, l.bv), kvd);
    }
  }
  if (d.qk_norm) {
    orc_rmsnorm_heads(m->bq.data(), f32s(m, l.q_norm), n * d.n_head, d.head_dim, d.eps);
    orc_rmsnorm_heads(m->bk.data(), f32s(m, l.k_norm), n * d.n_kv_head, d.head_dim, d.eps);
  }
  for (size_t i = 0; i < n; i++) {
    if (d.rope_neox) {
      orc_rope_neox(&m->bq[i * qd], d.n_head, d.head_dim, rot, cs + i * rot);
      orc_rope_neox(&m->bk[i * kvd], d.n_kv_head, d.head_dim, rot, cs + i * rot);
    } else {
      orc_rope(&m->bq[i * qd], d.n_head, d.head_dim, rot, cs + i * rot);
      orc_rope(&m->bk[i * kvd], d.n_kv_head, d.head_dim, rot, cs + i * rot);
    }
  }
  size_t at = (li * m->ctx + pos0) * kvd;
  memcpy(&m->k_cache[at], m->bk.data(), n * kvd * 4);
  memcpy(&m->v_cache[at], m->bv.data(), n * kvd * 4);
  orc_attention_rows(m->pool, m->bxb.data(), m->bq.data(), m->k_cache.data(), m->v_cache.data(), m->scores.data(),
                     &d, m->ctx, li, pos0, n, window);
  int ko[1] = {l.wo.kind};
  quantize_rows_for(m, m->bxb.data(), n * qd, ko, 1);
  mm(m, l.wo, m->bxb2.data(), m->bxb.data(), n);
  if (d.post_norms) {
    for (size_t i = 0; i < n; i++)
      orc_rmsnorm(&m->bxb[i * dim], &m->bxb2[i * dim], f32s(m, l.attn_post_norm), dim, d.eps);
    orc_add_inplace(m->bx.data(), m->bxb.data(), n * dim);
  } else {
    orc_add_inplace(m->bx.data(), m->bxb2.data(), n * dim);
  }
  for (size_t i = 0; i < n; i++)
    orc_rmsnorm(&m->bxb[i * dim], &m->bx[i * dim], f32s(m, l.ffn_norm), dim, d.eps);
  int kg[2] = {l.gate.kind, l.up.kind};
  quantize_rows_for(m, m->bxb.data(), n * dim, kg, 2);
  mm(m, l.gate, m->bhb.data(), m->bxb.data(), n);
  mm(m, l.up, m->bhb2.data(), m->bxb.data(), n);
  if (d.gelu) {
    orc_gelu_mul(m->bhb.data(), m->bhb2.data(), n * hidden);
  } else {
    orc_silu_mul(m->bhb.data(), m->bhb2.data(), n * hidden);
  }
  int kd[1] = {l.down.kind};
  quantize_rows_for(m, m->bhb.data(), n * hidden, kd, 1);
  mm(m, l.down, m->bxb2.data(), m->bhb.data(), n);
  if (d.post_norms) {
    for (size_t i = 0; i < n; i++)
      orc_rmsnorm(&m->bxb[i * dim], &m->bxb2[i * dim], f32s(m, l.ffn_post_norm), dim, d.eps);
    orc_add_inplace(m->bx.data(), m->bxb.data(), n * dim);
  } else {
    orc_add_inplace(m->bx.data(), m->bxb2.data(), n * dim);
  }
}

static void logits_from(orc_model* m, const float* xrow) {
  const orc_dims& d = m->head.dims;
  const orc_tensor& out_t = m->head.output.present ? m->head.output : m->head.token_embd;
  orc_rmsnorm(m->xb.data(), xrow, f32s(m, m->head.output_norm), d.dim, d.eps);
  int ko[1] = {out_t.kind};
  quantize_for(m, m->xb.data(), d.dim, ko, 1);
  mv(m, out_t, m->logits.data(), m->xb.data());
}

extern "C" {

orc_model* orc_model_new(const orc_model_head* head, const orc_layer* layers, const uint8_t* weights,
                         size_t weights_len, size_t ctx, size_t max_batch, int n_threads, int table) {
  orc_model* m = new orc_model();
  m->head = *head;
  const orc_dims& d = m->head.dims;
  m->layers.assign(layers, layers + d.n_layer);
  m->w = weights;
  m->w_len = weights_len;
  m->ctx = ctx;
  m->max_batch = max_batch < 1 ? 1 : max_batch;
  m->table = table;
  m->pool = orc_pool_new(n_threads);
  size_t dim = d.dim, qd = (size_t)d.n_head * d.head_dim, kvd = (size_t)d.n_kv_head * d.head_dim;
  size_t xbw = dim > qd ? dim : qd;
  size_t b = m->max_batch > 1 ? m->max_batch : 0;
  size_t nth = (size_t)n_threads;
  m->x.assign(dim, 0);
  m->xb.assign(xbw, 0);
  m->xb2.assign(dim, 0);
  m->q.assign(qd, 0);
  m->k.assign(kvd, 0);
  m->v.assign(kvd, 0);
  m->hb.assign(d.hidden, 0);
  m->hb2.assign(d.hidden, 0);
  m->logits.assign(d.vocab, 0);
  m->scores.assign(((size_t)d.n_head > nth ? (size_t)d.n_head : nth) * ctx, 0);
  m->k_cache.assign((size_t)d.n_layer * ctx * kvd, 0);
  m->v_cache.assign((size_t)d.n_layer * ctx * kvd, 0);
  m->inv_freq.assign(d.rot_dim / 2, 0);
  const float* ff = m->head.rope_freqs.present ? f32s(m, m->head.rope_freqs) : nullptr;
  orc_inv_freq(m->inv_freq.data(), d.rot_dim, d.rope_base, ff);
  m->rope_cs.assign(d.rot_dim, 0);
  if (d.swa_window > 0) {
    m->inv_freq_local.assign(d.rot_dim / 2, 0);
    orc_inv_freq(m->inv_freq_local.data(), d.rot_dim, d.rope_base_local, ff);
    m->rope_cs_local.assign(d.rot_dim, 0);
    m->brope_cs_local.assign(b * d.rot_dim, 0);
  }
  m->bx.assign(b * dim, 0);
  m->bxb.assign(b * xbw, 0);
  m->bxb2.assign(b * dim, 0);
  m->bq.assign(b * qd, 0);
  m->bk.assign(b * kvd, 0);
  m->bv.assign(b * kvd, 0);
  m->bhb.assign(b * d.hidden, 0);
  m->bhb2.assign(b * d.hidden, 0);
  m->brope_cs.assign(b * d.rot_dim, 0);
  return m;
}

void orc_model_free(orc_model* m) {
  if (!m) return;
  orc_pool_free(m->pool);
  delete m;
}

// emit.rs:466-486
int orc_forward(orc_model* m, uint32_t token, size_t pos, int want_logits) {
  const orc_dims& d = m->head.dims;
  if (token >= (uint32_t)d.vocab || pos >= m->ctx) return -1;
  const orc_tensor& e = m->head.token_embd;
  orc_dequant_row(e.kind, m->w + e.off + (size_t)token * orc_row_bytes(e.kind, e.cols), m->x.data(), d.dim);
  if (d.embd_scale) {
    float s = sqrtf((float)d.dim);
    for (int i = 0; i < d.dim; i++) m->x[i] *= s;
  }
  orc_rope_cos_sin(m->rope_cs.data(), m->inv_freq.data(), d.rot_dim / 2, (float)pos / d.rope_scale);
  if (d.swa_window > 0)
    orc_rope_cos_sin(m->rope_cs_local.data(), m->inv_freq_local.data(), d.rot_dim / 2, (float)pos / d.rope_scale_local);
  for (int i = 0; i < d.n_layer; i++) layer_decode(m, (size_t)i, pos);
  if (want_logits) logits_from(m, m->x.data());
  return 0;
}

// emit.rs:491-516
int orc_forward_batch(orc_model* m, const uint32_t* tokens, size_t n, size_t pos0, int want_logits) {
  const orc_dims& d = m->head.dims;
  if (n < 1 || n > m->max_batch || m->max_batch < 2 || pos0 + n > m->ctx) return -1;
  const orc_tensor& e = m->head.token_embd;
  for (size_t i = 0; i < n; i++) {
    if (tokens[i] >= (uint32_t)d.vocab) return -1;
    orc_dequant_row(e.kind, m->w + e.off + (size_t)tokens[i] * orc_row_bytes(e.kind, e.cols), &m->bx[i * d.dim], d.dim);
  }
  if (d.embd_scale) {
    float s = sqrtf((float)d.dim);
    for (size_t i = 0; i < n * d.dim; i++) m->bx[i] *= s;
  }
  // ops.rs:367-372
  for (size_t i = 0; i < n; i++)
    orc_rope_cos_sin(&m->brope_cs[i * d.rot_dim], m->inv_freq.data(), d.rot_dim / 2, (float)(pos0 + i) / d.rope_scale);
  if (d.swa_window > 0)
    for (size_t i = 0; i < n; i++)
      orc_rope_cos_sin(&m->brope_cs_local[i * d.rot_dim], m->inv_freq_local.data(), d.rot_dim / 2,
                       (float)(pos0 + i) / d.rope_scale_local);
  for (int i = 0; i < d.n_layer; i++) layer_batch(m, (size_t)i, pos0, n);
  if (want_logits) logits_from(m, &m->bx[(n - 1) * d.dim]);
  return 0;
}

float* orc_state_buf(orc_model* m, const char* name, size_t* len) {
  struct E {
    const char* n;
    std::vector<float>* v;
  } tab[] = {{"x", &m->x}, {"xb", &m->xb}, {"xb2", &m->xb2}, {"q", &m->q}, {"k", &m->k}, {"v", &m->v},
             {"hb", &m->hb}, {"hb2", &m->hb2}, {"logits", &m->logits}, {"k_cache", &m->k_cache},
             {"v_cache", &m->v_cache}, {"rope_cs", &m->rope_cs}, {"inv_freq", &m->inv_freq}, {"bx", &m->bx},
             {"bxb", &m->bxb}, {"bxb2", &m->bxb2}, {"bq", &m->bq}, {"bk", &m->bk}, {"bv", &m->bv},
             {"bhb", &m->bhb}, {"bhb2", &m->bhb2}, {"brope_cs", &m->brope_cs}};
  for (auto& e : tab) {
    if (std::string(e.n) == name) {
      if (len) *len = e.v->size();
      return e.v->data();
    }
  }
  return nullptr;
}

const void* orc_state_aqk(orc_model* m, size_t* n_blocks) {
  if (n_blocks) *n_blocks = m->aqk.size();
  return m->aqk.data();
}

const void* orc_state_aq0(orc_model* m, size_t* n_blocks) {
  if (n_blocks) *n_blocks = m->aq0.size();
  return m->aq0.data();
}

}  // extern "C"
