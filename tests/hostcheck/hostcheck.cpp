// Test-only harness: compiles the library's host/device arithmetic headers as plain
// C++ so the per-block integer sums, the f32 operation order, the element
// dequantizers and the exact expf can be checked against the oracle on a machine
// without a GPU. Nothing in the product links this file.
#include <stddef.h>
#include <stdint.h>

#include "../../aot-llm_b200/csrc/blockmath.cuh"
#include "../../aot-llm_b200/csrc/expf_exact.cuh"
#include "../../aot-llm_b200/csrc/seqsum.cuh"

#include <vector>

using namespace aot;

static inline uint32_t w32(const uint8_t* p, int i) {
  return (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) | ((uint32_t)p[4 * i + 3] << 24);
}

extern "C" {

void hc_expf(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; i++) y[i] = expf_exact(x[i]);
}

// Number of inputs in bit-pattern range [lo, hi) stepping by `step` where expf_exact
// and the C library's expf differ (NaNs skipped).
uint64_t hc_expf_mismatches(uint32_t lo, uint32_t hi, uint32_t step) {
  uint64_t bad = 0;
  for (uint64_t u = lo; u < hi; u += step) {
    float x = u2f((uint32_t)u);
    if (x != x) continue;
    if (f2u(expf_exact(x)) != f2u(expf(x))) bad++;
  }
  return bad;
}

float hc_half(uint16_t h) { return half_bits_to_float(h); }

void hc_dequant_row(int kind, const uint8_t* row, float* out, size_t n) {
  for (size_t e = 0; e < n; e++) out[e] = dequant_elem(kind, row, e);
}

// One full dot product assembled the way the GPU kernels assemble it.
float hc_dot(int kind, const uint8_t* w, const void* xv, size_t cols, int32_t* sumi_out, int32_t* summ_out) {
  if (kind_act(kind) == ACT_Q8_K) {
    const BlockQ8_K* x = (const BlockQ8_K*)xv;
    float sum = 0.0f;
    for (size_t b = 0; b < cols / 256; b++) {
      const uint8_t* wb = w + b * kind_size(kind);
      const BlockQ8_K* y = &x[b];
      auto yw = [&](int i) { return w32((const uint8_t*)y->qs, i); };
      float term;
      if (kind == Q6_K) {
        int si = q6k_block_sum([&](int i) { return w32(wb, i); }, yw, y->bsums);
        if (sumi_out) sumi_out[b] = si;
        term = q6k_term(half_bits_to_float(w32(wb, 52) & 0xFFFF), y->d, si);
      } else {
        const bool q5 = kind == Q5_K;
        K4Scales s = k4_unpack(w32(wb + 4, 0), w32(wb + 4, 1), w32(wb + 4, 2));
        const uint8_t* qs = wb + (q5 ? 48 : 16);
        const uint8_t* qh = wb + 16;
        int si, sm;
        if (q5) k4_block_sums<true>(s, [&](int i) { return w32(qs, i); }, [&](int i) { return w32(qh, i); }, yw, y->bsums, si, sm);
        else k4_block_sums<false>(s, [&](int i) { return w32(qs, i); }, [&](int i) { return w32(qh, i); }, yw, y->bsums, si, sm);
        if (sumi_out) sumi_out[b] = si;
        if (summ_out) summ_out[b] = sm;
        uint32_t h = w32(wb, 0);
        term = k4_term(half_bits_to_float(h & 0xFFFF), half_bits_to_float(h >> 16), y->d, si, sm);
      }
      sum = fadd(sum, term);
    }
    return sum;
  }
  if (kind_act(kind) == ACT_Q8_0) {
    const BlockQ8_0* x = (const BlockQ8_0*)xv;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t b = 0; b < cols / 32; b++) {
      const uint8_t* wb = w + b * kind_size(kind);
      const BlockQ8_0* y = &x[b];
      uint32_t h = (uint32_t)wb[0] | ((uint32_t)wb[1] << 8);
      float d = fmul(half_bits_to_float(h), y->d);
      int tot = 0;
      for (int k = 0; k < 8; k++) {
        uint32_t y4 = w32((const uint8_t*)y->qs, k);
        int p;
        if (kind == Q8_0) p = q8_0_lane(w32(wb + 2, k), y4);
        else if (kind == Q4_0) p = q4_0_lane(w32(wb + 2, k & 3), k, y4);
        else p = q5_0_lane(w32(wb + 6, k & 3), w32(wb + 2, 0), k, y4);
        tot += p;
        acc[k] = ffma(d, i2f(p), acc[k]);
      }
      if (sumi_out) sumi_out[b] = tot;
    }
    return hsum8(acc);
  }
  const float* x = (const float*)xv;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  size_t n8 = cols & ~(size_t)7;
  auto wf = [&](size_t j) {
    if (kind == F32) return u2f(w32(w, (int)j));
    uint32_t h = (uint32_t)w[2 * j] | ((uint32_t)w[2 * j + 1] << 8);
    return kind == F16 ? half_bits_to_float(h) : bf16_bits_to_float(h);
  };
  for (size_t j = 0; j < n8; j++) acc[j & 7] = ffma(wf(j), x[j], acc[j & 7]);
  float sum = hsum8(acc);
  for (size_t j = n8; j < cols; j++) sum = fadd(sum, fmul(wf(j), x[j]));
  return sum;
}


// The parallel evaluation of the sequential sum, simulated with T "threads" that own
// contiguous chunks (the same steps as the device routine: serial head, per-chunk
// composition, exclusive scan over chunks, replay to find the first term that leaves
// the binade, one real add, repeat). Returns the sum; *rounds receives the number of
// scan rounds.
float hc_seqsum(const float* p, size_t n, int T, int head, int* rounds) {
  float s = 0.0f;
  size_t i0 = 0;
  for (; i0 < n && (int)i0 < head; i0++) s = fadd(s, p[i0]);
  int nr = 0;
  while (i0 < n) {
    uint32_t sb = f2u(s);
    if ((sb >> 23) == 255) {  // inf / nan: finish serially
      for (; i0 < n; i0++) s = fadd(s, p[i0]);
      break;
    }
    nr++;
    int e, m0;
    sum_decompose(sb, e, m0);
    size_t rem = n - i0, C = (rem + T - 1) / T;
    std::vector<SumFn> comp(T), pre(T);
    for (int t = 0; t < T; t++) {
      SumFn f = sumfn_identity();
      for (size_t i = i0 + t * C; i < i0 + (t + 1) * C && i < n; i++) f = sumfn_compose(f, sumfn_elem(f2u(p[i]), e));
      comp[t] = f;
    }
    SumFn run = sumfn_identity();
    for (int t = 0; t < T; t++) {
      pre[t] = run;
      run = sumfn_compose(run, comp[t]);
    }
    size_t ov = n;
    int m_at = 0, m_final = sumfn_apply(run, m0);
    for (int t = 0; t < T && ov == n; t++) {
      int m = sumfn_apply(pre[t], m0);
      if (m >= SUMFN_LIMIT) break;
      for (size_t i = i0 + t * C; i < i0 + (t + 1) * C && i < n; i++) {
        int m2 = sumfn_apply(sumfn_elem(f2u(p[i]), e), m);
        if (m2 >= SUMFN_LIMIT) {
          ov = i;
          m_at = m;
          break;
        }
        m = m2;
      }
    }
    if (ov == n) {
      s = u2f(sum_pack(e, m_final));
      break;
    }
    s = fadd(u2f(sum_pack(e, m_at)), p[ov]);
    i0 = ov + 1;
  }
  if (rounds) *rounds = nr;
  return s;
}


// The speculative segmented evaluation used on the device: 32-term segments, the
// starting binade of each segment predicted from an inexact prefix sum, one exact
// composite per segment, then a serial walk that applies a composite when the
// prediction holds and the result stays inside the binade, and otherwise adds the
// segment's terms one by one. *fallbacks receives the number of serial segments.
float hc_seqsum_seg(const float* p, size_t n, int* fallbacks) {
  const size_t S = (n + 31) / 32;
  std::vector<float> est(S + 1, 0.0f);
  for (size_t g = 0; g < S; g++) {
    float t = 0.0f;  // any estimate works; use a pairwise-looking sum
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) t += p[i];
    est[g + 1] = est[g] + t;
  }
  std::vector<SumFn> comp(S);
  std::vector<int> epred(S);
  for (size_t g = 0; g < S; g++) {
    int e, m;
    uint32_t b = f2u(est[g]);
    if ((b >> 23) == 255) b = 0x7f000000u;
    sum_decompose(b, e, m);
    epred[g] = e;
    SumFn f = sumfn_identity();
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) f = sumfn_compose(f, sumfn_elem(f2u(p[i]), e));
    comp[g] = f;
  }
  float s = 0.0f;
  int nf = 0;
  for (size_t g = 0; g < S; g++) {
    uint32_t sb = f2u(s);
    int e, m;
    sum_decompose(sb, e, m);
    if ((sb >> 23) != 255 && e == epred[g]) {
      int m2 = sumfn_apply(comp[g], m);
      if (m2 < SUMFN_LIMIT) {
        s = u2f(sum_pack(e, m2));
        continue;
      }
    }
    nf++;
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) s = fadd(s, p[i]);
  }
  if (fallbacks) *fallbacks = nf;
  return s;
}


// Mirror of the device routine's final form: per 32-term segment an integer increment
// C = sum round(p/u) for the predicted binade, flagged "bad" when a term is an exact
// tie or leaves the binade; the walk adds integer prefix sums over runs of good
// segments and falls back to term-by-term adds for bad ones.
float hc_seqsum_int(const float* p, size_t n, int* fallbacks) {
  const size_t S = (n + 31) / 32;
  std::vector<float> est(S + 1, 0.0f);
  for (size_t g = 0; g < S; g++) {
    float t = 0.0f;
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) t += p[i];
    est[g + 1] = est[g] + t;
  }
  std::vector<int> csum(S), epred(S);
  for (size_t g = 0; g < S; g++) {
    uint32_t b = f2u(est[g]);
    if ((b >> 23) >= 255u || (b >> 31)) b = 0;
    int e, m;
    sum_decompose(b, e, m);
    long long C = 0;
    bool bad = false;
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) {
      SumFn f = sumfn_elem(f2u(p[i]), e);
      if (f.a0 != f.a1 || f.a0 >= SUMFN_SAT) bad = true;
      C += f.a0 > (1 << 25) ? (1 << 25) : f.a0;
    }
    csum[g] = (int)C;
    epred[g] = bad ? -1 : e;
  }
  int e, m, nf = 0;
  sum_decompose(0u, e, m);
  for (size_t g = 0; g < S; g++) {
    if (epred[g] == e && m + csum[g] < SUMFN_LIMIT) {
      m += csum[g];
      continue;
    }
    nf++;
    float s = u2f(sum_pack(e, m));
    for (size_t i = g * 32; i < n && i < (g + 1) * 32; i++) s = fadd(s, p[i]);
    sum_decompose(f2u(s), e, m);
  }
  if (fallbacks) *fallbacks = nf;
  return u2f(sum_pack(e, m));
}

}  // extern "C"
