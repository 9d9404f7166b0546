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


// Mirror of the device routine (groupsum.cuh): the opening add chain, chunks of SEQ_E
// terms, 32 chunks per group, exponents predicted from an inexact prefix sum (`skew`
// perturbs it, to provoke wrong predictions), integer increments of runs of fast chunks,
// item lists, then the walk shared with the device (seqsum_walk). *slow_chunks receives
// the number of chunks marked slow.
float hc_seqsum_runs(const float* p, size_t n, float skew, int* slow_chunks) {
  static SeqSumScratch sc;
  int n_slow = 0;
  if (n <= (size_t)SEQ_HEAD) {
    float s = 0.0f;
    for (size_t i = 0; i < n; i++) s = fadd(s, p[i]);
    if (slow_chunks) *slow_chunks = 0;
    return s;
  }
  float total = 0.0f;
  for (int i = 0; i < SEQ_HEAD; i++) total = fadd(total, p[i]);
  float approx = 0.0f;
  for (size_t base = 0; base < n; base += (size_t)SEQ_CHUNKS * SEQ_E) {
    const int len = (int)std::min(n - base, (size_t)SEQ_CHUNKS * SEQ_E), nch = (len + SEQ_E - 1) / SEQ_E, ngr = (nch + 31) / 32;
    float before = approx * skew;
    for (int gr = 0; gr < ngr; gr++) {
      const int head_lanes = base == 0 && gr == 0 ? SEQ_HEAD / SEQ_E : 0;
      int n_items = 0, eb_prev = 0, run_inc = 0, run_ep = 0, run_first = 0;
      bool slow_prev = false, in_run = false;
      auto close_run = [&](int end_elem) {
        if (!in_run) return;
        sc.item[32 * gr + n_items++] = SeqItem{run_inc, run_ep, run_first, std::max(0, std::min(len, end_elem) - run_first)};
        in_run = false;
      };
      for (int lane = 0; lane < 32; lane++) {
        const int c = gr * 32 + lane, i0 = c * SEQ_E;
        float t = 0.0f;
        uint32_t vb[SEQ_E];
        int cnt = 0;
        for (int j = 0; j < SEQ_E; j++) {
          const float v = i0 + j < len ? p[base + i0 + j] : 0.0f;
          vb[j] = f2u(v) & 0x7FFFFFFFu;
          cnt += i0 + j < len ? 1 : 0;
          t += v;
        }
        const int eb = seq_exp_field(before), ea = seq_exp_field(before + t);
        const bool live = lane >= head_lanes;
        bool bad = ea != eb || eb >= 255;
        int inc = 0;
        for (int j = 0; j < SEQ_E; j++) inc += seq_increment(vb[j], eb, bad);
        const bool slow = live && cnt > 0 && bad;
        inc = slow || !live ? 0 : std::min(inc, SUMFN_SAT);
        const bool starts = live && (lane == head_lanes || slow_prev || eb != eb_prev);
        if (slow || starts) close_run(i0);
        if (slow) {
          n_slow++;
          sc.item[32 * gr + n_items++] = SeqItem{0, -1, i0, std::max(0, std::min(len, i0 + SEQ_E) - i0)};
        } else if (live) {
          if (!in_run) {
            in_run = true;
            run_inc = 0;
            run_ep = eb;
            run_first = i0;
          }
          run_inc = std::min(run_inc + inc, SUMFN_SAT);
        }
        eb_prev = eb;
        slow_prev = slow;
        before = (before + t) * skew;
      }
      close_run((gr + 1) * 32 * SEQ_E);
      sc.n_items[gr] = n_items;
    }
    total = seqsum_walk(p + base, &sc, ngr, total);
    approx = before;
  }
  if (slow_chunks) *slow_chunks = n_slow;
  return total;
}

}  // extern "C"
