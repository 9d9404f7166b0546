// Sequential-order f32 summation of non-negative terms, evaluated in parallel
// with bit-identical results.
//
// The reference sums squares (rmsnorm, crates/aot-kernels/src/ops.rs:10-13) and
// softmax numerators (ops.rs:103-107) with a scalar loop `s += p[i]`, i.e.
// s_{i+1} = RN(s_i + p_i). A dependent chain of thousands of adds costs several
// microseconds on a GPU. For p_i >= 0 the chain can be evaluated exactly in
// parallel: while s stays inside one binade [2^e, 2^(e+1)) its ulp u is fixed,
// s = M*u with integer M in [2^23, 2^24), and
//     RN(s + p) = (M + c)*u            if frac(p/u) != 1/2   (c = round(p/u))
//               = roundup_even(M+Y)*u  if frac(p/u) == 1/2   (Y = floor(p/u))
// so every term is a function M -> M + A[M & 1] on integers. Such functions are
// closed under composition, which is associative: a prefix scan gives M after
// every term. The first term that pushes M to 2^24 or beyond leaves the binade;
// that single step is redone with a real f32 add (which rounds on the coarser
// grid), and the scan restarts from there. Ties, subnormals, zeros and overflow
// to infinity follow the same rules as the scalar loop.
#pragma once
#include "blockmath.cuh"

namespace aot {

struct SumFn {
  int a0, a1;  // offset applied when the running mantissa is even / odd
};

constexpr int SUMFN_SAT = 1 << 26;    // anything this large has left the binade
constexpr int SUMFN_LIMIT = 1 << 24;  // first mantissa value outside the binade

AOT_HD SumFn sumfn_identity() { return SumFn{0, 0}; }

AOT_HD int sumfn_apply(const SumFn& f, int m) {
  int r = m + ((m & 1) ? f.a1 : f.a0);
  return r > SUMFN_SAT ? SUMFN_SAT : r;
}

// First `f`, then `g`.
AOT_HD SumFn sumfn_compose(const SumFn& f, const SumFn& g) {
  SumFn h;
  int e0 = f.a0, e1 = 1 + f.a1;  // value reached (mod 2 matters) from an even / odd start
  h.a0 = f.a0 + ((e0 & 1) ? g.a1 : g.a0);
  h.a1 = f.a1 + ((e1 & 1) ? g.a1 : g.a0);
  h.a0 = h.a0 > SUMFN_SAT ? SUMFN_SAT : h.a0;
  h.a1 = h.a1 > SUMFN_SAT ? SUMFN_SAT : h.a1;
  return h;
}

// Exponent field (>= 1; subnormals share the ulp of the first normal binade) and
// integer mantissa of a non-negative float: value = m * 2^(e - 150).
AOT_HD void sum_decompose(uint32_t bits, int& e, int& m) {
  e = (int)(bits >> 23);
  m = (int)(bits & 0x7FFFFFu);
  if (e == 0) e = 1; else m |= 0x800000;
}
AOT_HD uint32_t sum_pack(int e, int m) {
  // m < 2^24. m < 2^23 only happens in the lowest binade (subnormal result).
  if (m < 0x800000) return (uint32_t)m;
  return ((uint32_t)e << 23) | ((uint32_t)m & 0x7FFFFFu);
}

// The function of adding the non-negative float with bit pattern `p_bits` while the
// running sum has exponent field `e`.
AOT_HD SumFn sumfn_elem(uint32_t p_bits, int e) {
  int pe, pm;
  sum_decompose(p_bits, pe, pm);
  if (pm == 0) return SumFn{0, 0};
  int sh = e - pe;
  if (sh < 0) return SumFn{SUMFN_SAT, SUMFN_SAT};
  if (sh == 0) return SumFn{pm, pm};
  if (sh > 24) return SumFn{0, 0};
  int y = pm >> sh, r = pm & ((1 << sh) - 1), half = 1 << (sh - 1);
  if (r > half) return SumFn{y + 1, y + 1};
  if (r < half) return SumFn{y, y};
  return (y & 1) ? SumFn{y + 1, y} : SumFn{y, y + 1};  // tie: to even
}

// ---- chunked evaluation ----------------------------------------------------------------
// The device routine (groupsum.cuh) cuts the terms into chunks of SEQ_E consecutive terms,
// one chunk per lane, 32 chunks per group. From an inexact prefix sum it predicts the
// exponent field with which the running sum enters each chunk. A chunk whose predicted
// sum changes binade inside it is "slow": its terms will be added one by one with real
// f32 adds. Every other chunk gets the composite function of its terms for its predicted
// exponent, and consecutive fast chunks with the same predicted exponent form a run
// whose composite is built by a segmented scan. One thread then walks the records below:
// a run is applied in one step when the running sum really has the predicted exponent
// and stays inside the binade, and is otherwise added term by term. Predictions decide
// only which path is taken, never the result.
constexpr int SEQ_E = 8;         // terms per chunk
constexpr int SEQ_CHUNKS = 256;  // chunks per pass (2048 terms)

struct SeqSumScratch {
  int a0[SEQ_CHUNKS];               // composite of the run of fast chunks that ends at this chunk, even start ...
  int a1[SEQ_CHUNKS];               // ... odd start
  int ep[SEQ_CHUNKS];               // predicted exponent field at the chunk's start
  uint32_t slow[SEQ_CHUNKS / 32];   // per group: chunks handled term by term
  uint32_t start[SEQ_CHUNKS / 32];  // per group: chunks at which a run starts
  float gtot[SEQ_CHUNKS / 32];      // inexact sum of each group
  float s;                          // running and final sum
};

AOT_HD int seq_ffs(uint32_t v) {  // index of the lowest set bit, v != 0
#if AOT_DEVICE_CODE
  return __ffs((int)v) - 1;
#else
  return __builtin_ctz(v);
#endif
}

// Terms p[0..len) of one pass, `nch` chunks, records in `sc`; returns start + the terms,
// rounded as the scalar loop rounds.
AOT_HD float seqsum_walk(const float* p, int len, const SeqSumScratch* sc, int nch, float start) {
  int e, m;
  sum_decompose(f2u(start) & 0x7FFFFFFFu, e, m);
  for (int c0 = 0; c0 < nch; c0 += 32) {
    const int gr = c0 >> 5, lanes = nch - c0 < 32 ? nch - c0 : 32;
    const uint32_t slow = sc->slow[gr], bounds = slow | sc->start[gr];
    int lane = 0;
    while (lane < lanes) {
      int end;  // one past the last chunk of this step
      bool by_terms = (slow >> lane) & 1u;
      if (by_terms) {
        end = lane + 1;
      } else {
        const uint32_t above = lane >= 31 ? 0u : (bounds >> (lane + 1)) << (lane + 1);
        end = above ? seq_ffs(above) : 32;
        if (end > lanes) end = lanes;
        const int last = c0 + end - 1;
        const int m2 = m + ((m & 1) ? sc->a1[last] : sc->a0[last]);
        if (e < 255 && sc->ep[c0 + lane] == e && m2 < SUMFN_LIMIT) m = m2; else by_terms = true;
      }
      if (by_terms) {
        float s = u2f(sum_pack(e, m));
        const int i1 = (c0 + end) * SEQ_E < len ? (c0 + end) * SEQ_E : len;
        for (int i = (c0 + lane) * SEQ_E; i < i1; i++) s = fadd(s, p[i]);
        sum_decompose(f2u(s) & 0x7FFFFFFFu, e, m);
      }
      lane = end;
    }
  }
  return u2f(sum_pack(e, m));
}

// Exponent field used for predictions: that of sum_decompose, 255 for anything not finite.
AOT_HD int seq_exp_field(float v) {
  const uint32_t b = f2u(v) & 0x7FFFFFFFu;
  const int e = (int)(b >> 23);
  return e == 0 ? 1 : e;
}

// Composite of the (up to SEQ_E) terms of one chunk for exponent field e.
AOT_HD SumFn seq_chunk_fn(const float* v, int cnt, int e) {
  SumFn f = sumfn_identity();
  for (int j = 0; j < cnt; j++) f = sumfn_compose(f, sumfn_elem(f2u(v[j]) & 0x7FFFFFFFu, e));
  return f;
}

}  // namespace aot
