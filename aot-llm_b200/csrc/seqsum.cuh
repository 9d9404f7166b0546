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
#include <stdint.h>
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
// sum changes binade inside it, or that holds an exact tie or a term as large as the
// binade, is "slow": its terms will be added one by one with real f32 adds. Every other
// chunk gets the integer by which its terms advance the mantissa for its predicted
// exponent, and consecutive fast chunks with the same predicted exponent form a run whose
// increment is built by a segmented scan. The result is a short list of items per group,
// in term order; one thread walks it: an item is applied in one step when the running sum
// really has the predicted exponent and stays inside the binade, and is otherwise added
// term by term. Predictions decide only which path is taken, never the result. The first
// SEQ_HEAD terms, where the sum changes binade every few terms, are one plain add chain.
constexpr int SEQ_E = 8;         // terms per chunk
constexpr int SEQ_CHUNKS = 256;  // chunks per pass (2048 terms)
constexpr int SEQ_HEAD = 64;     // terms of the opening add chain (a multiple of SEQ_E)

struct SeqItem {
  int csum;   // mantissa increment of the whole item for exponent field ep
  int ep;     // predicted exponent field at the item's start; -1: add term by term
  int first;  // index of the item's first term inside the pass
  int count;  // terms
};

struct SeqSumScratch {
  SeqItem item[SEQ_CHUNKS];        // group g's items start at item[32 g]
  int n_items[SEQ_CHUNKS / 32];
  float gtot[SEQ_CHUNKS / 32];     // inexact sum of each group
  float excl[SEQ_CHUNKS];          // inexact sum of the group's chunks before this one
  float s;                         // running and final sum
  float head;                      // sum of the opening chain
};

// Mantissa increment of adding p (bit pattern, non-negative) while the sum has exponent
// field e, without branches. `bad` is set when the add cannot be an integer step: p is as
// large as the binade, or the dropped bits are an exact tie.
AOT_HD int seq_increment(uint32_t bits, int e, bool& bad) {
  int pe = (int)(bits >> 23);
  const uint32_t pm = (bits & 0x7FFFFFu) | (pe ? 0x800000u : 0u);
  pe = pe ? pe : 1;
  const int sh = e - pe;
  const int shc = sh < 1 ? 1 : (sh > 25 ? 25 : sh);
  const uint32_t y = pm >> shc, r = pm & ((1u << shc) - 1u), half = 1u << (shc - 1);
  bad = bad || (sh < 1 && bits != 0u) || (r == half && pm != 0u);
  return (int)(y + (r > half ? 1u : 0u));
}

// Items of one pass in order -> start + the terms p[0..), rounded as the scalar loop rounds.
// The running sum is kept as its bit pattern: for a normal float, adding an integer to the
// pattern adds it to the mantissa, and the sum has left the binade exactly when the
// exponent field changes. The next item is fetched while the current one is applied.
AOT_HD float seqsum_walk(const float* p, const SeqSumScratch* sc, int n_groups, float start) {
  uint32_t bits = f2u(start) & 0x7FFFFFFFu;
  for (int g = 0; g < n_groups; g++) {
    const int cnt = sc->n_items[g];
    const SeqItem* items = sc->item + 32 * g;
    SeqItem nxt = items[0];
    for (int k = 0; k < cnt; k++) {
      const SeqItem it = nxt;
      if (k + 1 < cnt) nxt = items[k + 1];
      // ep >= 2: the pattern arithmetic needs a normal sum (the lowest binade, which
      // includes the subnormals, goes term by term)
      const uint32_t nb = bits + (uint32_t)it.csum;
      const bool fits = (it.ep >= 2) & ((int)(bits >> 23) == it.ep) & ((int)(nb >> 23) == it.ep);
      if (fits) {
        bits = nb;
        continue;
      }
      float s = u2f(bits);
      const float* q = p + it.first;
      if (it.count == SEQ_E) {
        const float a0 = q[0], a1 = q[1], a2 = q[2], a3 = q[3], a4 = q[4], a5 = q[5], a6 = q[6], a7 = q[7];
        s = fadd(s, a0);
        s = fadd(s, a1);
        s = fadd(s, a2);
        s = fadd(s, a3);
        s = fadd(s, a4);
        s = fadd(s, a5);
        s = fadd(s, a6);
        s = fadd(s, a7);
      } else {
        for (int i = 0; i < it.count; i++) s = fadd(s, q[i]);
      }
      bits = f2u(s) & 0x7FFFFFFFu;
    }
  }
  return u2f(bits);
}

// Exponent field used for predictions: that of sum_decompose, 255 for anything not finite.
AOT_HD int seq_exp_field(float v) {
  const uint32_t b = f2u(v) & 0x7FFFFFFFu;
  const int e = (int)(b >> 23);
  return e == 0 ? 1 : e;
}

}  // namespace aot
