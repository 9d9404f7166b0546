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

}  // namespace aot
