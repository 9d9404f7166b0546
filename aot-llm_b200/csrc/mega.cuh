// One decode step (crates/aot-codegen/src/emit.rs:243-333, 466-486) as a single
// persistent kernel: one CTA per SM, a producer warp that streams this CTA's
// share of every weight matrix of the step through a shared-memory ring with 1-D
// bulk copies (it runs ahead across phases, because weights never depend on
// activations) and consumer warps that do the arithmetic. Activation vectors pass
// from one phase to the next as tagged 64-bit words (value + phase tag in one store),
// so a consumer starts as soon as the words it needs have arrived; the only grid-wide
// barrier left is the one in front of the argmax. All results are bit-identical to the
// reference's CPU path (see blockmath.cuh, seqsum.cuh, expf_exact.cuh).
#pragma once
#include <cuda_fp16.h>

#include "blockmath.cuh"
#include "device_utils.cuh"
#include "expf_exact.cuh"
#include "gemv.cuh"
#include "groupsum.cuh"
#include "ops.cuh"
#include "seqsum.cuh"

namespace aot {

// ---- warp-per-row dot products, four lanes per 256-weight super-block -----------------
__device__ __forceinline__ float half_to_float_hw(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

__device__ __forceinline__ U4 lds128q(uint32_t a) {
  U4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32q(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

// Lane (b = lane/4, c = lane%4) of a warp: quarter c of block b. Returns the two
// integers of the whole block (summed over the four lanes) to all four lanes, and the
// block's d|dmin word.
template <bool Q5>
__device__ __forceinline__ void quarter_k4(uint32_t wb, uint32_t xb, int c, int& sumi, int& summ, uint32_t& dd) {
  const U4 hdr = lds128q(wb);
  dd = hdr.x;
  const K4Scales s = k4_unpack(hdr.y, hdr.z, hdr.w);
  const uint32_t qs = wb + (Q5 ? 48 : 16) + 32 * c;
  const U4 wa = lds128q(qs), wc = lds128q(qs + 16);
  const U4 y0 = lds128q(xb + 64 * c), y1 = lds128q(xb + 64 * c + 16), y2 = lds128q(xb + 64 * c + 32), y3 = lds128q(xb + 64 * c + 48);
  U4 h0{0, 0, 0, 0}, h1{0, 0, 0, 0};
  if (Q5) {
    h0 = lds128q(wb + 16);
    h1 = lds128q(wb + 32);
  }
  int s_lo = 0, s_hi = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t w = i < 4 ? u4_get(wa, i) : u4_get(wc, i - 4);
    uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    if (Q5) {
      const uint32_t h = i < 4 ? u4_get(h0, i) : u4_get(h1, i - 4);
      lo |= ((h >> (2 * c)) & 0x01010101u) << 4;
      hi |= ((h >> (2 * c + 1)) & 0x01010101u) << 4;
    }
    s_lo = __dp4a((int)lo, (int)(i < 4 ? u4_get(y0, i) : u4_get(y1, i - 4)), s_lo);
    s_hi = __dp4a((int)hi, (int)(i < 4 ? u4_get(y2, i) : u4_get(y3, i - 4)), s_hi);
  }
  const uint32_t scw = c < 2 ? s.sc_lo : s.sc_hi, mw = c < 2 ? s.m_lo : s.m_hi;
  const int sh = (c & 1) * 16;
  const int sc0 = (scw >> sh) & 0xFF, sc1 = (scw >> (sh + 8)) & 0xFF;
  const int m0 = (mw >> sh) & 0xFF, m1 = (mw >> (sh + 8)) & 0xFF;
  // bsums[4c..4c+3]: pairs (4c,4c+1) for sub-block 2c and (4c+2,4c+3) for 2c+1
  const uint32_t bx = lds32q(xb + XK_BSUMS + 8 * c), by = lds32q(xb + XK_BSUMS + 8 * c + 4);
  int si = sc0 * s_lo + sc1 * s_hi;
  int sm = m0 * ((int)(short)(bx & 0xFFFF) + ((int)bx >> 16)) + m1 * ((int)(short)(by & 0xFFFF) + ((int)by >> 16));
  si += __shfl_xor_sync(0xffffffffu, si, 1);
  sm += __shfl_xor_sync(0xffffffffu, sm, 1);
  si += __shfl_xor_sync(0xffffffffu, si, 2);
  sm += __shfl_xor_sync(0xffffffffu, sm, 2);
  sumi = si;
  summ = sm;
}

// Q6_K: lane c covers half n = c/2 of the block and elements l in [16*(c%2), +16) of
// each of its four 32-element quarters. Blocks are only 2-byte aligned: words come from
// the aligned stream through a funnel shift.
__device__ __forceinline__ int quarter_q6k(uint32_t wb, uint32_t xb, int c) {
  const uint32_t sh = (wb & 2u) * 8u, p = wb & ~3u;
  auto wload = [&](int k) -> uint32_t { return funnel_r(lds32q(p + 4 * k), lds32q(p + 4 * k + 4), sh); };
  const int n = c >> 1, half = c & 1;
  const U4 y1 = lds128q(xb + 128 * n + 16 * half), y2 = lds128q(xb + 128 * n + 32 + 16 * half),
           y3 = lds128q(xb + 128 * n + 64 + 16 * half), y4 = lds128q(xb + 128 * n + 96 + 16 * half);
  int a1 = 0, a2 = 0, a3 = 0, a4 = 0;
#pragma unroll
  for (int ii = 0; ii < 4; ii++) {
    const int i = 4 * half + ii;
    const uint32_t l0 = wload(16 * n + i), l32 = wload(16 * n + 8 + i), h = wload(32 + 8 * n + i);
    const uint32_t q1 = (l0 & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
    const uint32_t q2 = (l32 & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
    const uint32_t q3 = ((l0 >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
    const uint32_t q4 = ((l32 >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
    a1 = __dp4a((int)q1, (int)u4_get(y1, ii), a1);
    a2 = __dp4a((int)q2, (int)u4_get(y2, ii), a2);
    a3 = __dp4a((int)q3, (int)u4_get(y3, ii), a3);
    a4 = __dp4a((int)q4, (int)u4_get(y4, ii), a4);
  }
  const uint32_t s01 = wload(48 + 2 * n), s23 = wload(49 + 2 * n);
  const int g = 8 * n + half;
  const int c1 = (int)(int8_t)((s01 >> (8 * half)) & 0xFF), c2 = (int)(int8_t)((s01 >> (8 * half + 16)) & 0xFF);
  const int c3 = (int)(int8_t)((s23 >> (8 * half)) & 0xFF), c4 = (int)(int8_t)((s23 >> (8 * half + 16)) & 0xFF);
  const uint32_t bsa = xb + XK_BSUMS + 2 * g;
  auto bs16 = [&](uint32_t a) -> int {
    int v;
    asm("ld.shared.s16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
  };
  int tot = c1 * a1 + c2 * a2 + c3 * a3 + c4 * a4;
  tot -= 32 * (c1 * bs16(bsa) + c2 * bs16(bsa + 4) + c3 * bs16(bsa + 8) + c4 * bs16(bsa + 12));
  tot += __shfl_xor_sync(0xffffffffu, tot, 1);
  tot += __shfl_xor_sync(0xffffffffu, tot, 2);
  return tot;
}

// Dot product of one K-quant row (in shared memory) with the Q8_K activation images,
// computed by one warp, four lanes per block; terms are added in block order. All lanes
// return the sum. `row` and `sx` are shared-space addresses.
__device__ __forceinline__ float warp_row_dot_s(int kind, uint32_t row, uint32_t sx, int nb) {
  const int lane = threadIdx.x & 31, bl = lane >> 2, c = lane & 3;
  const int bs = kind_size(kind);
  float sum = 0.0f;
  for (int g0 = 0; g0 < nb; g0 += 8) {
    const int b = g0 + bl;
    // Idle lanes recompute the last block so every lane reaches the shuffles.
    const int bb = b < nb ? b : nb - 1;
    const uint32_t wb = row + (uint32_t)bb * bs, xb = sx + (uint32_t)bb * XK_STRIDE;
    const float d_x = __uint_as_float(lds32q(xb + XK_D));
    float term;
    if (kind == Q6_K) {
      const int si = quarter_q6k(wb, xb, c);
      const uint32_t da = wb + 208;
      const uint32_t dw = lds32q(da & ~3u) >> ((da & 2u) * 8u);
      term = q6k_term(half_to_float_hw(dw & 0xFFFFu), d_x, si);
    } else {
      int si, sm;
      uint32_t dd;
      if (kind == Q5_K) quarter_k4<true>(wb, xb, c, si, sm, dd); else quarter_k4<false>(wb, xb, c, si, sm, dd);
      term = k4_term(half_to_float_hw(dd & 0xFFFFu), half_to_float_hw(dd >> 16), d_x, si, sm);
    }
    const int nbg = min(8, nb - g0);
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; j++) t[j] = __shfl_sync(0xffffffffu, term, 4 * j);
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (j < nbg) sum = fadd(sum, t[j]);
  }
  return sum;
}

// ---- lane-per-block dot products ---------------------------------------------------------
// One lane decodes one whole 256-weight super-block; the L = 2^k >= blocks-per-row lanes
// of a group cover one row, a warp covers 32/L rows at once. Fewer instructions per
// weight byte than the four-lane split above, which matters because these phases are
// bound by instruction issue, not by HBM.
__device__ __forceinline__ U4 lds128s(uint32_t a) {
  U4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32s(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

template <bool Q5>
__device__ __forceinline__ float block_term_k4(uint32_t wb, uint32_t xb) {
  const U4 hdr = lds128s(wb);
  const K4Scales s = k4_unpack(hdr.y, hdr.z, hdr.w);
  U4 h0{0, 0, 0, 0}, h1{0, 0, 0, 0};
  uint32_t qs = wb + 16;
  if (Q5) {
    h0 = lds128s(wb + 16);
    h1 = lds128s(wb + 32);
    qs = wb + 48;
  }
  int sumi = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const U4 wa = lds128s(qs + 32 * c), wc = lds128s(qs + 32 * c + 16);
    const U4 y0 = lds128s(xb + 64 * c), y1 = lds128s(xb + 64 * c + 16), y2 = lds128s(xb + 64 * c + 32),
             y3 = lds128s(xb + 64 * c + 48);
    int s_lo = 0, s_hi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t w = i < 4 ? u4_get(wa, i) : u4_get(wc, i - 4);
      uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
      if (Q5) {
        const uint32_t h = i < 4 ? u4_get(h0, i) : u4_get(h1, i - 4);
        lo |= ((h >> (2 * c)) & 0x01010101u) << 4;
        hi |= ((h >> (2 * c + 1)) & 0x01010101u) << 4;
      }
      s_lo = __dp4a((int)lo, (int)(i < 4 ? u4_get(y0, i) : u4_get(y1, i - 4)), s_lo);
      s_hi = __dp4a((int)hi, (int)(i < 4 ? u4_get(y2, i) : u4_get(y3, i - 4)), s_hi);
    }
    const uint32_t scw = c < 2 ? s.sc_lo : s.sc_hi;
    sumi += byte_of(scw, (2 * c) & 3) * s_lo + byte_of(scw, (2 * c + 1) & 3) * s_hi;
  }
  const U4 b0 = lds128s(xb + XK_BSUMS), b1 = lds128s(xb + XK_BSUMS + 16);
  const uint32_t m01 = __byte_perm(s.m_lo, 0, 0x1100), m23 = __byte_perm(s.m_lo, 0, 0x3322);
  const uint32_t m45 = __byte_perm(s.m_hi, 0, 0x1100), m67 = __byte_perm(s.m_hi, 0, 0x3322);
  int summ = 0;
  summ = dp2a_lo(b0.x, m01, summ);
  summ = dp2a_hi(b0.y, m01, summ);
  summ = dp2a_lo(b0.z, m23, summ);
  summ = dp2a_hi(b0.w, m23, summ);
  summ = dp2a_lo(b1.x, m45, summ);
  summ = dp2a_hi(b1.y, m45, summ);
  summ = dp2a_lo(b1.z, m67, summ);
  summ = dp2a_hi(b1.w, m67, summ);
  const float d_x = __uint_as_float(lds32s(xb + XK_D));
  return k4_term(half_to_float_hw(hdr.x & 0xFFFFu), half_to_float_hw(hdr.x >> 16), d_x, sumi, summ);
}

__device__ __forceinline__ float block_term_q6k(uint32_t wb, uint32_t xb) {
  // Blocks are 2-byte aligned: four consecutive words come from five aligned ones.
  const uint32_t sh = (wb & 2u) * 8u, p = wb & ~3u;
  auto load4 = [&](int k, uint32_t w[4]) {
    uint32_t a0 = lds32s(p + 4 * k), a1 = lds32s(p + 4 * k + 4), a2 = lds32s(p + 4 * k + 8), a3 = lds32s(p + 4 * k + 12),
             a4 = lds32s(p + 4 * k + 16);
    w[0] = funnel_r(a0, a1, sh);
    w[1] = funnel_r(a1, a2, sh);
    w[2] = funnel_r(a2, a3, sh);
    w[3] = funnel_r(a3, a4, sh);
  };
  uint32_t scw[4];
  load4(48, scw);
  int total = 0;
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      uint32_t l0[4], l32[4], h[4];
      load4(16 * n + 4 * half, l0);
      load4(16 * n + 8 + 4 * half, l32);
      load4(32 + 8 * n + 4 * half, h);
      const U4 y1 = lds128s(xb + 128 * n + 16 * half), y2 = lds128s(xb + 128 * n + 32 + 16 * half),
               y3 = lds128s(xb + 128 * n + 64 + 16 * half), y4 = lds128s(xb + 128 * n + 96 + 16 * half);
      int a1 = 0, a2 = 0, a3 = 0, a4 = 0;
#pragma unroll
      for (int ii = 0; ii < 4; ii++) {
        const uint32_t q1 = (l0[ii] & 0x0F0F0F0Fu) | ((h[ii] << 4) & 0x30303030u);
        const uint32_t q2 = (l32[ii] & 0x0F0F0F0Fu) | ((h[ii] << 2) & 0x30303030u);
        const uint32_t q3 = ((l0[ii] >> 4) & 0x0F0F0F0Fu) | (h[ii] & 0x30303030u);
        const uint32_t q4 = ((l32[ii] >> 4) & 0x0F0F0F0Fu) | ((h[ii] >> 2) & 0x30303030u);
        a1 = __dp4a((int)q1, (int)u4_get(y1, ii), a1);
        a2 = __dp4a((int)q2, (int)u4_get(y2, ii), a2);
        a3 = __dp4a((int)q3, (int)u4_get(y3, ii), a3);
        a4 = __dp4a((int)q4, (int)u4_get(y4, ii), a4);
      }
      const int g = 8 * n + half;
      total += (int)(int8_t)byte_of(scw[g >> 2], g & 3) * a1;
      total += (int)(int8_t)byte_of(scw[(g + 2) >> 2], (g + 2) & 3) * a2;
      total += (int)(int8_t)byte_of(scw[(g + 4) >> 2], (g + 4) & 3) * a3;
      total += (int)(int8_t)byte_of(scw[(g + 6) >> 2], (g + 6) & 3) * a4;
    }
  }
  const U4 b0 = lds128s(xb + XK_BSUMS), b1 = lds128s(xb + XK_BSUMS + 16);
  int bias = 0;
  bias = dp2a_lo(b0.x, scw[0], bias);
  bias = dp2a_hi(b0.y, scw[0], bias);
  bias = dp2a_lo(b0.z, scw[1], bias);
  bias = dp2a_hi(b0.w, scw[1], bias);
  bias = dp2a_lo(b1.x, scw[2], bias);
  bias = dp2a_hi(b1.y, scw[2], bias);
  bias = dp2a_lo(b1.z, scw[3], bias);
  bias = dp2a_hi(b1.w, scw[3], bias);
  const uint32_t da = wb + 208;
  const uint32_t dw = lds32s(da & ~3u) >> ((da & 2u) * 8u);
  const float d_x = __uint_as_float(lds32s(xb + XK_D));
  return q6k_term(half_to_float_hw(dw & 0xFFFFu), d_x, total - 32 * bias);
}

// Dot products of the rows a warp owns in one pass: lane = (group gi = lane / L, block
// slot bl = lane % L). `row` is this lane's row in shared memory (0 when the group has
// no row), `kind` its weight kind. Returns the row's sum to every lane of its group,
// block terms added in block order (matvec.rs:84-106).
__device__ __forceinline__ float group_row_dot(uint32_t row, int kind, uint32_t sx, int nb, int L) {
  const int lane = threadIdx.x & 31, bl = lane & (L - 1), gbase = lane & ~(L - 1);
  const int bs = kind_size(kind);
  float sum = 0.0f;
  for (int g0 = 0; g0 < nb; g0 += L) {
    const int b = g0 + bl;
    float term = 0.0f;
    if (row != 0 && b < nb) {
      const uint32_t wb = row + (uint32_t)b * bs, xb = sx + (uint32_t)b * XK_STRIDE;
      if (kind == Q4_K) term = block_term_k4<false>(wb, xb);
      else if (kind == Q6_K) term = block_term_q6k(wb, xb);
      else term = block_term_k4<true>(wb, xb);
    }
    __syncwarp();
    const int cnt = min(L, nb - g0);
    for (int j = 0; j < cnt; j++) sum = fadd(sum, __shfl_sync(0xffffffffu, term, gbase + j));
  }
  return sum;
}

// ---- tagged activation words ---------------------------------------------------------------
// Activation vectors that cross CTAs inside the step travel as 64-bit words {f32 value,
// 32-bit tag}. A writer stores value and tag with one 8-byte store; a reader polls the word
// until it carries the tag of the phase it expects. Data and "ready" arrive together, so
// no fence, counter or grid-wide barrier sits between a matrix product and its consumers.
// Tags are unique per (launch, phase): (launch count << 10) | phase id, phase id >= 1;
// a zeroed buffer therefore never matches.
typedef unsigned long long LLWord;
// Polls before a wait gives up (about a microsecond each). The host raises it when several
// GPUs step together: a rank whose host thread is late must not make its peers give up.
__constant__ uint32_t c_ll_spin_limit = 1u << 21;

__device__ __forceinline__ void ll_store(LLWord* p, float v, uint32_t tag) {
  const LLWord w = ((LLWord)tag << 32) | (LLWord)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ LLWord ll_load(const LLWord* p) {
  LLWord w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ void ll_load2(const LLWord* p, LLWord& a, LLWord& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// Value of a word whose tag may be ignored (this CTA wrote it in an earlier phase).
__device__ __forceinline__ float ll_value(const LLWord* p) { return __uint_as_float((uint32_t)ll_load(p)); }

// Spin (bounded) until the word carries `tag`. On expiry the CTA's abort flag and the
// device error word are set; every later wait then returns at once, so the kernel drains.
__device__ __forceinline__ float ll_settle(const LLWord* p, LLWord w, uint32_t tag, volatile int* abort, int* err) {
  if ((uint32_t)(w >> 32) != tag) {
    uint32_t it = 0;
    const uint32_t limit = c_ll_spin_limit;
    for (; it < limit; ++it) {
      w = ll_load(p);
      if ((uint32_t)(w >> 32) == tag) break;
      if ((it & 31u) == 31u && *abort) break;
    }
    if ((uint32_t)(w >> 32) != tag && !*abort) {
      *abort = 1;
      if (err) atomicOr(err, DEVERR_GRID_TIMEOUT);
    }
  }
  return __uint_as_float((uint32_t)w);
}
__device__ __forceinline__ float ll_wait(const LLWord* p, uint32_t tag, volatile int* abort, int* err) {
  return ll_settle(p, ll_load(p), tag, abort, err);
}

// Rows [c0, c1) of a row space of `span` rows that belong to this CTA: an even split with
// the remainder spread over the first CTAs, so every CTA owns a row when span >= gridDim.x.
__device__ __forceinline__ void cta_rows(int span, int& c0, int& c1) {
  const int base = span / (int)gridDim.x, rem = span - base * (int)gridDim.x, b = (int)blockIdx.x;
  c0 = b * base + min(b, rem);
  c1 = c0 + base + (b < rem ? 1 : 0);
}

// ---- tagged words across GPUs -----------------------------------------------------------------
// Row-sharded models (each GPU holds some heads and some FFN rows) produce partial rows of
// attn_output and ffn_down. A rank stores its partial of row i as a tagged word into slot
// [product][its rank][i] of every rank's inbox (plain 8-byte stores to peer memory over
// NVLink); the CTA that owns row i on each rank waits for the world's words, adds them in
// rank order (so every rank gets the same bits) and publishes the new residual row locally.
struct TpExchange {
  int world, rank, dim;
  LLWord* inbox[8];  // inbox of rank d (peer mapping), layout [2 products][world][dim]
};

__device__ __forceinline__ void ll_store_sys(LLWord* p, float v, uint32_t tag) {
  const LLWord w = ((LLWord)tag << 32) | (LLWord)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ float ll_wait_sys(const LLWord* p, uint32_t tag, volatile int* abort, int* err) {
  LLWord w;
  uint32_t it = 0;
  for (;;) {
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    if ((uint32_t)(w >> 32) == tag) break;
    if (++it >= c_ll_spin_limit || ((it & 31u) == 31u && *abort)) {
      if (!*abort) {
        *abort = 1;
        if (err) atomicOr(err, DEVERR_GRID_TIMEOUT);
      }
      break;
    }
  }
  return __uint_as_float((uint32_t)w);
}

// ---- step description (built once by the host, lives in global memory) ------------------
// One matrix-product phase as both the producer and the consumers see it. The row
// space (concatenated rows, or shared rows in pair mode) is split evenly over the
// grid; a CTA walks its share in tiles of `tile_rows` rows.
struct MegaOp {
  GemvSeg seg[3];
  uint32_t row_bytes[3];
  int nseg, pair, cols, span_rows, rows_per_cta, tile_rows, epilogue;
  int ll;  // outputs are tagged words (seg[].out points at LLWord), not plain floats
};

struct StepLayer {
  const float* attn_norm;
  const float* ffn_norm;
  const float* q_norm;
  const float* k_norm;
  MegaOp qkv, wo, gu, down;
};

struct StepParams {
  int dim, hidden, n_layer, n_head, n_kv_head, head_dim, rot_dim, vocab, n_ctx;
  float eps;
  int qk_norm, neox;
  const StepLayer* layers;
  const float* output_norm;
  const MegaOp* out_op;
  const uint8_t* token_embd;
  int embd_kind;
  size_t embd_row_bytes;
  LLWord *xl, *ql, *kl, *vl, *attl, *hbl;  // tagged activation vectors (residual, q, k, v, attention out, hidden)
  float *x;                                // plain copy of the final residual stream, for readers outside the kernel
  float *logits, *k_cache, *v_cache;
  unsigned* epoch;                         // launch count; bumped by CTA 0 when the kernel ends
  TpExchange tp;                           // world > 1: this GPU holds one shard of the model
  const float* rope_table;
  int* step;  // {token, pos, n_generated}
  int* history;
  int history_cap;
  int* out_token;
  int want_logits, with_argmax;
  unsigned* grid_bar;  // arrival counter, zero at launch
  int* err;
  int n_stages, stage_bytes;
  int scratch_bytes;   // f32 scratch region (norm rows, attention)
  int v_chunk;         // positions per staged V chunk
  int table_bytes;     // bytes of the StepLayer table staged in shared memory (n_layer + 1 entries)
  unsigned long long* prof;  // optional: cycles per phase, accumulated by one CTA
  int prof_cta;
};

// ---- shared-memory ring --------------------------------------------------------------------
struct Ring {
  uint8_t* stages;
  uint64_t* full;
  uint64_t* empty;
  int n_stages, stage_bytes;
  volatile int* abort;  // set when any bounded wait of this CTA expired
  int* err;
};

// Position of a producer or consumer in the ring: stage index and use parity.
struct RingPos {
  int st;
  uint32_t parity;
  __device__ __forceinline__ void advance(int n_stages) {
    if (++st == n_stages) {
      st = 0;
      parity ^= 1u;
    }
  }
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool ring_wait(const Ring& R, uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*R.abort) return false;
  }
  *R.abort = 1;
  if (R.err) atomicOr(R.err, DEVERR_MBAR_TIMEOUT);
  return false;
}

// Byte ranges of the tile covering rows [t0, t1) of the op's row space.
__device__ __forceinline__ int op_tile_parts(const MegaOp& op, int t0, int t1, TilePart parts[3]) {
  if (op.pair || op.nseg == 1) {
    const int np = op.pair ? 2 : 1;
    uint32_t soff = 0;
#pragma unroll
    for (int s = 0; s < 2; s++) {
      if (s < np) {
        TilePart& tp = parts[s];
        tp.seg = s;
        tp.row0 = t0;
        tp.rows = t1 - t0;
        tp.src = op.seg[s].w + (size_t)t0 * op.row_bytes[s];
        tp.len = (uint32_t)(t1 - t0) * op.row_bytes[s];
        tp.soff = soff;
        soff += bulk_superset_bytes(tp.src, tp.len) + 16;
      }
    }
    return np;
  }
  int n = 0, base = 0;
  uint32_t soff = 0;
  for (int s = 0; s < op.nseg; s++) {
    const int a = max(t0, base), b = min(t1, base + op.seg[s].rows);
    if (a < b) {
      TilePart& tp = parts[n++];
      tp.seg = s;
      tp.row0 = a - base;
      tp.rows = b - a;
      tp.src = op.seg[s].w + (size_t)(a - base) * op.row_bytes[s];
      tp.len = (uint32_t)(b - a) * op.row_bytes[s];
      tp.soff = soff;
      soff += bulk_superset_bytes(tp.src, tp.len) + 16;
    }
    base += op.seg[s].rows;
  }
  return n;
}

// Producer side (one thread): request every tile of this CTA's share of `op`.
__device__ __forceinline__ void produce_op(const MegaOp& op, const Ring& R, RingPos& pp) {
  int c0, c1;
  cta_rows(op.span_rows, c0, c1);
  for (int t0 = c0; t0 < c1; t0 += op.tile_rows) {
    if (!ring_wait(R, &R.empty[pp.st], pp.parity ^ 1u)) return;
    TilePart parts[3];
    const int t1 = min(t0 + op.tile_rows, c1);
    const int np = op_tile_parts(op, t0, t1, parts);
    uint32_t total = 0;
    for (int i = 0; i < np; i++) total += bulk_superset_bytes(parts[i].src, parts[i].len);
    mbar_expect_tx(&R.full[pp.st], total);
    for (int i = 0; i < np; i++)
      bulk_g2s_superset(R.stages + (size_t)pp.st * R.stage_bytes + parts[i].soff, parts[i].src, parts[i].len, &R.full[pp.st]);
    pp.advance(R.n_stages);
  }
}

// Consumer side (every consumer warp). A warp pass covers 32/L rows (L lanes per row);
// passes are dealt to warps round robin, continuing across tiles (`rot`), so that
// consecutive small tiles keep all warps busy at once. In pair mode the lower half of
// the warp takes gate rows and the upper half the matching up rows, and the SiLU gate
// is applied in the epilogue. `sx` holds the Q8_K images of the activation vector;
// `op` lives in shared memory.
template <bool TP = false>
__device__ __forceinline__ void consume_op(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, int warp,
                                           int n_warps, uint32_t tag, const TpExchange* tpx = nullptr, int which = 0) {
  const int rows_per_cta = op.rows_per_cta, tile_rows = op.tile_rows, pair = op.pair;
  const int epilogue = op.epilogue, nb = op.cols >> 8, ll = op.ll;
  int c0, c1;
  cta_rows(op.span_rows, c0, c1);
  const int lane = threadIdx.x & 31;
  // Small ops (a row or less per warp) use the short-latency four-lanes-per-block dot, one
  // row per warp; large ones the cheaper lane-per-block form.
  const bool narrow = rows_per_cta * (pair ? 2 : 1) <= n_warps;
  int L = 1;
  while (L < nb && L < 32) L <<= 1;
  if (narrow) L = 32;
  const int G = 32 / L;                             // rows per warp pass
  const bool split = pair && G >= 2;                // gate | up halves of one warp
  const int rows_per_pass = split ? G / 2 : G;
  const int gi = lane / L;
  const uint32_t sxa = smem_addr(sx);
  int rot = 0;
  for (int t0 = c0; t0 < c1; t0 += tile_rows) {
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    const int t1 = min(t0 + tile_rows, c1);
    const uint32_t stage = smem_addr(R.stages + (size_t)cp.st * R.stage_bytes);
    const int R_rows = t1 - t0;
    const int n_pass = (R_rows + rows_per_pass - 1) / rows_per_pass;
    int ps = warp - rot;
    if (ps < 0) ps += n_warps;
    if (ps < n_pass) {
      TilePart parts[3];
      const int np = op_tile_parts(op, t0, t1, parts);
      for (; ps < n_pass; ps += n_warps) {
        if (pair) {
          const uint32_t base0 = stage + parts[0].soff + ((uint32_t)(uintptr_t)parts[0].src & 15u);
          const uint32_t base1 = stage + parts[1].soff + ((uint32_t)(uintptr_t)parts[1].src & 15u);
          if (split) {
            const int which = gi >= rows_per_pass ? 1 : 0;
            const int u = ps * rows_per_pass + (gi - which * rows_per_pass);
            const uint32_t row = u < R_rows ? (which ? base1 : base0) + (uint32_t)u * op.row_bytes[which] : 0u;
            const float v = group_row_dot(row, op.seg[which].kind, sxa, nb, L);
            const float up = __shfl_down_sync(0xffffffffu, v, 16);
            if (u < R_rows && which == 0 && (lane & (L - 1)) == 0) {
              const int r = t0 + u;
              const float hv = epilogue == EPI_SILU_MUL ? silu_mul_exact(v, up) : v;
              if (ll) {
                ll_store(reinterpret_cast<LLWord*>(op.seg[0].out) + r, hv, tag);
              } else {
                op.seg[0].out[r] = hv;
                op.seg[1].out[r] = up;
              }
            }
          } else {
            const int u = ps;  // one row per pass: gate, then up
            float g, up;
            if (narrow) {
              g = warp_row_dot_s(op.seg[0].kind, base0 + (uint32_t)u * op.row_bytes[0], sxa, nb);
              up = warp_row_dot_s(op.seg[1].kind, base1 + (uint32_t)u * op.row_bytes[1], sxa, nb);
            } else {
              g = group_row_dot(base0 + (uint32_t)u * op.row_bytes[0], op.seg[0].kind, sxa, nb, L);
              up = group_row_dot(base1 + (uint32_t)u * op.row_bytes[1], op.seg[1].kind, sxa, nb, L);
            }
            if (lane == 0) {
              const int r = t0 + u;
              const float hv = epilogue == EPI_SILU_MUL ? silu_mul_exact(g, up) : g;
              if (ll) {
                ll_store(reinterpret_cast<LLWord*>(op.seg[0].out) + r, hv, tag);
              } else {
                op.seg[0].out[r] = hv;
                op.seg[1].out[r] = up;
              }
            }
          }
        } else {
          const int u = ps * G + gi;
          uint32_t row = 0;
          int kind = Q4_K, pi = 0, lr = u;
          if (u < R_rows) {
            while (pi < np - 1 && lr >= parts[pi].rows) {
              lr -= parts[pi].rows;
              pi++;
            }
            const TilePart& tp = parts[pi];
            row = stage + tp.soff + ((uint32_t)(uintptr_t)tp.src & 15u) + (uint32_t)lr * op.row_bytes[tp.seg];
            kind = op.seg[tp.seg].kind;
          }
          const float v = narrow ? (row ? warp_row_dot_s(kind, row, sxa, nb) : 0.0f) : group_row_dot(row, kind, sxa, nb, L);
          if (u < R_rows && (lane & (L - 1)) == 0) {
            const int oi = parts[pi].row0 + lr;
            if (TP && ll && tpx && epilogue == EPI_ACCUM) {
              // a partial row of a sharded product: hand it to every rank (this one included)
              for (int dst = 0; dst < tpx->world; dst++)
                ll_store_sys(tpx->inbox[dst] + ((size_t)which * tpx->world + tpx->rank) * tpx->dim + oi, v, tag);
            } else if (ll) {
              // a residual row is only ever written by its owner, so its old value needs no tag check
              LLWord* o = reinterpret_cast<LLWord*>(op.seg[parts[pi].seg].out) + oi;
              ll_store(o, epilogue == EPI_ACCUM ? fadd(ll_value(o), v) : v, tag);
            } else {
              float* o = op.seg[parts[pi].seg].out + oi;
              *o = epilogue == EPI_ACCUM ? fadd(__ldcg(o), v) : v;
            }
          }
        }
      }
    }
    rot = (rot + n_pass) % n_warps;
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
}

// ---- grid-wide barrier for the consumer warps ---------------------------------------------
// Arrival counter in global memory, zero at launch, never reset: barrier number k
// completes when it reaches k * gridDim.x. The spin is bounded; when it gives up the
// error word is set and every later barrier returns at once, so the kernel drains.
__device__ __forceinline__ bool grid_sync(const StepParams& P, const CtaGroup& g, unsigned& target, volatile int* abort) {
  g.sync();
  if (g.tid == 0) {
    target += gridDim.x;
    if (!*abort) {
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.grid_bar) : "memory");
      bool ok = false;
      for (uint32_t it = 0; it < (1u << 24); ++it) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.grid_bar) : "memory");
        if (v >= target) {
          ok = true;
          break;
        }
        if ((it & 1023u) == 1023u && *(volatile int*)P.err) break;
      }
      if (!ok) {
        *abort = 1;
        atomicOr(P.err, DEVERR_GRID_TIMEOUT);
      }
    }
  }
  g.sync();
  return !*abort;
}

// ---- activation phases -----------------------------------------------------------------------
struct MegaSmem {
  uint8_t* sx;          // Q8_K images of the current activation vector
  float* scr;           // f32 scratch
  SeqSumScratch* ss;
  float* red;           // 32 floats
  volatile int* abort;  // this CTA gave up on a bounded wait
  int* err;             // device error word
};

// x -> rmsnorm -> Q8_K images in shared memory (ops.rs:7-18 then quant.rs:248-283).
// `src` holds tagged words other CTAs publish under `tag`; for the embedding the row is
// already in scr[0..n). `mirror`, when given, receives a plain copy of the row.
__device__ __forceinline__ void phase_norm_quant(const LLWord* src, uint32_t tag, bool src_in_scr, float* mirror, const float* w,
                                                 int n, float eps, const MegaSmem& M, const CtaGroup& g,
                                                 SubProf sp = SubProf{nullptr, 0}) {
  sp.last = clock64();
  float* row = M.scr;
  float* sq = M.scr + n;
  // Scaling and quantization are one pass: warp b takes super-block b, lane l its elements
  // 8l..8l+7. The norm weights of the warp's first block are requested before the wait.
  const int warp = g.tid >> 5, nw = g.nthreads >> 5, lane = g.tid & 31, nblk = n >> 8;
  float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
  if (warp < nblk) {
    w0 = __ldg(reinterpret_cast<const float4*>(w + warp * 256 + 8 * lane));
    w1 = __ldg(reinterpret_cast<const float4*>(w + warp * 256 + 8 * lane) + 1);
  }
  if (src_in_scr) {
    for (int i = g.tid; i < n; i += g.nthreads) sq[i] = fmul(row[i], row[i]);
  } else {
    // all of a thread's words are requested before the first one is examined
    constexpr int U = 4;
    for (int base = g.tid; base < n; base += U * g.nthreads) {
      LLWord wd[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = base + u * g.nthreads;
        if (i < n) wd[u] = ll_load(src + i);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = base + u * g.nthreads;
        if (i < n) {
          const float v = ll_settle(src + i, wd[u], tag, M.abort, M.err);
          row[i] = v;
          sq[i] = fmul(v, v);
          if (mirror) mirror[i] = v;
        }
      }
    }
  }
  g.sync();
  sp.mark(16);
  float ss = group_seq_sum(sq, n, M.ss, g, &sp);
  sp.mark(17);
  float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)n), eps)));
  sp.mark(18);
  for (int b = warp; b < nblk; b += nw) {
    if (b != warp) {
      w0 = __ldg(reinterpret_cast<const float4*>(w + b * 256 + 8 * lane));
      w1 = __ldg(reinterpret_cast<const float4*>(w + b * 256 + 8 * lane) + 1);
    }
    const float4 x0 = *reinterpret_cast<const float4*>(row + b * 256 + 8 * lane);
    const float4 x1 = *(reinterpret_cast<const float4*>(row + b * 256 + 8 * lane) + 1);
    float v[8];
    v[0] = fmul(fmul(x0.x, r), w0.x); v[1] = fmul(fmul(x0.y, r), w0.y);
    v[2] = fmul(fmul(x0.z, r), w0.z); v[3] = fmul(fmul(x0.w, r), w0.w);
    v[4] = fmul(fmul(x1.x, r), w1.x); v[5] = fmul(fmul(x1.y, r), w1.y);
    v[6] = fmul(fmul(x1.z, r), w1.z); v[7] = fmul(fmul(x1.w, r), w1.w);
    warp_quantize_q8k_vals(v, M.sx + b * XK_STRIDE, 1);
  }
  g.sync();
  sp.mark(19);
}

// A vector other CTAs publish under `tag` -> Q8_K images.
__device__ __forceinline__ void phase_quant(const LLWord* src, uint32_t tag, int n, const MegaSmem& M, const CtaGroup& g) {
  const int warp = g.tid >> 5, nw = g.nthreads >> 5, lane = g.tid & 31;
  for (int b = warp; b < n / 256; b += nw) {
    const LLWord* p = src + b * 256 + 8 * lane;
    LLWord wd[8];
#pragma unroll
    for (int i = 0; i < 4; i++) ll_load2(p + 2 * i, wd[2 * i], wd[2 * i + 1]);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = ll_settle(p + i, wd[i], tag, M.abort, M.err);
    warp_quantize_q8k_vals(v, M.sx + b * XK_STRIDE, 1);
  }
  g.sync();
}

// Stage rows [c0, c0 + cn) of one KV head (row `pos` comes from `cur`, the row of the token
// being decoded, which is not in the cache yet) into `buf` with row stride `stride` floats.
// Cached rows travel with cp.async (no registers, completion by cp.async.wait_group), so
// the next chunk loads while the current one is consumed.
__device__ __forceinline__ void stage_kv_rows(float* buf, int stride, const float* cache, size_t kvd, int head_off, int hd4,
                                              int c0, int cn, int pos, const float* cur, int tid, int T) {
  for (int j = tid; j < cn * hd4; j += T) {
    const int t = j / hd4, i4 = j - t * hd4, tt = c0 + t;
    float* dst = buf + t * stride + 4 * i4;
    if (tt == pos) *reinterpret_cast<float4*>(dst) = reinterpret_cast<const float4*>(cur)[i4];
    else asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(cache + (size_t)tt * kvd + head_off + 4 * i4) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// Per-head q/k norm, RoPE, KV store and attention for head `h` (ops.rs:74-87, 40-70,
// 152-157, 185-218), by the consumer warps of one CTA.
__device__ void phase_attention(const StepParams& P, int li, int h, int pos, uint32_t tag_in, uint32_t tag_out,
                                const MegaSmem& M, const CtaGroup& g, SubProf pf = SubProf{nullptr, 0}) {
  pf.last = clock64();
  const int hd = P.head_dim, kvd = P.n_kv_head * hd, gqa = P.n_head / P.n_kv_head, kvh = h / gqa;
  const int n = pos + 1, tid = g.tid, T = g.nthreads;
  float* sq = M.scr;            // hd
  float* sk = sq + hd;          // hd
  float* sv = sk + hd;          // hd
  float* sp = sv + hd;          // hd (squares)
  float* sc = sp + hd;          // n_ctx scores
  float* vbuf = sc + ((P.n_ctx + 3) & ~3);  // two chunk buffers of v_chunk x (hd + 4) floats, 16-byte aligned
  const float* const q_norm_w = P.layers[li].q_norm;
  const float* const k_norm_w = P.layers[li].k_norm;
  float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd;
  float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd;
  // RoPE factors of this thread's pair, requested before the wait below
  const int rope_half = P.rot_dim / 2;
  float rope_c = 0.0f, rope_s = 0.0f;
  if (tid < 2 * rope_half) {
    const float* cs = P.rope_table + (size_t)pos * P.rot_dim;
    const int i = tid < rope_half ? tid : tid - rope_half;
    rope_c = cs[2 * i];
    rope_s = cs[2 * i + 1];
  }
  // this head's q and its group's k, v rows as the q/k/v products publish them
  for (int j = tid; j < 3 * hd; j += T) {
    const int which = j / hd, i = j - which * hd;
    const LLWord* src = which == 0 ? P.ql + h * hd + i : (which == 1 ? P.kl : P.vl) + kvh * hd + i;
    sq[j] = ll_wait(src, tag_in, M.abort, M.err);  // sq, sk, sv are consecutive
  }
  g.sync();
  if (P.qk_norm) {
    for (int which = 0; which < 2; which++) {
      float* v = which ? sk : sq;
      const float* nw = which ? k_norm_w : q_norm_w;
      for (int i = tid; i < hd; i += T) sp[i] = fmul(v[i], v[i]);
      float ss = group_seq_sum(sp, hd, M.ss, g);
      float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)hd), P.eps)));
      g.sync();
      for (int i = tid; i < hd; i += T) v[i] = fmul(fmul(v[i], r), nw[i]);
      g.sync();
    }
  }
  if (tid < 2 * rope_half) {  // rot_dim <= head_dim <= the group's thread count
    float* v = tid < rope_half ? sq : sk;
    const int i = tid < rope_half ? tid : tid - rope_half;
    const int i0 = P.neox ? i : 2 * i, i1 = P.neox ? i + rope_half : 2 * i + 1;
    const float x0 = v[i0], x1 = v[i1];
    v[i0] = fsub(fmul(x0, rope_c), fmul(x1, rope_s));
    v[i1] = fadd(fmul(x0, rope_s), fmul(x1, rope_c));
  }
  g.sync();
  if (h % gqa == 0) {
    for (int i = tid; i < hd; i += T) {
      kc[(size_t)pos * kvd + kvh * hd + i] = sk[i];
      vc[(size_t)pos * kvd + kvh * hd + i] = sv[i];
    }
  }
  pf.mark(20);
  // scores: cached K rows are staged through shared memory in chunks, double buffered; rows
  // are padded by one float4 to spread the banks
  const float scale = 1.0f / sqrtf((float)hd);
  const int hd4 = hd >> 2, kstride = hd + 4, chunk = P.v_chunk;
  const int buf_floats = chunk * kstride;
  float lmax = -INFINITY;
  stage_kv_rows(vbuf, kstride, kc, kvd, kvh * hd, hd4, 0, min(chunk, n), pos, sk, tid, T);
  for (int c0 = 0, ci = 0; c0 < n; c0 += chunk, ci++) {
    const int cn = min(chunk, n - c0);
    float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + chunk < n) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, kstride, kc, kvd, kvh * hd, hd4, c0 + chunk, min(chunk, n - c0 - chunk), pos, sk,
                    tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    for (int t = tid; t < cn; t += T) {
      const float4* kt = reinterpret_cast<const float4*>(cur_buf + t * kstride);
      const float4* qt = reinterpret_cast<const float4*>(sq);
      float s = 0.0f;
      for (int i0 = 0; i0 < hd4; i0 += 4) {
        // products first (independent), then the chain of adds in element order
        float pr[16];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const float4 kk = kt[i0 + u], qq = qt[i0 + u];
          pr[4 * u] = fmul(qq.x, kk.x);
          pr[4 * u + 1] = fmul(qq.y, kk.y);
          pr[4 * u + 2] = fmul(qq.z, kk.z);
          pr[4 * u + 3] = fmul(qq.w, kk.w);
        }
#pragma unroll
        for (int u = 0; u < 16; u++) s = fadd(s, pr[u]);
      }
      s = fmul(s, scale);
      sc[c0 + t] = s;
      lmax = fmaxf(lmax, s);
    }
    g.sync();  // this buffer is refilled two chunks later
  }
  // the first chunk of V rows loads while the softmax runs
  stage_kv_rows(vbuf, hd, vc, kvd, kvh * hd, hd4, 0, min(chunk, n), pos, sv, tid, T);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
  if ((tid & 31) == 0) M.red[tid >> 5] = lmax;
  g.sync();
  pf.mark(21);
  float mx = M.red[0];
  for (int w = 1; w < (T >> 5); w++) mx = fmaxf(mx, M.red[w]);
  for (int t = tid; t < n; t += T) sc[t] = expf_exact(fsub(sc[t], mx));
  g.sync();
  pf.mark(22);
  float sum = group_seq_sum(sc, n, M.ss, g);
  pf.mark(23);
  float inv = fdiv(1.0f, sum);
  g.sync();
  for (int t = tid; t < n; t += T) sc[t] = fmul(sc[t], inv);
  // value mix, positions in order (ops.rs:208-214); cached rows staged as above
  float o = 0.0f;
  for (int c0 = 0, ci = 0; c0 < n; c0 += chunk, ci++) {
    const int cn = min(chunk, n - c0);
    const float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + chunk < n) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, hd, vc, kvd, kvh * hd, hd4, c0 + chunk, min(chunk, n - c0 - chunk), pos, sv, tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    if (tid < hd) {
      int t = 0;
      for (; t + 8 <= cn; t += 8) {
        float pr[8];
#pragma unroll
        for (int u = 0; u < 8; u++) pr[u] = fmul(sc[c0 + t + u], cur_buf[(t + u) * hd + tid]);
#pragma unroll
        for (int u = 0; u < 8; u++) o = fadd(o, pr[u]);
      }
      for (; t < cn; t++) o = fadd(o, fmul(sc[c0 + t], cur_buf[t * hd + tid]));
    }
    g.sync();
  }
  if (tid < hd) ll_store(P.attl + h * hd + tid, o, tag_out);
  pf.mark(24);
}

// Greedy argmax of the logits (sampler.rs:99-109) and the cursor update, CTA 0 only.
__device__ void phase_argmax(const StepParams& P, const MegaSmem& M, const CtaGroup& g) {
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = g.tid; i < P.vocab; i += g.nthreads) {
    float v = __ldcg(P.logits + i);
    if (v > best) {
      best = v;
      idx = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float v2 = __shfl_xor_sync(0xffffffffu, best, o);
    int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
    if (v2 > best || (v2 == best && i2 < idx)) {
      best = v2;
      idx = i2;
    }
  }
  int* redi = reinterpret_cast<int*>(M.red + 32);
  if ((g.tid & 31) == 0) {
    M.red[g.tid >> 5] = best;
    redi[g.tid >> 5] = idx;
  }
  g.sync();
  if (g.tid == 0) {
    for (int w = 1; w < (g.nthreads >> 5); w++) {
      if (M.red[w] > best || (M.red[w] == best && redi[w] < idx)) {
        best = M.red[w];
        idx = redi[w];
      }
    }
    if (idx == 0x7fffffff) idx = 0;
    if (P.out_token) *P.out_token = idx;
    int gcount = P.step[2];
    if (P.history && gcount < P.history_cap) P.history[gcount] = idx;
    P.step[0] = idx;
    P.step[1] = P.step[1] + 1;
    P.step[2] = gcount + 1;
  }
}

// ---- the kernel ---------------------------------------------------------------------------------
#ifndef MEGA_THREADS_N
#define MEGA_THREADS_N 768
#endif
constexpr int MEGA_THREADS = MEGA_THREADS_N;
constexpr int MEGA_CONSUMER_WARPS = MEGA_THREADS / 32 - 1;
constexpr int MEGA_BAR_BYTES = 128;     // up to 8 stages x (full, empty)
constexpr int MEGA_SEQSUM_BYTES = 2064;  // sizeof(SeqSumScratch) rounded up to 16
static_assert(sizeof(SeqSumScratch) <= MEGA_SEQSUM_BYTES, "SeqSumScratch layout");
// Bytes of shared memory besides the ring stages, the activation images and the scratch.
constexpr int MEGA_TAIL_BYTES = MEGA_BAR_BYTES + MEGA_SEQSUM_BYTES + 64 * 4 + 16;

// TP: this GPU holds one shard of a row-sharded model and exchanges partial rows with its peers.
template <bool TP>
__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_step_kernel(const StepParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][sx images][scratch][barriers 128 B][SeqSumScratch][red 64 floats][abort]
  const int nb_max = (max(max(P.dim, P.hidden), P.n_head * P.head_dim)) / 256;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  uint8_t* cur = sx + (size_t)nb_max * XK_STRIDE;  // 16-byte aligned: 304 = 19 * 16
  float* scr = reinterpret_cast<float*>(cur);
  cur += P.scratch_bytes;                          // a multiple of 128
  uint64_t* bars = reinterpret_cast<uint64_t*>(cur);
  cur += MEGA_BAR_BYTES;
  SeqSumScratch* ssc = reinterpret_cast<SeqSumScratch*>(cur);
  cur += MEGA_SEQSUM_BYTES;
  float* red = reinterpret_cast<float*>(cur);
  cur += 64 * sizeof(float);
  volatile int* abort = reinterpret_cast<volatile int*>(cur);
  cur += 16;
  // The step's tensor table (one StepLayer per layer + the output head), copied from
  // global memory once so that no phase waits on a descriptor load.
  StepLayer* const table = reinterpret_cast<StepLayer*>(cur);
  {
    const uint4* src = reinterpret_cast<const uint4*>(P.layers);
    uint4* dst = reinterpret_cast<uint4*>(table);
    for (int i = threadIdx.x; i < P.table_bytes / 16; i += blockDim.x) dst[i] = src[i];
  }

  Ring R;
  R.stages = stages;
  R.full = bars;
  R.empty = bars + P.n_stages;
  R.n_stages = P.n_stages;
  R.stage_bytes = P.stage_bytes;
  R.abort = abort;
  R.err = P.err;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) {
      mbar_init(&R.full[s], 1);
      mbar_init(&R.empty[s], MEGA_CONSUMER_WARPS);
    }
    *abort = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5;
  const int qd = P.n_head * P.head_dim;

  if (warp == MEGA_CONSUMER_WARPS) {
    // ---- producer warp: one thread walks every matrix product of the step ----
    if ((threadIdx.x & 31) == 0) {
      RingPos pp{0, 0u};
      for (int li = 0; li < P.n_layer && !*abort; li++) {
        const StepLayer& L = table[li];
        produce_op(L.qkv, R, pp);
        produce_op(L.wo, R, pp);
        produce_op(L.gu, R, pp);
        produce_op(L.down, R, pp);
      }
      if (P.want_logits && !*abort) produce_op(table[P.n_layer].qkv, R, pp);
    }
    return;
  }

  // ---- consumer warps ----
  CtaGroup g{(int)threadIdx.x, MEGA_CONSUMER_WARPS * 32, 1};
  MegaSmem M{sx, scr, ssc, red, abort, P.err};
  RingPos cp{0, 0u};
  unsigned bar_target = 0;
  const int token = P.step[0], pos = P.step[1];
  // Tags of this launch: phase k (1..5) of layer li is tag_base + 5 * li + k.
  const uint32_t tag_base = *P.epoch << 10;
  const bool prof_on = P.prof && (int)blockIdx.x == P.prof_cta && g.tid == 0;
  long long prof_last = clock64();
#define MEGA_PROF(slot)                                 \
  do {                                                  \
    if (prof_on) {                                      \
      long long now_ = clock64();                       \
      atomicAdd(&P.prof[slot], (unsigned long long)(now_ - prof_last)); \
      prof_last = now_;                                 \
    }                                                   \
  } while (0)

  // embedding row (quant.rs:300-443 via emit.rs:469): every CTA keeps a copy and publishes
  // the residual rows it owns (the rows of wo / down it computes)
  {
    const uint8_t* row = P.token_embd + (size_t)token * P.embd_row_bytes;
    int r0, r1;
    cta_rows(P.dim, r0, r1);
    for (int e = g.tid; e < P.dim; e += g.nthreads) {
      float v = dequant_elem(P.embd_kind, row, (size_t)e);
      scr[e] = v;
      if (e >= r0 && e < r1) ll_store(P.xl + e, v, 0u);
    }
    g.sync();
  }
  MEGA_PROF(0);

  // One loop over the step's matrix products (four per layer, then the output head), so
  // that each phase's code exists once. Phases hand their vectors on as tagged words;
  // the only grid-wide barrier left is the one in front of the argmax.
  const int n_stage = 4 * P.n_layer + (P.want_logits ? 1 : 0);
#pragma unroll 1
  for (int st = 0; st < n_stage; st++) {
    const int li = st >> 2, ph = st & 3;
    const bool head = li == P.n_layer;
    const StepLayer& L = table[li];
    const MegaOp& op = (&L.qkv)[ph];  // qkv, wo, gu, down are consecutive members
    const int slot = ph == 0 ? 1 : 3 * ph + 3;
    const uint32_t tl = tag_base + 5u * (uint32_t)li;  // + k: phase k of this layer
    if (ph == 0 && !head) {
      // The cached K and V rows this CTA's heads will read were evicted from L2 by the weight
      // stream; ask for them now, two phases ahead of their use.
      for (int h = blockIdx.x; h < P.n_head; h += gridDim.x) {
        const int kvd = P.n_kv_head * P.head_dim, kvh = h / (P.n_head / P.n_kv_head);
        const int lines = (P.head_dim * 4 + 127) / 128;  // 128-byte lines per cached row of one head
        const float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd + kvh * P.head_dim;
        const float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd + kvh * P.head_dim;
        for (int j = g.tid; j < pos * lines; j += g.nthreads) {
          const int t = j / lines, ln = j - t * lines;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + (size_t)t * kvd + 32 * ln));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + (size_t)t * kvd + 32 * ln));
        }
      }
    }
    if ((ph & 1) == 0) {
      // attention norm -> q/k/v, ffn norm -> gate/up + SiLU, output norm -> logits
      const float* w = head ? P.output_norm : (ph == 0 ? L.attn_norm : L.ffn_norm);
      const uint32_t tin = ph == 0 ? tl : tl + 3u;  // residual after the previous layer's down / this layer's wo
      phase_norm_quant(P.xl, tin, st == 0, head && blockIdx.x == 0 ? P.x : nullptr, w, P.dim, P.eps, M, g,
                       SubProf{prof_on && ph == 0 && !head ? P.prof : nullptr, 0});
    } else {
      // attention output -> wo, activated hidden -> down; both join the residual stream
      if (ph == 1) phase_quant(P.attl, tl + 2u, qd, M, g);
      else phase_quant(P.hbl, tl + 4u, P.hidden, M, g);
    }
    if (!head) MEGA_PROF(slot);
    // q/k/v: tl+1, wo: tl+3, gate/up: tl+4, down: tl+5 (the head writes plain floats)
    const uint32_t tag_out = tl + (ph == 0 ? 1u : (uint32_t)ph + 2u);
    const bool exchange = TP && (ph & 1) && !head;
    consume_op<TP>(op, R, cp, sx, warp, MEGA_CONSUMER_WARPS, tag_out, exchange ? &P.tp : nullptr, ph >> 1);
    if (head) break;
    // The next phase rewrites the activation images and the scratch rows; warps that are
    // done must also not start polling while others still compute.
    g.sync();
    if (TP && exchange) {
      // The rows this CTA owns: wait for every rank's partial, add them in rank order, join
      // the residual stream and publish the row for this GPU's CTAs.
      int r0, r1;
      cta_rows(P.dim, r0, r1);
      for (int i = r0 + g.tid; i < r1; i += g.nthreads) {
        const LLWord* in = P.tp.inbox[P.tp.rank] + (size_t)(ph >> 1) * P.tp.world * P.dim + i;
        float sum = ll_wait_sys(in, tag_out, abort, P.err);
        for (int src = 1; src < P.tp.world; src++) sum = fadd(sum, ll_wait_sys(in + (size_t)src * P.dim, tag_out, abort, P.err));
        ll_store(P.xl + i, fadd(ll_value(P.xl + i), sum), tag_out);
      }
    }
    MEGA_PROF(slot + 1);
    if (ph == 0) {
      // attention, one head per CTA
      for (int h = blockIdx.x; h < P.n_head; h += gridDim.x) {
        phase_attention(P, li, h, pos, tl + 1u, tl + 2u, M, g, SubProf{prof_on ? P.prof : nullptr, 0});
        g.sync();
      }
      MEGA_PROF(4);
    }
  }
  if (!P.want_logits && blockIdx.x == 0) {
    // no output head: still leave a plain copy of the final residual stream
    const uint32_t tin = tag_base + 5u * (uint32_t)P.n_layer;
    for (int i = g.tid; i < P.dim; i += g.nthreads) P.x[i] = ll_wait(P.xl + i, tin, abort, P.err);
  }
  if (P.want_logits && P.with_argmax) {
    const bool ok = grid_sync(P, g, bar_target, abort);  // uniform across the CTA
    if (blockIdx.x == 0 && ok) phase_argmax(P, M, g);
  }
  // Next launch, next tags. Every CTA read the count before it published anything, and
  // CTA 0 gets here only after consuming words from every CTA.
  if (blockIdx.x == 0 && g.tid == 0) *P.epoch = *P.epoch + 1u;
  MEGA_PROF(15);
#undef MEGA_PROF
}

// ---- Q4_0 / Q5_0 / Q8_0 rows from the ring --------------------------------------------------
// The reference's AVX2 kernels keep eight f32 lane accumulators per row; lane k adds
// fma(d_w*d_x, float(p_k), acc_k) per 32-weight block, in block order, and the row ends
// with a fixed 8-lane tree (simd_avx2.rs:29-34, 61-72). Here eight threads own the eight
// lane chains of a row (four rows per warp pass).
__device__ __forceinline__ uint32_t lds32_a2s(uint32_t a) {  // 32-bit word at a 2-byte aligned shared address
  uint32_t lo, hi;
  asm("ld.shared.u16 %0, [%1];" : "=r"(lo) : "r"(a));
  asm("ld.shared.u16 %0, [%1];" : "=r"(hi) : "r"(a + 2));
  return lo | (hi << 16);
}

template <int KIND>
__device__ __forceinline__ float row_chain_q80(uint32_t row, uint32_t sx, int nb, int k) {
  constexpr int BS = KIND == Q4_0 ? 18 : (KIND == Q5_0 ? 22 : 34);
  float acc = 0.0f;
#pragma unroll 4
  for (int b = 0; b < nb; b++) {
    const uint32_t wb = row + (uint32_t)b * BS, xb = sx + (uint32_t)b * X0_STRIDE;
    uint32_t hd;
    asm("ld.shared.u16 %0, [%1];" : "=r"(hd) : "r"(wb));
    const float d = fmul(half_to_float_hw(hd), __uint_as_float(lds32q(xb + X0_D)));
    const uint32_t y = lds32q(xb + 4 * k);
    int p;
    if (KIND == Q8_0) p = q8_0_lane(lds32_a2s(wb + 2 + 4 * k), y);
    else if (KIND == Q4_0) p = q4_0_lane(lds32_a2s(wb + 2 + 4 * (k & 3)), k, y);
    else p = q5_0_lane(lds32_a2s(wb + 6 + 4 * (k & 3)), lds32_a2s(wb + 2), k, y);
    acc = ffma(d, i2f(p), acc);
  }
  return acc;
}

// Consumer side for matrices of the Q8_0 family; `sx` holds the 48-byte Q8_0 images.
// `m` activation rows (their images back to back in `sx`) are applied to every resident row;
// output element (token, row) goes to out[token * rows + row].
__device__ __forceinline__ void consume_op_q80(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, int warp,
                                               int n_warps, int m) {
  const int tile_rows = op.tile_rows, pair = op.pair, epilogue = op.epilogue, nb = op.cols >> 5;
  int c0, c1;
  cta_rows(op.span_rows, c0, c1);
  const int lane = threadIdx.x & 31, k = lane & 7, gi = lane >> 3;
  const uint32_t sxa = smem_addr(sx);
  int rot = 0;
  for (int t0 = c0; t0 < c1; t0 += tile_rows) {
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    const int t1 = min(t0 + tile_rows, c1);
    const uint32_t stage = smem_addr(R.stages + (size_t)cp.st * R.stage_bytes);
    const int R_rows = t1 - t0;
    const int n_pass = (R_rows + 3) / 4;  // four rows per warp pass
    int ps = warp - rot;
    if (ps < 0) ps += n_warps;
    if (ps < n_pass) {
      TilePart parts[3];
      const int np = op_tile_parts(op, t0, t1, parts);
      for (; ps < n_pass; ps += n_warps) {
        const int u = ps * 4 + gi;
        float v[2] = {0.0f, 0.0f};
        int pi = 0, lr = u;
        if (!pair && u < R_rows) {
          while (pi < np - 1 && lr >= parts[pi].rows) {
            lr -= parts[pi].rows;
            pi++;
          }
        }
        const int n_mat = pair ? 2 : 1;
        for (int tok = 0; tok < m; tok++) {
          const uint32_t sxt = sxa + (uint32_t)tok * (uint32_t)nb * X0_STRIDE;
          for (int mt = 0; mt < n_mat; mt++) {
            const TilePart& tp = parts[pair ? mt : pi];
            const int kind = op.seg[tp.seg].kind;
            const uint32_t row = stage + tp.soff + ((uint32_t)(uintptr_t)tp.src & 15u) + (uint32_t)(pair ? u : lr) * op.row_bytes[tp.seg];
            float a = 0.0f;
            if (u < R_rows) {
              if (kind == Q4_0) a = row_chain_q80<Q4_0>(row, sxt, nb, k);
              else if (kind == Q5_0) a = row_chain_q80<Q5_0>(row, sxt, nb, k);
              else a = row_chain_q80<Q8_0>(row, sxt, nb, k);
            }
            // ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)) over the row's eight lanes
            a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 4));
            a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 2));
            a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 1));
            v[mt] = a;
          }
          if (u < R_rows && k == 0) {
            if (pair) {
              const size_t r = (size_t)tok * op.seg[0].rows + t0 + u;
              op.seg[0].out[r] = epilogue == EPI_SILU_MUL ? silu_mul_exact(v[0], v[1]) : v[0];
              op.seg[1].out[r] = v[1];
            } else {
              float* o = op.seg[parts[pi].seg].out + (size_t)tok * op.seg[parts[pi].seg].rows + parts[pi].row0 + lr;
              *o = epilogue == EPI_ACCUM ? fadd(__ldcg(o), v[0]) : v[0];
            }
          }
        }
      }
    }
    rot = (rot + n_pass) % n_warps;
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
}

// ---- one matrix product with the same machinery ------------------------------------------
// A single K-quant product (up to three matrices, or a gate/up pair) against one Q8_K
// activation vector: the producer warp streams this CTA's rows through the ring while the
// consumer warps take whole rows, with no CTA-wide barrier per tile. Used for single-row
// products outside the one-kernel step (the operator API, models the step does not cover).
struct StreamGemvParams {
  MegaOp op;
  const void* x;  // activation images (x_image) or reference-layout blocks
  int x_image;
  int q80;        // matrices of the Q8_0 family (Q8_0 activations) instead of K-quants
  int m;          // activation rows (more than one only for the Q8_0 family)
  int n_stages, stage_bytes;
  int* err;
};

__global__ void __launch_bounds__(MEGA_THREADS, 1) gemv_stream_kernel(const StreamGemvParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][sx images][barriers 128 B][abort]
  const int nb = P.q80 ? P.op.cols >> 5 : P.op.cols >> 8;
  const int xstride = P.q80 ? X0_STRIDE : XK_STRIDE;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sx + (size_t)P.m * nb * xstride);
  volatile int* abort = reinterpret_cast<volatile int*>(bars + MEGA_BAR_BYTES / 8);
  Ring R;
  R.stages = stages;
  R.full = bars;
  R.empty = bars + P.n_stages;
  R.n_stages = P.n_stages;
  R.stage_bytes = P.stage_bytes;
  R.abort = abort;
  R.err = P.err;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) {
      mbar_init(&R.full[s], 1);
      mbar_init(&R.empty[s], MEGA_CONSUMER_WARPS);
    }
    *abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  if (warp == MEGA_CONSUMER_WARPS) {
    // weights do not depend on the previous kernel: stream them right away
    if ((threadIdx.x & 31) == 0) {
      RingPos pp{0, 0u};
      produce_op(P.op, R, pp);
    }
    return;
  }
  pdl_wait();
  CtaGroup g{(int)threadIdx.x, MEGA_CONSUMER_WARPS * 32, 1};
  const int nbm = nb * P.m;  // blocks of all activation rows, back to back
  if (P.x_image) {
    const uint4* src4 = reinterpret_cast<const uint4*>(P.x);
    for (int i = g.tid; i < nbm * (xstride / 16); i += g.nthreads) reinterpret_cast<uint4*>(sx)[i] = src4[i];
  } else if (P.q80) {
    // BlockQ8_0 {f32 d; i8 qs[32]} (quant.rs:16-20) -> image {qs; d}
    const uint32_t* src = reinterpret_cast<const uint32_t*>(P.x);
    for (int i = g.tid; i < nbm * 9; i += g.nthreads) {
      const int b = i / 9, w = i - b * 9;
      *reinterpret_cast<uint32_t*>(sx + b * X0_STRIDE + (w == 0 ? X0_D : (w - 1) * 4)) = src[i];
    }
  } else {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(P.x);
    for (int i = g.tid; i < nb * 73; i += g.nthreads) {
      const int b = i / 73, w = i - b * 73;
      const int off = w == 0 ? XK_D : (w <= 64 ? (w - 1) * 4 : XK_BSUMS + (w - 65) * 4);
      *reinterpret_cast<uint32_t*>(sx + b * XK_STRIDE + off) = src[i];
    }
  }
  g.sync();
  RingPos cp{0, 0u};
  if (P.q80) consume_op_q80(P.op, R, cp, sx, warp, MEGA_CONSUMER_WARPS, P.m);
  else consume_op(P.op, R, cp, sx, warp, MEGA_CONSUMER_WARPS, 0u);
}


}  // namespace aot
