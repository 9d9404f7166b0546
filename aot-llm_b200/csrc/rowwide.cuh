// K-quant row products for launches with many rows per CTA: one lane per 256-weight
// super-block, 32 / L rows per warp pass (matvec.rs:82-167).
//
// rowdot.cuh spreads a super-block over four lanes, which is the quick way through a
// handful of rows (the one-kernel decode step). A launch that hands every CTA hundreds of
// rows is a throughput problem instead: here a lane forms a whole block term on its own
// (no cross-lane traffic until the row's terms are added), a group of L lanes covers a
// row's blocks, and the groups of a warp work on different rows. Block terms are added in
// block order through shuffles, so the sums are the reference's, bit for bit.
#pragma once
#include "rowdot.cuh"

namespace aot {

template <bool Q5>
__device__ __forceinline__ float wide_term_k4(uint32_t wb, uint32_t xb) {
  const U4 hdr = rd_lds128(wb);
  const K4Scales s = k4_unpack(hdr.y, hdr.z, hdr.w);
  U4 h0{0, 0, 0, 0}, h1{0, 0, 0, 0};
  uint32_t qs = wb + 16;
  if (Q5) {
    h0 = rd_lds128(wb + 16);
    h1 = rd_lds128(wb + 32);
    qs = wb + 48;
  }
  int sumi = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const U4 wa = rd_lds128(qs + 32 * c), wc = rd_lds128(qs + 32 * c + 16);
    const U4 y0 = rd_lds128(xb + 64 * c), y1 = rd_lds128(xb + 64 * c + 16), y2 = rd_lds128(xb + 64 * c + 32),
             y3 = rd_lds128(xb + 64 * c + 48);
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
  // matvec.rs:89-103: summ = sum_j m_j * (bsums[2j] + bsums[2j+1])
  const U4 b0 = rd_lds128(xb + XK_BSUMS), b1 = rd_lds128(xb + XK_BSUMS + 16);
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
  const float d_x = __uint_as_float(rd_lds32(xb + XK_D));
  return k4_term(half_bits_hw(hdr.x & 0xFFFFu), half_bits_hw(hdr.x >> 16), d_x, sumi, summ);
}

__device__ __forceinline__ float wide_term_q6k(uint32_t wb, uint32_t xb) {
  // Blocks are 2-byte aligned: four consecutive words come from five aligned ones.
  const uint32_t sh = (wb & 2u) * 8u, p = wb & ~3u;
  auto load4 = [&](int k, uint32_t w[4]) {
    const uint32_t a0 = rd_lds32(p + 4 * k), a1 = rd_lds32(p + 4 * k + 4), a2 = rd_lds32(p + 4 * k + 8), a3 = rd_lds32(p + 4 * k + 12),
                   a4 = rd_lds32(p + 4 * k + 16);
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
      const U4 y1 = rd_lds128(xb + 128 * n + 16 * half), y2 = rd_lds128(xb + 128 * n + 32 + 16 * half),
               y3 = rd_lds128(xb + 128 * n + 64 + 16 * half), y4 = rd_lds128(xb + 128 * n + 96 + 16 * half);
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
  // the weights are stored with an offset of 32: subtract 32 * sum_g sc_g * bsum_g (matvec.rs:150-160)
  const U4 b0 = rd_lds128(xb + XK_BSUMS), b1 = rd_lds128(xb + XK_BSUMS + 16);
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
  const uint32_t dw = rd_lds32(da & ~3u) >> ((da & 2u) * 8u);
  const float d_x = __uint_as_float(rd_lds32(xb + XK_D));
  return q6k_term(half_bits_hw(dw & 0xFFFFu), d_x, total - 32 * bias);
}

// Dot product of the row this lane's group owns: lane = (group lane / L, block slot
// lane % L). `row` is the row's shared address (0: the group has no row), `kind` its weight
// kind. Returns the row's sum to every lane of the group, block terms added in block order
// (matvec.rs:84-106).
__device__ __forceinline__ float wide_row_dot(uint32_t row, int kind, uint32_t sxa, int nb, int L) {
  const int lane = threadIdx.x & 31, bl = lane & (L - 1), gbase = lane & ~(L - 1);
  const int bs = kind_size(kind);
  float sum = 0.0f;
#pragma unroll 1
  for (int g0 = 0; g0 < nb; g0 += L) {
    const int b = g0 + bl;
    float term = 0.0f;
    if (row != 0 && b < nb) {
      const uint32_t wb = row + (uint32_t)b * bs, xb = sxa + (uint32_t)b * XK_STRIDE;
      if (kind == Q4_K) term = wide_term_k4<false>(wb, xb);
      else if (kind == Q6_K) term = wide_term_q6k(wb, xb);
      else term = wide_term_k4<true>(wb, xb);
    }
    __syncwarp();
    const int cnt = min(L, nb - g0);
    for (int j = 0; j < cnt; j++) sum = fadd(sum, __shfl_sync(0xffffffffu, term, gbase + j));
  }
  return sum;
}

}  // namespace aot
