// K-quant row products for weights that sit in shared memory, one warp per row,
// four lanes per 256-weight super-block (matvec.rs:82-167).
//
// A lane (block slot bl = lane / 4, quarter c = lane % 4) keeps its slice of the Q8_K
// activation block in registers, so a warp that walks many rows of the same matrix reads
// each weight byte once from shared memory and the activations not at all. Integer sums
// are exact in any order; the f32 term of a block, (d_w*d_x)*sumi - (dmin_w*d_x)*summ, is
// formed by the block's first lane and parked in a per-warp strip of shared memory. When
// the strip is full (or the product ends) the warp turns lane-parallel: lane i adds the
// terms of pending row i in block order (the reference's `sumf +=` loop) and runs the
// epilogue, so the sequential part and the SiLU are paid once per batch of rows and not
// once per row.
#pragma once
#include "blockmath.cuh"
#include "device_utils.cuh"
#include "gemv.cuh"

namespace aot {

__device__ __forceinline__ U4 rd_lds128(uint32_t a) {
  U4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t rd_lds32(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ int rd_lds_s16(uint32_t a) {
  int v;
  asm("ld.shared.s16 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
// unsigned bytes x signed bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float half_bits_hw(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// A lane's slice of one Q8_K block image: 64 int8 values, the partial sums it needs and
// the block scale. Two layouts, because the K-quant kinds pair weights and activations
// differently:
//   K4 (Q4_K, Q5_K): quarter c = elements [64c, 64c+64); b[0], b[1] = sums of its two
//       32-element sub-blocks.
//   Q6 (Q6_K): half n = c/2, elements l in [16*(c%2), +16) of each of the half's four
//       32-element quarters; b[k] = the 16-element sum that belongs to quarter k.
struct YQuarter {
  uint32_t y[16];
  int b[4];
  float d;
};
enum YLayout : int { YL_NONE = 0, YL_K4 = 1, YL_Q6 = 2 };

__device__ __forceinline__ void yq_load_k4(YQuarter& Y, uint32_t xb, int c) {
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const U4 v = rd_lds128(xb + 64 * c + 16 * k);
    Y.y[4 * k] = v.x;
    Y.y[4 * k + 1] = v.y;
    Y.y[4 * k + 2] = v.z;
    Y.y[4 * k + 3] = v.w;
  }
  const uint32_t bx = rd_lds32(xb + XK_BSUMS + 8 * c), by = rd_lds32(xb + XK_BSUMS + 8 * c + 4);
  Y.b[0] = (int)(short)(bx & 0xFFFF) + ((int)bx >> 16);
  Y.b[1] = (int)(short)(by & 0xFFFF) + ((int)by >> 16);
  Y.b[2] = 0;
  Y.b[3] = 0;
  Y.d = __uint_as_float(rd_lds32(xb + XK_D));
}
__device__ __forceinline__ void yq_load_q6(YQuarter& Y, uint32_t xb, int c) {
  const int n = c >> 1, half = c & 1;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const U4 v = rd_lds128(xb + 128 * n + 16 * half + 32 * k);
    Y.y[4 * k] = v.x;
    Y.y[4 * k + 1] = v.y;
    Y.y[4 * k + 2] = v.z;
    Y.y[4 * k + 3] = v.w;
  }
  const uint32_t bsa = xb + XK_BSUMS + 2 * (8 * n + half);
#pragma unroll
  for (int k = 0; k < 4; k++) Y.b[k] = rd_lds_s16(bsa + 4 * k);
  Y.d = __uint_as_float(rd_lds32(xb + XK_D));
}

// Quarter c of a Q4_K / Q5_K block at shared address wb (16-byte aligned): this lane's
// share of the two integers of matvec.rs:89-103 (the four lanes of a block add theirs up
// with two shuffles), and the block's d|dmin word.
template <bool Q5>
__device__ __forceinline__ void k4_partial(uint32_t wb, int c, const YQuarter& Y, int& sumi, int& summ, uint32_t& dd) {
  const U4 hdr = rd_lds128(wb);
  dd = hdr.x;
  const uint32_t qs = wb + (Q5 ? 48 : 16) + 32 * c;
  const U4 wa = rd_lds128(qs), wc = rd_lds128(qs + 16);
  U4 h0{0, 0, 0, 0}, h1{0, 0, 0, 0};
  if (Q5) {
    h0 = rd_lds128(wb + 16);
    h1 = rd_lds128(wb + 32);
  }
  const K4Scales s = k4_unpack(hdr.y, hdr.z, hdr.w);
  // two accumulators per sub-block halve the length of the dp4a chains
  int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t w = i < 4 ? u4_get(wa, i) : u4_get(wc, i - 4);
    int& alo = (i & 1) ? lo1 : lo0;
    int& ahi = (i & 1) ? hi1 : hi0;
    if (Q5) {
      const uint32_t h = i < 4 ? u4_get(h0, i) : u4_get(h1, i - 4);
      const uint32_t lo = (w & 0x0F0F0F0Fu) | (((h >> (2 * c)) & 0x01010101u) << 4);
      const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) | (((h >> (2 * c + 1)) & 0x01010101u) << 4);
      alo = __dp4a((int)lo, (int)Y.y[i], alo);
      ahi = __dp4a((int)hi, (int)Y.y[8 + i], ahi);
    } else {
      // the high nibbles stay in place (16 x their value, as unsigned bytes); the sum is
      // an exact multiple of 16 and is shifted back below
      alo = __dp4a((int)(w & 0x0F0F0F0Fu), (int)Y.y[i], alo);
      ahi = dp4a_us(w & 0xF0F0F0F0u, Y.y[8 + i], ahi);
    }
  }
  const int s_lo = lo0 + lo1;
  int s_hi = hi0 + hi1;
  if (!Q5) s_hi >>= 4;
  const uint32_t scw = c < 2 ? s.sc_lo : s.sc_hi, mw = c < 2 ? s.m_lo : s.m_hi;
  const int sh = (c & 1) * 16;
  const int sc0 = (scw >> sh) & 0xFF, sc1 = (scw >> (sh + 8)) & 0xFF;
  const int m0 = (mw >> sh) & 0xFF, m1 = (mw >> (sh + 8)) & 0xFF;
  sumi = sc0 * s_lo + sc1 * s_hi;
  summ = m0 * Y.b[0] + m1 * Y.b[1];
}

// Lane c's share of a Q6_K block at shared address wb (2-byte aligned): words come from the
// 4-byte aligned stream through a funnel shift, four consecutive words from five loads.
// Returns the lane's share of the block's integer sum (matvec.rs:146-163) and the d half.
__device__ __forceinline__ int q6k_partial(uint32_t wb, int c, const YQuarter& Y, uint32_t& dbits) {
  const uint32_t sh = (wb & 2u) * 8u, p = wb & ~3u;
  auto load4 = [&](int k, uint32_t w[4]) {
    const uint32_t a0 = rd_lds32(p + 4 * k), a1 = rd_lds32(p + 4 * k + 4), a2 = rd_lds32(p + 4 * k + 8),
                   a3 = rd_lds32(p + 4 * k + 12), a4 = rd_lds32(p + 4 * k + 16);
    w[0] = funnel_r(a0, a1, sh);
    w[1] = funnel_r(a1, a2, sh);
    w[2] = funnel_r(a2, a3, sh);
    w[3] = funnel_r(a3, a4, sh);
  };
  const int n = c >> 1, half = c & 1;
  uint32_t l0[4], l32[4], h[4];
  load4(16 * n + 4 * half, l0);
  load4(16 * n + 8 + 4 * half, l32);
  load4(32 + 8 * n + 4 * half, h);
  // scale words 48+2n, 49+2n and the d half at byte 208 (word 52, low half)
  const uint32_t sa = p + 4 * (48 + 2 * n);
  const uint32_t t0 = rd_lds32(sa), t1 = rd_lds32(sa + 4), t2 = rd_lds32(sa + 8);
  const uint32_t s01 = funnel_r(t0, t1, sh), s23 = funnel_r(t1, t2, sh);
  const uint32_t da = wb + 208;
  dbits = (rd_lds32(da & ~3u) >> ((da & 2u) * 8u)) & 0xFFFFu;
  int a1 = 0, a2 = 0, a3 = 0, a4 = 0;
#pragma unroll
  for (int ii = 0; ii < 4; ii++) {
    const uint32_t q1 = (l0[ii] & 0x0F0F0F0Fu) | ((h[ii] << 4) & 0x30303030u);
    const uint32_t q2 = (l32[ii] & 0x0F0F0F0Fu) | ((h[ii] << 2) & 0x30303030u);
    const uint32_t q3 = ((l0[ii] >> 4) & 0x0F0F0F0Fu) | (h[ii] & 0x30303030u);
    const uint32_t q4 = ((l32[ii] >> 4) & 0x0F0F0F0Fu) | ((h[ii] >> 2) & 0x30303030u);
    a1 = __dp4a((int)q1, (int)Y.y[ii], a1);
    a2 = __dp4a((int)q2, (int)Y.y[4 + ii], a2);
    a3 = __dp4a((int)q3, (int)Y.y[8 + ii], a3);
    a4 = __dp4a((int)q4, (int)Y.y[12 + ii], a4);
  }
  const int c1 = (int)(int8_t)((s01 >> (8 * half)) & 0xFF), c2 = (int)(int8_t)((s01 >> (8 * half + 16)) & 0xFF);
  const int c3 = (int)(int8_t)((s23 >> (8 * half)) & 0xFF), c4 = (int)(int8_t)((s23 >> (8 * half + 16)) & 0xFF);
  int tot = c1 * a1 + c2 * a2 + c3 * a3 + c4 * a4;
  tot -= 32 * (c1 * Y.b[0] + c2 * Y.b[1] + c3 * Y.b[2] + c4 * Y.b[3]);
  return tot;
}

// The activation slice a warp currently holds: layout and the first block of the group
// of eight blocks it belongs to.
struct YCache {
  YQuarter Y;
  int lay, g0;
};

// Block terms of NR K-quant rows of the same kind (NR = 2: a gate row and its up row, whose
// dependent chains interleave): row[r] = shared address of the row's first block, `sxa` =
// shared address of the activation images, nb blocks. terms[r][b] receives the f32 term of
// block b. Every lane of the warp calls it; control flow is warp-uniform.
// `dbg_i` / `dbg_m`, when given, receive the integers of every (row, block) before any
// float arithmetic (parity export): dbg_i[dbg_row[r] * nb + b].
template <int NR>
__device__ __forceinline__ void warp_rows_terms(int kind, const uint32_t (&row)[NR], uint32_t sxa, int nb, YCache& yc,
                                                float* const (&terms)[NR], int* dbg_i = nullptr, int* dbg_m = nullptr,
                                                const int* dbg_row = nullptr) {
  const int lane = threadIdx.x & 31, bl = lane >> 2, c = lane & 3;
  const int bs = kind_size(kind);
  const int lay = kind == Q6_K ? YL_Q6 : YL_K4;
#pragma unroll 1
  for (int g0 = 0; g0 < nb; g0 += 8) {
    const int b = g0 + bl;
    // idle lanes recompute the last block so that every lane reaches the shuffles
    const int bb = b < nb ? b : nb - 1;
    if (yc.lay != lay || yc.g0 != g0) {
      const uint32_t xb = sxa + (uint32_t)bb * XK_STRIDE;
      if (lay == YL_Q6) yq_load_q6(yc.Y, xb, c); else yq_load_k4(yc.Y, xb, c);
      yc.lay = lay;
      yc.g0 = g0;
    }
    int si[NR], sm[NR];
    uint32_t dd[NR];
    if (kind == Q6_K) {
#pragma unroll
      for (int r = 0; r < NR; r++) {
        si[r] = q6k_partial(row[r] + (uint32_t)bb * bs, c, yc.Y, dd[r]);
        sm[r] = 0;
      }
    } else if (kind == Q5_K) {
#pragma unroll
      for (int r = 0; r < NR; r++) k4_partial<true>(row[r] + (uint32_t)bb * bs, c, yc.Y, si[r], sm[r], dd[r]);
    } else {
#pragma unroll
      for (int r = 0; r < NR; r++) k4_partial<false>(row[r] + (uint32_t)bb * bs, c, yc.Y, si[r], sm[r], dd[r]);
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
#pragma unroll
      for (int r = 0; r < NR; r++) {
        si[r] += __shfl_xor_sync(0xffffffffu, si[r], o);
        if (kind != Q6_K) sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], o);
      }
    }
    if (dbg_i && c == 0 && b < nb) {
#pragma unroll
      for (int r = 0; r < NR; r++) {
        dbg_i[(size_t)dbg_row[r] * nb + b] = si[r];
        if (dbg_m && kind != Q6_K) dbg_m[(size_t)dbg_row[r] * nb + b] = sm[r];
      }
    }
    if (c == 0 && b < nb) {
#pragma unroll
      for (int r = 0; r < NR; r++)
        terms[r][b] = kind == Q6_K ? q6k_term(half_bits_hw(dd[r]), yc.Y.d, si[r])
                                   : k4_term(half_bits_hw(dd[r] & 0xFFFFu), half_bits_hw(dd[r] >> 16), yc.Y.d, si[r], sm[r]);
    }
  }
}

// (((0 + t[0]) + t[1]) + ...), the order of the reference's per-row loop.
__device__ __forceinline__ float terms_seq_sum(const float* t, int nb) {
  float s = 0.0f;
  int b = 0;
  for (; b + 4 <= nb; b += 4) {
    const float t0 = t[b], t1 = t[b + 1], t2 = t[b + 2], t3 = t[b + 3];
    s = fadd(s, t0);
    s = fadd(s, t1);
    s = fadd(s, t2);
    s = fadd(s, t3);
  }
  for (; b < nb; b++) s = fadd(s, t[b]);
  return s;
}

}  // namespace aot
