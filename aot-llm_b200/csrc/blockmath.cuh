// Per-block arithmetic of the quantized dot products, written once for device
// code and (for CPU-side unit checks of the arithmetic only) plain C++.
//
// Every function reproduces the integer sums and the order of f32 operations of
// the reference CPU kernels (crates/aot-kernels/src/matvec.rs:82-167 scalar,
// crates/aot-kernels/src/simd_avx2.rs AVX2) so results are bit-identical:
//   * integer block sums are exact in any order;
//   * f32 products and sums use explicit round-to-nearest mul/add/sub (never
//     contracted) except where the reference issues an explicit fmadd.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define AOT_HD __host__ __device__ __forceinline__
#else
#define AOT_HD inline
#endif

#if defined(__CUDA_ARCH__)
#define AOT_DEVICE_CODE 1
#else
#define AOT_DEVICE_CODE 0
#include <math.h>
#endif

namespace aot {

// Kind order of crates/aot-kernels/src/quant.rs:34-44.
enum Kind : int { F32 = 0, F16 = 1, BF16 = 2, Q4_0 = 3, Q5_0 = 4, Q8_0 = 5, Q4_K = 6, Q5_K = 7, Q6_K = 8, N_KINDS = 9 };
enum Act : int { ACT_F32 = 0, ACT_Q8_0 = 1, ACT_Q8_K = 2 };

AOT_HD int kind_block(int k) { return k <= BF16 ? 1 : (k <= Q8_0 ? 32 : 256); }
AOT_HD int kind_size(int k) {
  switch (k) {
    case F32: return 4;
    case F16: case BF16: return 2;
    case Q4_0: return 18;
    case Q5_0: return 22;
    case Q8_0: return 34;
    case Q4_K: return 144;
    case Q5_K: return 176;
    default: return 210;
  }
}
AOT_HD size_t kind_row_bytes(int k, size_t n) { return n / (size_t)kind_block(k) * (size_t)kind_size(k); }
AOT_HD int kind_act(int k) { return k <= BF16 ? ACT_F32 : (k <= Q8_0 ? ACT_Q8_0 : ACT_Q8_K); }

// Activation blocks as the reference lays them out (quant.rs:194-216).
struct BlockQ8_0 {
  float d;
  int8_t qs[32];
};
struct BlockQ8_K {
  float d;
  int8_t qs[256];
  int16_t bsums[16];
};
static_assert(sizeof(BlockQ8_0) == 36 && sizeof(BlockQ8_K) == 292, "activation block layout");

// ---- exact scalar helpers ---------------------------------------------------
AOT_HD float fmul(float a, float b) {
#if AOT_DEVICE_CODE
  return __fmul_rn(a, b);
#else
  volatile float r = a * b;
  return r;
#endif
}
AOT_HD float fadd(float a, float b) {
#if AOT_DEVICE_CODE
  return __fadd_rn(a, b);
#else
  volatile float r = a + b;
  return r;
#endif
}
AOT_HD float fsub(float a, float b) {
#if AOT_DEVICE_CODE
  return __fsub_rn(a, b);
#else
  volatile float r = a - b;
  return r;
#endif
}
AOT_HD float ffma(float a, float b, float c) {
#if AOT_DEVICE_CODE
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}
AOT_HD float fdiv(float a, float b) {
#if AOT_DEVICE_CODE
  return __fdiv_rn(a, b);
#else
  volatile float r = a / b;
  return r;
#endif
}
AOT_HD float fsqrt(float a) {
#if AOT_DEVICE_CODE
  return __fsqrt_rn(a);
#else
  return sqrtf(a);
#endif
}
AOT_HD float i2f(int v) {
#if AOT_DEVICE_CODE
  return __int2float_rn(v);
#else
  return (float)v;
#endif
}

AOT_HD uint32_t f2u(float f) {
#if AOT_DEVICE_CODE
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
AOT_HD float u2f(uint32_t u) {
#if AOT_DEVICE_CODE
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

// binary16 bits -> f32, exact for every input including subnormals
// (quant.rs:96-125).
AOT_HD float half_bits_to_float(uint32_t h) {
  h &= 0xFFFFu;
  uint32_t sign = (h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  if (e == 0) {
    // value = m * 2^-24: the int->float conversion and the power-of-two scale
    // are both exact.
    float v = fmul((float)m, 5.9604644775390625e-08f);
    return u2f(f2u(v) | sign);
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
AOT_HD float bf16_bits_to_float(uint32_t h) { return u2f((h & 0xFFFFu) << 16); }

// Signed 4x8-bit dot product with accumulate.
AOT_HD int dp4a(uint32_t a, uint32_t b, int c) {
#if AOT_DEVICE_CODE
  return __dp4a((int)a, (int)b, c);
#else
  for (int i = 0; i < 4; i++) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
#endif
}

// ---- K-quant 6-bit scales ---------------------------------------------------
// The eight (scale, min) pairs of quant.rs:292-298 as four packed words, four
// values per word: sc[0..3], sc[4..7], m[0..3], m[4..7]. `s0,s1,s2` are the three
// little-endian words of the 12-byte scale array.
struct K4Scales {
  uint32_t sc_lo, sc_hi, m_lo, m_hi;
};
AOT_HD K4Scales k4_unpack(uint32_t s0, uint32_t s1, uint32_t s2) {
  K4Scales r;
  r.sc_lo = s0 & 0x3F3F3F3Fu;
  r.m_lo = s1 & 0x3F3F3F3Fu;
  r.sc_hi = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
  r.m_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
  return r;
}
AOT_HD int byte_of(uint32_t w, int i) { return (int)((w >> (8 * i)) & 0xFFu); }

// ---- Q4_K / Q5_K: one 256-weight super-block against one Q8_K block ----------
// `hdr`: d|dmin halves and the 12 scale bytes (block bytes 0..15). `qh`: the 32
// fifth-bit bytes of Q5_K as 8 words (unused for Q4_K). `qs`: 128 nibble bytes as
// 32 words. `y`: 256 int8 as 64 words. `bsums`: the 16 partial sums of y.
// Outputs the two integers of matvec.rs:89-103.
template <bool Q5, class QsLoad, class QhLoad, class YLoad>
AOT_HD void k4_block_sums(const K4Scales& s, QsLoad qs, QhLoad qh, YLoad y, const int16_t* bsums, int& sumi,
                          int& summ) {
  int si = 0, sm = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    int s_lo = 0, s_hi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      uint32_t w = qs(8 * c + i);
      uint32_t lo = w & 0x0F0F0F0Fu;
      uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;
      if (Q5) {
        uint32_t h = qh(i);
        lo |= ((h >> (2 * c)) & 0x01010101u) << 4;
        hi |= ((h >> (2 * c + 1)) & 0x01010101u) << 4;
      }
      s_lo = dp4a(lo, y(16 * c + i), s_lo);
      s_hi = dp4a(hi, y(16 * c + 8 + i), s_hi);
    }
    int j0 = 2 * c, j1 = 2 * c + 1;
    int sc0 = byte_of(j0 < 4 ? s.sc_lo : s.sc_hi, j0 & 3);
    int sc1 = byte_of(j1 < 4 ? s.sc_lo : s.sc_hi, j1 & 3);
    int m0 = byte_of(j0 < 4 ? s.m_lo : s.m_hi, j0 & 3);
    int m1 = byte_of(j1 < 4 ? s.m_lo : s.m_hi, j1 & 3);
    si += sc0 * s_lo + sc1 * s_hi;
    sm += m0 * ((int)bsums[2 * j0] + (int)bsums[2 * j0 + 1]) + m1 * ((int)bsums[2 * j1] + (int)bsums[2 * j1 + 1]);
  }
  sumi = si;
  summ = sm;
}

// matvec.rs:84-85,104 / simd_avx2.rs:152-153,169: d and dmin are scaled by the
// activation scale first, then `d*sumi - dmin*summ`, all unfused.
AOT_HD float k4_term(float d_w, float dmin_w, float d_x, int sumi, int summ) {
  float d = fmul(d_w, d_x);
  float dmin = fmul(dmin_w, d_x);
  return fsub(fmul(d, i2f(sumi)), fmul(dmin, i2f(summ)));
}

// ---- Q6_K ---------------------------------------------------------------------
// `w(k)`: word k of the 210-byte block (ql 0..31, qh 32..47, scales 48..51,
// d in the low half of word 52). Values are used unsigned (0..63) and the -32
// offset goes through the activation block sums, which is integer-identical to
// the signed form (simd_avx2.rs:234-239, 264).
template <class WLoad, class YLoad>
AOT_HD int q6k_block_sum(WLoad w, YLoad y, const int16_t* bsums) {
  int total = 0, bias = 0;
  uint32_t scw[4] = {w(48), w(49), w(50), w(51)};
#pragma unroll
  for (int g = 0; g < 16; g++) bias += (int)(int8_t)byte_of(scw[g >> 2], g & 3) * (int)bsums[g];
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int half = 0; half < 2; half++) {  // l in [16*half, 16*half+16)
      int a1 = 0, a2 = 0, a3 = 0, a4 = 0;
#pragma unroll
      for (int ii = 0; ii < 4; ii++) {
        int i = 4 * half + ii;
        uint32_t l0 = w(16 * n + i), l32 = w(16 * n + 8 + i), h = w(32 + 8 * n + i);
        uint32_t q1 = (l0 & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
        uint32_t q2 = (l32 & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
        uint32_t q3 = ((l0 >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
        uint32_t q4 = ((l32 >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
        a1 = dp4a(q1, y(32 * n + i), a1);
        a2 = dp4a(q2, y(32 * n + 8 + i), a2);
        a3 = dp4a(q3, y(32 * n + 16 + i), a3);
        a4 = dp4a(q4, y(32 * n + 24 + i), a4);
      }
      int g = 8 * n + half;
      total += (int)(int8_t)byte_of(scw[g >> 2], g & 3) * a1;
      total += (int)(int8_t)byte_of(scw[(g + 2) >> 2], (g + 2) & 3) * a2;
      total += (int)(int8_t)byte_of(scw[(g + 4) >> 2], (g + 4) & 3) * a3;
      total += (int)(int8_t)byte_of(scw[(g + 6) >> 2], (g + 6) & 3) * a4;
    }
  }
  return total - 32 * bias;
}

// matvec.rs:144,165
AOT_HD float q6k_term(float d_w, float d_x, int sumi) { return fmul(fmul(d_w, d_x), i2f(sumi)); }

// ---- Q4_0 / Q5_0 / Q8_0: one AVX2 lane of one 32-weight block -----------------
// The AVX2 kernels keep eight f32 lane accumulators; lane k sums elements
// 4k..4k+3 of each block (maddubs pairs folded by madd with ones,
// simd_avx2.rs:40-45) and does acc = fma(d_w*d_x, float(p), acc) per block
// (simd_avx2.rs:61-72). These return p for lane k.
// Q4_0: `qs4` = the four nibble bytes that hold lane k's elements: bytes
// 4*(k&3)..+3 of qs; lanes 0..3 use the low nibbles, 4..7 the high ones.
AOT_HD int q4_0_lane(uint32_t qs4, int k, uint32_t y4) {
  uint32_t v = (k < 4 ? qs4 : (qs4 >> 4)) & 0x0F0F0F0Fu;
  // subtract 8 from each byte: values 0..15 -> -8..7, no borrow across bytes
  // once bit 7 is protected.
  uint32_t s = ((v | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
  return dp4a(s, y4, 0);
}
// Q5_0: fifth bits come from qh bits 4k..4k+3.
AOT_HD int q5_0_lane(uint32_t qs4, uint32_t qh, int k, uint32_t y4) {
  uint32_t v = (k < 4 ? qs4 : (qs4 >> 4)) & 0x0F0F0F0Fu;
  uint32_t b = (qh >> (4 * k)) & 0xFu;
  // spread bits 0..3 of b to bit 4 of bytes 0..3
  uint32_t hb = ((b & 1u) << 4) | ((b & 2u) << 11) | ((b & 4u) << 18) | ((b & 8u) << 25);
  v |= hb;
  uint32_t s = ((v | 0x80808080u) - 0x10101010u) ^ 0x80808080u;  // 0..31 -> -16..15
  return dp4a(s, y4, 0);
}
AOT_HD int q8_0_lane(uint32_t w4, uint32_t y4) { return dp4a(w4, y4, 0); }

// hsum_f32 of simd_avx2.rs:29-34 over the eight lane accumulators.
AOT_HD float hsum8(const float a[8]) {
  float s0 = fadd(a[0], a[4]), s1 = fadd(a[1], a[5]), s2 = fadd(a[2], a[6]), s3 = fadd(a[3], a[7]);
  float t0 = fadd(s0, s2), t1 = fadd(s1, s3);
  return fadd(t0, t1);
}

// ---- element dequantizers (token embedding rows, quant.rs:300-443) ----------------
// Value of element `e` of a row of `kind`; `row` points at the row's first byte.
AOT_HD float dequant_elem(int kind, const uint8_t* row, size_t e) {
  auto rd16 = [](const uint8_t* p) -> uint32_t { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); };
  auto rd32 = [](const uint8_t* p) -> uint32_t {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
  };
  switch (kind) {
    case F32: return u2f(rd32(row + 4 * e));
    case F16: return half_bits_to_float(rd16(row + 2 * e));
    case BF16: return bf16_bits_to_float(rd16(row + 2 * e));
    case Q4_0: {
      const uint8_t* b = row + (e / 32) * 18;
      int j = (int)(e % 32);
      uint8_t q = b[2 + (j & 15)];
      int v = (j < 16 ? (q & 0x0F) : (q >> 4)) - 8;
      return fmul(i2f(v), half_bits_to_float(rd16(b)));
    }
    case Q5_0: {
      const uint8_t* b = row + (e / 32) * 22;
      int j = (int)(e % 32);
      uint32_t qh = rd32(b + 2);
      uint8_t q = b[6 + (j & 15)];
      int v = (int)((j < 16 ? (uint32_t)(q & 0x0F) : (uint32_t)(q >> 4)) | (((qh >> j) & 1u) << 4)) - 16;
      return fmul(i2f(v), half_bits_to_float(rd16(b)));
    }
    case Q8_0: {
      const uint8_t* b = row + (e / 32) * 34;
      return fmul(i2f((int)(int8_t)b[2 + e % 32]), half_bits_to_float(rd16(b)));
    }
    case Q4_K:
    case Q5_K: {
      const bool q5 = kind == Q5_K;
      const uint8_t* b = row + (e / 256) * (q5 ? 176 : 144);
      int r = (int)(e % 256), j = r / 32, l = r % 32, c = j / 2;
      float d = half_bits_to_float(rd16(b)), dmin = half_bits_to_float(rd16(b + 2));
      K4Scales s = k4_unpack(rd32(b + 4), rd32(b + 8), rd32(b + 12));
      int sc = byte_of(j < 4 ? s.sc_lo : s.sc_hi, j & 3), m = byte_of(j < 4 ? s.m_lo : s.m_hi, j & 3);
      uint8_t q = b[(q5 ? 48 : 16) + 32 * c + l];
      int v = (j & 1) ? (q >> 4) : (q & 0x0F);
      if (q5 && (b[16 + l] & (1u << j))) v += 16;
      // quant.rs:366-374: (d*sc)*q - dmin*m
      return fsub(fmul(fmul(d, i2f(sc)), i2f(v)), fmul(dmin, i2f(m)));
    }
    default: {  // Q6_K
      const uint8_t* b = row + (e / 256) * 210;
      int r = (int)(e % 256), n = r / 128, rr = r % 128, quarter = rr / 32, l = rr % 32;
      uint8_t lb = b[64 * n + l + 32 * (quarter & 1)];
      int lo = quarter < 2 ? (lb & 0x0F) : (lb >> 4);
      int hi = (b[128 + 32 * n + l] >> (2 * quarter)) & 3;
      int q = (lo | (hi << 4)) - 32;
      int sc = (int)(int8_t)b[192 + 8 * n + l / 16 + 2 * quarter];
      // quant.rs:422-425: d * sc * q, left to right
      return fmul(fmul(half_bits_to_float(rd16(b + 208)), i2f(sc)), i2f(q));
    }
  }
}

}  // namespace aot
