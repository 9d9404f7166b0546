// Oracle (test infrastructure): dot products of one quantized weight row with
// one (or four) activation vectors. Restates the scalar table of
// crates/aot-kernels/src/matvec.rs:30-192 and the AVX2(+FMA, +F16C) table of
// crates/aot-kernels/src/simd_avx2.rs, instruction for instruction where the
// order of floating-point operations is observable.
#include <immintrin.h>
#include <math.h>

#include "oracle_internal.h"

#define AVX2 __attribute__((target("avx2,fma")))
#define AVX2_F16C __attribute__((target("avx2,fma,f16c")))

typedef orc_block_q8_0 B0;
typedef orc_block_q8_k BK;

static inline void k4(int j, const uint8_t* s, int* sc, int* m) {
  uint8_t a, b;
  orc_scale_min_k4(j, s, &a, &b);
  *sc = a;
  *m = b;
}

// ---------------------------------------------------------------------------
// Integer block sums (shared by the scalar dots and the parity export)
// ---------------------------------------------------------------------------

// matvec.rs:38-43
static int isum_q4_0(const uint8_t* b, const B0* y) {
  int s = 0;
  for (int j = 0; j < 16; j++) {
    uint8_t q = b[2 + j];
    s += ((int)(q & 0x0F) - 8) * (int)y->qs[j];
    s += ((int)(q >> 4) - 8) * (int)y->qs[j + 16];
  }
  return s;
}

// matvec.rs:54-62
static int isum_q5_0(const uint8_t* b, const B0* y) {
  uint32_t qh = rd_u32(b + 2);
  int s = 0;
  for (int j = 0; j < 16; j++) {
    uint8_t q = b[6 + j];
    int lo = (int)((uint32_t)(q & 0x0F) | (((qh >> j) & 1u) << 4)) - 16;
    int hi = (int)((uint32_t)(q >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16;
    s += lo * (int)y->qs[j];
    s += hi * (int)y->qs[j + 16];
  }
  return s;
}

// matvec.rs:73-76
static int isum_q8_0(const uint8_t* b, const B0* y) {
  int s = 0;
  for (int j = 0; j < 32; j++) s += (int)(int8_t)b[2 + j] * (int)y->qs[j];
  return s;
}

// matvec.rs:89-103 (hbits == 0) and 117-135 (hbits == 1)
static void isum_k4(const uint8_t* scales, const uint8_t* qh, const uint8_t* qs, const BK* y, int* sumi_out,
                    int* summ_out) {
  int sumi = 0, summ = 0;
  for (int j = 0; j < 8; j++) {
    int sc, m;
    k4(j, scales, &sc, &m);
    summ += m * ((int)y->bsums[2 * j] + (int)y->bsums[2 * j + 1]);
    int c = j / 2;
    uint8_t hbit = (uint8_t)(1u << j);
    int s = 0;
    for (int l = 0; l < 32; l++) {
      uint8_t q = qs[32 * c + l];
      int v = (j % 2 == 0) ? (q & 0x0F) : (q >> 4);
      if (qh && (qh[l] & hbit)) v += 16;
      s += v * (int)y->qs[32 * j + l];
    }
    sumi += sc * s;
  }
  *sumi_out = sumi;
  *summ_out = summ;
}

// matvec.rs:146-163
static int isum_q6_k(const uint8_t* b, const BK* y) {
  int sumi = 0;
  for (int n = 0; n < 2; n++) {
    const uint8_t* ql = b + 64 * n;
    const uint8_t* qh = b + 128 + 32 * n;
    const int8_t* sc = (const int8_t*)(b + 192 + 8 * n);
    const int8_t* yy = y->qs + 128 * n;
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
      int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      sumi += (int)sc[is] * q1 * (int)yy[l];
      sumi += (int)sc[is + 2] * q2 * (int)yy[l + 32];
      sumi += (int)sc[is + 4] * q3 * (int)yy[l + 64];
      sumi += (int)sc[is + 6] * q4 * (int)yy[l + 96];
    }
  }
  return sumi;
}

// ---------------------------------------------------------------------------
// Scalar table (matvec.rs:30-192)
// ---------------------------------------------------------------------------

static float s_q4_0(const uint8_t* w, const void* xv, size_t cols) {
  const B0* x = (const B0*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 32; i++) {
    const uint8_t* b = w + i * 18;
    sum += (float)isum_q4_0(b, &x[i]) * rd_f16(b) * x[i].d;
  }
  return sum;
}

static float s_q5_0(const uint8_t* w, const void* xv, size_t cols) {
  const B0* x = (const B0*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 32; i++) {
    const uint8_t* b = w + i * 22;
    sum += (float)isum_q5_0(b, &x[i]) * rd_f16(b) * x[i].d;
  }
  return sum;
}

static float s_q8_0(const uint8_t* w, const void* xv, size_t cols) {
  const B0* x = (const B0*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 32; i++) {
    const uint8_t* b = w + i * 34;
    sum += (float)isum_q8_0(b, &x[i]) * rd_f16(b) * x[i].d;
  }
  return sum;
}

static float s_q4_k(const uint8_t* w, const void* xv, size_t cols) {
  const BK* x = (const BK*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 144;
    float d = rd_f16(b) * x[i].d;
    float dmin = rd_f16(b + 2) * x[i].d;
    int sumi, summ;
    isum_k4(b + 4, NULL, b + 16, &x[i], &sumi, &summ);
    sum += d * (float)sumi - dmin * (float)summ;
  }
  return sum;
}

static float s_q5_k(const uint8_t* w, const void* xv, size_t cols) {
  const BK* x = (const BK*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 176;
    float d = rd_f16(b) * x[i].d;
    float dmin = rd_f16(b + 2) * x[i].d;
    int sumi, summ;
    isum_k4(b + 4, b + 16, b + 48, &x[i], &sumi, &summ);
    sum += d * (float)sumi - dmin * (float)summ;
  }
  return sum;
}

static float s_q6_k(const uint8_t* w, const void* xv, size_t cols) {
  const BK* x = (const BK*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 210;
    float d = rd_f16(b + 208) * x[i].d;
    sum += d * (float)isum_q6_k(b, &x[i]);
  }
  return sum;
}

static float s_f16(const uint8_t* w, const void* xv, size_t cols) {
  const float* x = (const float*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols; i++) sum += rd_f16(w + 2 * i) * x[i];
  return sum;
}

static float s_bf16(const uint8_t* w, const void* xv, size_t cols) {
  const float* x = (const float*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols; i++) sum += orc_bf16_to_f32(rd_u16(w + 2 * i)) * x[i];
  return sum;
}

static float s_f32(const uint8_t* w, const void* xv, size_t cols) {
  const float* x = (const float*)xv;
  float sum = 0.0f;
  for (size_t i = 0; i < cols; i++) sum += rd_f32(w + 4 * i) * x[i];
  return sum;
}

// ---------------------------------------------------------------------------
// AVX2 table (simd_avx2.rs)
// ---------------------------------------------------------------------------

// simd_avx2.rs:19-25: fold the halves, then lanes (2,3) onto (0,1), then 1 onto 0.
AVX2 static inline int hsum_i32(__m256i v) {
  __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
  s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x01));
  return _mm_cvtsi128_si32(s);
}

// simd_avx2.rs:29-34: ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)).
AVX2 static inline float hsum_f32(__m256 v) {
  __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 0x55));
  return _mm_cvtss_f32(s);
}

// simd_avx2.rs:40-45: signed x signed through |a| and b*sign(a).
AVX2 static inline __m256i dot32_i8(__m256i a, __m256i b) {
  __m256i ax = _mm256_sign_epi8(a, a);
  __m256i sy = _mm256_sign_epi8(b, a);
  return _mm256_madd_epi16(_mm256_maddubs_epi16(ax, sy), _mm256_set1_epi16(1));
}

// simd_avx2.rs:51-55: low nibbles in the low lane, high nibbles in the high lane.
AVX2 static inline __m256i nib32(const uint8_t* p) {
  __m128i t = _mm_loadu_si128((const __m128i*)p);
  __m256i both = _mm256_set_m128i(_mm_srli_epi16(t, 4), t);
  return _mm256_and_si256(both, _mm256_set1_epi8(0x0F));
}

// simd_avx2.rs:81-88
AVX2 static inline __m256i bits_to_bytes32(const uint8_t* p) {
  int32_t qh = (int32_t)rd_u32(p);
  __m256i shuf =
      _mm256_set_epi64x(0x0303030303030303LL, 0x0202020202020202LL, 0x0101010101010101LL, 0x0000000000000000LL);
  __m256i bytes = _mm256_shuffle_epi8(_mm256_set1_epi32(qh), shuf);
  __m256i mask = _mm256_set1_epi64x(0x7fbfdfeff7fbfdfeLL);
  return _mm256_cmpeq_epi8(_mm256_or_si256(bytes, mask), _mm256_set1_epi64x(-1));
}

// simd_avx2.rs:94-98
AVX2 static inline __m256i q5_0_bytes(const uint8_t* b) {
  __m256i bx = nib32(b + 6);
  __m256i hi = _mm256_andnot_si256(bits_to_bytes32(b + 2), _mm256_set1_epi8((char)0xF0));
  return _mm256_or_si256(bx, hi);
}

enum { W_Q4_0, W_Q5_0, W_Q8_0 };

template <int W>
AVX2 static inline __m256i load_w32(const uint8_t* b) {
  if (W == W_Q4_0) return _mm256_sub_epi8(nib32(b + 2), _mm256_set1_epi8(8));
  if (W == W_Q5_0) return q5_0_bytes(b);
  return _mm256_loadu_si256((const __m256i*)(b + 2));
}

// simd_avx2.rs:58-72, 101-129: eight lane accumulators, one fmadd per block.
template <int W, int SZ>
AVX2 static float a_q32(const uint8_t* w, const void* xv, size_t cols) {
  const B0* x = (const B0*)xv;
  __m256 acc = _mm256_setzero_ps();
  for (size_t i = 0; i < cols / 32; i++) {
    const uint8_t* b = w + i * SZ;
    __m256 d = _mm256_set1_ps(rd_f16(b) * x[i].d);
    __m256i bx = load_w32<W>(b);
    __m256i by = _mm256_loadu_si256((const __m256i*)x[i].qs);
    acc = _mm256_fmadd_ps(d, _mm256_cvtepi32_ps(dot32_i8(bx, by)), acc);
  }
  return hsum_f32(acc);
}

// simd_avx2.rs:273-337
template <int W, int SZ>
AVX2 static void a_q32_x4(const uint8_t* w, const void* const xs[4], size_t cols, float out[4]) {
  __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps()};
  for (size_t i = 0; i < cols / 32; i++) {
    const uint8_t* b = w + i * SZ;
    float d = rd_f16(b);
    __m256i bx = load_w32<W>(b);
    __m256i ax = _mm256_sign_epi8(bx, bx);
    for (int k = 0; k < 4; k++) {
      const B0* y = (const B0*)xs[k] + i;
      __m256i by = _mm256_loadu_si256((const __m256i*)y->qs);
      __m256i sy = _mm256_sign_epi8(by, bx);
      __m256 p = _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_maddubs_epi16(ax, sy), _mm256_set1_epi16(1)));
      acc[k] = _mm256_fmadd_ps(_mm256_set1_ps(d * y->d), p, acc[k]);
    }
  }
  for (int k = 0; k < 4; k++) out[k] = hsum_f32(acc[k]);
}

// simd_avx2.rs:146-172 (Q4_K) and 195-222 (Q5_K).
AVX2 static inline __m256i qh_to_16(__m256i v, int bit) {
  __m256i s;
  switch (bit) {
    case 0: s = _mm256_slli_epi16(v, 4); break;
    case 1: s = _mm256_slli_epi16(v, 3); break;
    case 2: s = _mm256_slli_epi16(v, 2); break;
    case 3: s = _mm256_slli_epi16(v, 1); break;
    case 4: s = v; break;
    case 5: s = _mm256_srli_epi16(v, 1); break;
    case 6: s = _mm256_srli_epi16(v, 2); break;
    default: s = _mm256_srli_epi16(v, 3); break;
  }
  return _mm256_and_si256(s, _mm256_set1_epi8(0x10));
}

template <int Q5>
AVX2 static float a_k4(const uint8_t* w, const void* xv, size_t cols) {
  const BK* x = (const BK*)xv;
  const int SZ = Q5 ? 176 : 144;
  const __m256i m4 = _mm256_set1_epi8(0x0F);
  float sumf = 0.0f;
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * SZ;
    const BK* y = &x[i];
    float d = rd_f16(b) * y->d;
    float dmin = rd_f16(b + 2) * y->d;
    int16_t sc[8];
    int summ = 0;
    for (int j = 0; j < 8; j++) {
      int a, m;
      k4(j, b + 4, &a, &m);
      sc[j] = (int16_t)a;
      summ += m * ((int)y->bsums[2 * j] + (int)y->bsums[2 * j + 1]);
    }
    __m256i qh = _mm256_setzero_si256();
    if (Q5) qh = _mm256_loadu_si256((const __m256i*)(b + 16));
    const uint8_t* qs = b + (Q5 ? 48 : 16);
    __m256i sumi = _mm256_setzero_si256();
    for (int j = 0; j < 4; j++) {
      __m256i q = _mm256_loadu_si256((const __m256i*)(qs + 32 * j));
      __m256i lo = _mm256_and_si256(q, m4);
      __m256i hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), m4);
      if (Q5) {
        lo = _mm256_or_si256(lo, qh_to_16(qh, 2 * j));
        hi = _mm256_or_si256(hi, qh_to_16(qh, 2 * j + 1));
      }
      __m256i y0 = _mm256_loadu_si256((const __m256i*)(y->qs + 64 * j));
      __m256i y1 = _mm256_loadu_si256((const __m256i*)(y->qs + 64 * j + 32));
      __m256i p0 = _mm256_madd_epi16(_mm256_maddubs_epi16(lo, y0), _mm256_set1_epi16(sc[2 * j]));
      __m256i p1 = _mm256_madd_epi16(_mm256_maddubs_epi16(hi, y1), _mm256_set1_epi16(sc[2 * j + 1]));
      sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p0, p1));
    }
    sumf += d * (float)hsum_i32(sumi) - dmin * (float)summ;
  }
  return sumf;
}

// simd_avx2.rs:340-384
AVX2 static void a_q4_k_x4(const uint8_t* w, const void* const xs[4], size_t cols, float out[4]) {
  const __m256i m4 = _mm256_set1_epi8(0x0F);
  float sumf[4] = {0, 0, 0, 0};
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 144;
    float d = rd_f16(b), dmin = rd_f16(b + 2);
    int16_t sc[8];
    int mn[8];
    for (int j = 0; j < 8; j++) {
      int a, m;
      k4(j, b + 4, &a, &m);
      sc[j] = (int16_t)a;
      mn[j] = m;
    }
    const uint8_t* qs = b + 16;
    __m256i sumi[4] = {_mm256_setzero_si256(), _mm256_setzero_si256(), _mm256_setzero_si256(),
                       _mm256_setzero_si256()};
    for (int j = 0; j < 4; j++) {
      __m256i q = _mm256_loadu_si256((const __m256i*)(qs + 32 * j));
      __m256i lo = _mm256_and_si256(q, m4);
      __m256i hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), m4);
      __m256i s0 = _mm256_set1_epi16(sc[2 * j]), s1 = _mm256_set1_epi16(sc[2 * j + 1]);
      for (int k = 0; k < 4; k++) {
        const int8_t* yp = ((const BK*)xs[k])[i].qs;
        __m256i y0 = _mm256_loadu_si256((const __m256i*)(yp + 64 * j));
        __m256i y1 = _mm256_loadu_si256((const __m256i*)(yp + 64 * j + 32));
        __m256i p0 = _mm256_madd_epi16(_mm256_maddubs_epi16(lo, y0), s0);
        __m256i p1 = _mm256_madd_epi16(_mm256_maddubs_epi16(hi, y1), s1);
        sumi[k] = _mm256_add_epi32(sumi[k], _mm256_add_epi32(p0, p1));
      }
    }
    for (int k = 0; k < 4; k++) {
      const BK* y = &((const BK*)xs[k])[i];
      int summ = 0;
      for (int j = 0; j < 8; j++) summ += mn[j] * ((int)y->bsums[2 * j] + (int)y->bsums[2 * j + 1]);
      sumf[k] += (d * y->d) * (float)hsum_i32(sumi[k]) - (dmin * y->d) * (float)summ;
    }
  }
  for (int k = 0; k < 4; k++) out[k] = sumf[k];
}

// The four 32-value groups of one 128-value half of a Q6_K block as unsigned
// bytes 0..63 (simd_avx2.rs:250-257).
AVX2 static inline void q6_groups(const uint8_t* ql, const uint8_t* qh, __m256i qv[4]) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), m30 = _mm256_set1_epi8(0x30);
  __m256i ql0 = _mm256_loadu_si256((const __m256i*)ql);
  __m256i ql32 = _mm256_loadu_si256((const __m256i*)(ql + 32));
  __m256i h = _mm256_loadu_si256((const __m256i*)qh);
  qv[0] = _mm256_or_si256(_mm256_and_si256(ql0, m4), _mm256_and_si256(_mm256_slli_epi16(h, 4), m30));
  qv[1] = _mm256_or_si256(_mm256_and_si256(ql32, m4), _mm256_and_si256(_mm256_slli_epi16(h, 2), m30));
  qv[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(ql0, 4), m4), _mm256_and_si256(h, m30));
  qv[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(ql32, 4), m4), _mm256_and_si256(_mm256_srli_epi16(h, 2), m30));
}

// simd_avx2.rs:225-267: unsigned values, -32 applied through the block sums.
AVX2 static float a_q6_k(const uint8_t* w, const void* xv, size_t cols) {
  const BK* x = (const BK*)xv;
  float sumf = 0.0f;
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 210;
    const BK* y = &x[i];
    float d = rd_f16(b + 208) * y->d;
    const int8_t* scales = (const int8_t*)(b + 192);
    int bias = 0;
    for (int k = 0; k < 16; k++) bias += (int)scales[k] * (int)y->bsums[k];
    __m256i sumi = _mm256_setzero_si256();
    for (int n = 0; n < 2; n++) {
      const int8_t* sc = scales + 8 * n;
      const int8_t* yp = y->qs + 128 * n;
      __m256i qv[4];
      q6_groups(b + 64 * n, b + 128 + 32 * n, qv);
      for (int k = 0; k < 4; k++) {
        __m256i yv = _mm256_loadu_si256((const __m256i*)(yp + 32 * k));
        __m256i p16 = _mm256_maddubs_epi16(qv[k], yv);
        __m256i scv = _mm256_set_m128i(_mm_set1_epi16(sc[2 * k + 1]), _mm_set1_epi16(sc[2 * k]));
        sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(p16, scv));
      }
    }
    sumf += d * (float)(hsum_i32(sumi) - 32 * bias);
  }
  return sumf;
}

// simd_avx2.rs:387-430
AVX2 static void a_q6_k_x4(const uint8_t* w, const void* const xs[4], size_t cols, float out[4]) {
  float sumf[4] = {0, 0, 0, 0};
  for (size_t i = 0; i < cols / 256; i++) {
    const uint8_t* b = w + i * 210;
    float d = rd_f16(b + 208);
    const int8_t* scales = (const int8_t*)(b + 192);
    __m256i sumi[4] = {_mm256_setzero_si256(), _mm256_setzero_si256(), _mm256_setzero_si256(),
                       _mm256_setzero_si256()};
    for (int n = 0; n < 2; n++) {
      const int8_t* sc = scales + 8 * n;
      __m256i qv[4];
      q6_groups(b + 64 * n, b + 128 + 32 * n, qv);
      for (int kq = 0; kq < 4; kq++) {
        __m256i scv = _mm256_set_m128i(_mm_set1_epi16(sc[2 * kq + 1]), _mm_set1_epi16(sc[2 * kq]));
        for (int k = 0; k < 4; k++) {
          const int8_t* yp = ((const BK*)xs[k])[i].qs + 128 * n;
          __m256i yv = _mm256_loadu_si256((const __m256i*)(yp + 32 * kq));
          sumi[k] = _mm256_add_epi32(sumi[k], _mm256_madd_epi16(_mm256_maddubs_epi16(qv[kq], yv), scv));
        }
      }
    }
    for (int k = 0; k < 4; k++) {
      const BK* y = &((const BK*)xs[k])[i];
      int bias = 0;
      for (int j = 0; j < 16; j++) bias += (int)scales[j] * (int)y->bsums[j];
      sumf[k] += (d * y->d) * (float)(hsum_i32(sumi[k]) - 32 * bias);
    }
  }
  for (int k = 0; k < 4; k++) out[k] = sumf[k];
}

// simd_avx2.rs:433-493: eight fmadd lanes over groups of 8 columns, the fixed
// hsum tree, then an unfused sequential tail.
AVX2_F16C static float a_f16(const uint8_t* w, const void* xv, size_t n) {
  const float* x = (const float*)xv;
  __m256 acc = _mm256_setzero_ps();
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m128i h = _mm_loadu_si128((const __m128i*)(w + 2 * i));
    acc = _mm256_fmadd_ps(_mm256_cvtph_ps(h), _mm256_loadu_ps(x + i), acc);
  }
  float sum = hsum_f32(acc);
  for (; i < n; i++) sum += rd_f16(w + 2 * i) * x[i];
  return sum;
}

AVX2 static float a_bf16(const uint8_t* w, const void* xv, size_t n) {
  const float* x = (const float*)xv;
  __m256 acc = _mm256_setzero_ps();
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m128i h = _mm_loadu_si128((const __m128i*)(w + 2 * i));
    __m256 f = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(h), 16));
    acc = _mm256_fmadd_ps(f, _mm256_loadu_ps(x + i), acc);
  }
  float sum = hsum_f32(acc);
  for (; i < n; i++) sum += orc_bf16_to_f32(rd_u16(w + 2 * i)) * x[i];
  return sum;
}

AVX2 static float a_f32(const uint8_t* w, const void* xv, size_t n) {
  const float* x = (const float*)xv;
  __m256 acc = _mm256_setzero_ps();
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    acc = _mm256_fmadd_ps(_mm256_loadu_ps((const float*)(w + 4 * i)), _mm256_loadu_ps(x + i), acc);
  }
  float sum = hsum_f32(acc);
  for (; i < n; i++) sum += rd_f32(w + 4 * i) * x[i];
  return sum;
}

// ---------------------------------------------------------------------------
// Tables (matvec.rs:221-237, simd_avx2.rs:536-571)
// ---------------------------------------------------------------------------

orc_dot_fn orc_get_dot(int table, int kind) {
  if (table == ORC_SCALAR) {
    static const orc_dot_fn t[9] = {s_f32, s_f16, s_bf16, s_q4_0, s_q5_0, s_q8_0, s_q4_k, s_q5_k, s_q6_k};
    return t[kind];
  }
  switch (kind) {
    case ORC_F32: return a_f32;
    case ORC_F16: return table == ORC_AVX2_F16C ? a_f16 : s_f16;  // simd_avx2.rs:544
    case ORC_BF16: return a_bf16;
    case ORC_Q4_0: return a_q32<W_Q4_0, 18>;
    case ORC_Q5_0: return a_q32<W_Q5_0, 22>;
    case ORC_Q8_0: return a_q32<W_Q8_0, 34>;
    case ORC_Q4_K: return a_k4<0>;
    case ORC_Q5_K: return a_k4<1>;
    default: return a_q6_k;
  }
}

orc_dot4_fn orc_get_dot4(int table, int kind) {
  if (table == ORC_SCALAR) return NULL;
  switch (kind) {
    case ORC_Q4_0: return a_q32_x4<W_Q4_0, 18>;
    case ORC_Q5_0: return a_q32_x4<W_Q5_0, 22>;
    case ORC_Q8_0: return a_q32_x4<W_Q8_0, 34>;
    case ORC_Q4_K: return a_q4_k_x4;
    case ORC_Q6_K: return a_q6_k_x4;
    default: return NULL;  // matvec.rs:541-545: no x4 for Q5_K and the float kinds
  }
}

extern "C" {

int orc_table_supported(int table) {
  if (table == ORC_SCALAR) return 1;
  int ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  if (table == ORC_AVX2_F16C) ok = ok && __builtin_cpu_supports("f16c");
  return ok;
}

// matvec.rs:240-257
int orc_detect_table(void) {
  if (orc_table_supported(ORC_AVX2_F16C)) return ORC_AVX2_F16C;
  if (orc_table_supported(ORC_AVX2)) return ORC_AVX2;
  return ORC_SCALAR;
}

float orc_dot(int table, int kind, const uint8_t* w, const void* x, size_t cols) {
  return orc_get_dot(table, kind)(w, x, cols);
}

int orc_dot_x4(int table, int kind, const uint8_t* w, const void* x0, const void* x1, const void* x2,
               const void* x3, size_t cols, float out[4]) {
  orc_dot4_fn f = orc_get_dot4(table, kind);
  if (!f) return 0;
  const void* xs[4] = {x0, x1, x2, x3};
  f(w, xs, cols, out);
  return 1;
}

void orc_block_sums(int kind, const uint8_t* w, const void* x, size_t cols, int32_t* sumi, int32_t* summ) {
  size_t nb = cols / orc_block_size(kind);
  for (size_t i = 0; i < nb; i++) {
    int a = 0, m = 0;
    switch (kind) {
      case ORC_Q4_0: a = isum_q4_0(w + i * 18, (const B0*)x + i); break;
      case ORC_Q5_0: a = isum_q5_0(w + i * 22, (const B0*)x + i); break;
      case ORC_Q8_0: a = isum_q8_0(w + i * 34, (const B0*)x + i); break;
      case ORC_Q4_K: isum_k4(w + i * 144 + 4, NULL, w + i * 144 + 16, (const BK*)x + i, &a, &m); break;
      case ORC_Q5_K: isum_k4(w + i * 176 + 4, w + i * 176 + 16, w + i * 176 + 48, (const BK*)x + i, &a, &m); break;
      case ORC_Q6_K: a = isum_q6_k(w + i * 210, (const BK*)x + i); break;
      default: break;
    }
    sumi[i] = a;
    if (summ) summ[i] = m;
  }
}

}  // extern "C"
