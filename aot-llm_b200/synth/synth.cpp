// Synthetic weights for tests and benchmarks (host code, no part of the forward
// pass): the valid-but-not-optimal GGUF block encoders of
// crates/aot-kernels/src/quantize.rs restated, a counter-based uniform generator
// so tensors can be filled by many threads with a reproducible result, and a
// field-uniform block filler for single-kernel benchmarks.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/aot_cuda.h"
#include "../csrc/blockmath.cuh"
#include "aot_synth.h"

using namespace aot;

namespace {

// f32 -> binary16, round to nearest even (crates/aot-kernels/src/quant.rs:127-161).
uint16_t f32_to_f16(float f) {
  uint32_t x = f2u(f);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  int e = (int)((x >> 23) & 0xFFu);
  uint32_t mant = x & 0x7FFFFFu;
  if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0u));
  e -= 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e < -25) return sign;
  if (e < -14) {
    uint32_t m = mant | 0x800000u;
    uint32_t shift = (uint32_t)(-14 - e) + 13u;
    uint32_t half = 1u << (shift - 1), rem = m & ((1u << shift) - 1u), r = m >> shift;
    if (rem > half || (rem == half && (r & 1u))) r++;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(e + 15) << 10) | (mant >> 13), rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
  return (uint16_t)(sign | r);
}

uint16_t f32_to_bf16(float f) {
  uint32_t x = f2u(f);
  if ((x & 0x7F800000u) == 0x7F800000u) return (uint16_t)((x >> 16) | ((x & 0x7FFFFFu) ? 0x40u : 0u));
  return (uint16_t)((x + 0x7FFFu + ((x >> 16) & 1u)) >> 16);
}

inline void put16(uint8_t* p, uint16_t v) {
  p[0] = (uint8_t)v;
  p[1] = (uint8_t)(v >> 8);
}
inline int nearest(float x) { return (int)roundf(x); }
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Signed extreme of a group: first value with strictly larger magnitude.
inline float signed_extreme(const float* x, int n) {
  float amax = 0.0f, mx = 0.0f;
  for (int i = 0; i < n; i++) {
    float a = fabsf(x[i]);
    if (a > amax) {
      amax = a;
      mx = x[i];
    }
  }
  return mx;
}

// quantize.rs:16-41
void enc_q4_0(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 32; b++, x += 32, out += 18) {
    float d = signed_extreme(x, 32) / -8.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    put16(out, f32_to_f16(d));
    for (int j = 0; j < 16; j++) {
      int lo = clampi(nearest(x[j] * id) + 8, 0, 15), hi = clampi(nearest(x[j + 16] * id) + 8, 0, 15);
      out[2 + j] = (uint8_t)(lo | (hi << 4));
    }
  }
}

// quantize.rs:44-74
void enc_q5_0(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 32; b++, x += 32, out += 22) {
    float d = signed_extreme(x, 32) / -16.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint32_t qh = 0;
    for (int j = 0; j < 16; j++) {
      uint32_t lo = (uint32_t)clampi(nearest(x[j] * id) + 16, 0, 31), hi = (uint32_t)clampi(nearest(x[j + 16] * id) + 16, 0, 31);
      out[6 + j] = (uint8_t)((lo & 0xF) | ((hi & 0xF) << 4));
      qh |= (lo >> 4) << j;
      qh |= (hi >> 4) << (j + 16);
    }
    put16(out, f32_to_f16(d));
    memcpy(out + 2, &qh, 4);
  }
}

// quantize.rs:77-91
void enc_q8_0(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 32; b++, x += 32, out += 34) {
    float amax = 0.0f;
    for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(x[j]));
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    put16(out, f32_to_f16(d));
    for (int j = 0; j < 32; j++) out[2 + j] = (uint8_t)(int8_t)clampi(nearest(x[j] * id), -127, 127);
  }
}

// quantize.rs:95-166: shared body of the Q4_K / Q5_K encoders.
void enc_k4_block(const float* blk, float qmax, float* d_out, float* dmin_out, uint8_t sc12[12], uint8_t q[256]) {
  float scales[8], mins[8];
  for (int j = 0; j < 8; j++) {
    float lo = 3.402823466e+38f, hi = -3.402823466e+38f;
    for (int l = 0; l < 32; l++) {
      lo = fminf(lo, blk[32 * j + l]);
      hi = fmaxf(hi, blk[32 * j + l]);
    }
    float mn = fmaxf(-lo, 0.0f);
    scales[j] = fmaxf((hi + mn) / qmax, 0.0f);
    mins[j] = mn;
  }
  float max_scale = 0.0f, max_min = 0.0f;
  for (int j = 0; j < 8; j++) {
    max_scale = fmaxf(max_scale, scales[j]);
    max_min = fmaxf(max_min, mins[j]);
  }
  float d = max_scale / 63.0f, dmin = max_min / 63.0f;
  float inv_d = d != 0.0f ? 1.0f / d : 0.0f, inv_m = dmin != 0.0f ? 1.0f / dmin : 0.0f;
  uint8_t ls[8], lm[8];
  for (int j = 0; j < 8; j++) {
    ls[j] = (uint8_t)clampi(nearest(scales[j] * inv_d), 0, 63);
    lm[j] = (uint8_t)clampi(nearest(mins[j] * inv_m), 0, 63);
  }
  d = half_bits_to_float(f32_to_f16(d));
  dmin = half_bits_to_float(f32_to_f16(dmin));
  for (int j = 0; j < 8; j++) {
    float sc = d * (float)ls[j], m = dmin * (float)lm[j];
    float inv = sc != 0.0f ? 1.0f / sc : 0.0f;
    for (int l = 0; l < 32; l++) q[32 * j + l] = (uint8_t)clampi(nearest((blk[32 * j + l] + m) * inv), 0, (int)qmax);
  }
  memset(sc12, 0, 12);
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      sc12[j] |= ls[j];
      sc12[j + 4] |= lm[j];
    } else {
      sc12[j + 4] = (uint8_t)((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
      sc12[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
      sc12[j] |= (uint8_t)((lm[j] >> 4) << 6);
    }
  }
  *d_out = d;
  *dmin_out = dmin;
}

// quantize.rs:169-184
void enc_q4_k(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 256; b++, x += 256, out += 144) {
    float d, dmin;
    uint8_t q[256];
    enc_k4_block(x, 15.0f, &d, &dmin, out + 4, q);
    put16(out, f32_to_f16(d));
    put16(out + 2, f32_to_f16(dmin));
    for (int j = 0; j < 4; j++)
      for (int l = 0; l < 32; l++) out[16 + 32 * j + l] = (uint8_t)(q[64 * j + l] | (q[64 * j + 32 + l] << 4));
  }
}

// quantize.rs:187-217
void enc_q5_k(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 256; b++, x += 256, out += 176) {
    float d, dmin;
    uint8_t q[256];
    enc_k4_block(x, 31.0f, &d, &dmin, out + 4, q);
    put16(out, f32_to_f16(d));
    put16(out + 2, f32_to_f16(dmin));
    uint8_t* qh = out + 16;
    uint8_t* qs = out + 48;
    memset(qh, 0, 32);
    for (int j = 0; j < 4; j++) {
      for (int l = 0; l < 32; l++) {
        uint8_t a = q[64 * j + l], c = q[64 * j + 32 + l];
        qs[32 * j + l] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
        if (a & 16) qh[l] |= (uint8_t)(1u << (2 * j));
        if (c & 16) qh[l] |= (uint8_t)(2u << (2 * j));
      }
    }
  }
}

// quantize.rs:220-278
void enc_q6_k(const float* x, size_t n, uint8_t* out) {
  for (size_t b = 0; b < n / 256; b++, x += 256, out += 210) {
    float scales[16];
    for (int j = 0; j < 16; j++) scales[j] = signed_extreme(x + 16 * j, 16) / -32.0f;
    float max_scale = signed_extreme(scales, 16);
    float iscale = max_scale != 0.0f ? -128.0f / max_scale : 0.0f;
    float d = half_bits_to_float(f32_to_f16(1.0f / iscale));
    int8_t ls[16];
    uint8_t q[256];
    for (int j = 0; j < 16; j++) ls[j] = (int8_t)clampi(nearest(iscale * scales[j]), -128, 127);
    for (int j = 0; j < 16; j++) {
      float sc = d * (float)ls[j];
      float inv = sc != 0.0f ? 1.0f / sc : 0.0f;
      for (int l = 0; l < 16; l++) q[16 * j + l] = (uint8_t)(clampi(nearest(x[16 * j + l] * inv), -32, 31) + 32);
    }
    uint8_t* ql = out;
    uint8_t* qh = out + 128;
    for (int h = 0; h < 2; h++) {
      for (int l = 0; l < 32; l++) {
        uint8_t q1 = q[128 * h + l], q2 = q[128 * h + l + 32], q3 = q[128 * h + l + 64], q4 = q[128 * h + l + 96];
        ql[64 * h + l] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
        ql[64 * h + l + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
        qh[32 * h + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
      }
    }
    memcpy(out + 192, ls, 16);
    put16(out + 208, f32_to_f16(d));
  }
}

void encode_row(int kind, const float* x, size_t n, uint8_t* out) {
  switch (kind) {
    case F32: memcpy(out, x, n * 4); break;
    case F16: for (size_t i = 0; i < n; i++) put16(out + 2 * i, f32_to_f16(x[i])); break;
    case BF16: for (size_t i = 0; i < n; i++) put16(out + 2 * i, f32_to_bf16(x[i])); break;
    case Q4_0: enc_q4_0(x, n, out); break;
    case Q5_0: enc_q5_0(x, n, out); break;
    case Q8_0: enc_q8_0(x, n, out); break;
    case Q4_K: enc_q4_k(x, n, out); break;
    case Q5_K: enc_q5_k(x, n, out); break;
    default: enc_q6_k(x, n, out); break;
  }
}

// splitmix64 of (seed, index): a counter-based generator, so any element can be
// produced independently of the others.
inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
inline float uniform_pm1(uint64_t seed, uint64_t idx) {
  uint64_t r = mix64(seed * 0xD1342543DE82EF95ULL + idx);
  // 24 random bits -> [0,1) -> (-1,1)
  return (float)(r >> 40) * (1.0f / 16777216.0f) * 2.0f - 1.0f;
}

template <class F>
void parallel_rows(size_t rows, F f) {
  unsigned nt = std::thread::hardware_concurrency();
  nt = nt < 1 ? 1 : (nt > 32 ? 32 : nt);
  if (rows < 64) nt = 1;
  std::vector<std::thread> th;
  for (unsigned t = 0; t < nt; t++) {
    th.emplace_back([=]() {
      size_t a = rows * t / nt, b = rows * (t + 1) / nt;
      for (size_t r = a; r < b; r++) f(r);
    });
  }
  for (auto& x : th) x.join();
}

}  // namespace

extern "C" {

int aotcu_synth_quantize_row(int kind, const float* x, size_t n, uint8_t* out) {
  if (kind < 0 || kind >= N_KINDS || !x || !out || n % (size_t)kind_block(kind) != 0) return AOTCU_ERR_BAD_ARG;
  encode_row(kind, x, n, out);
  return 0;
}

int aotcu_synth_tensor(int kind, size_t rows, size_t cols, float amp, float offset, uint64_t seed, uint8_t* out) {
  if (kind < 0 || kind >= N_KINDS || !out || cols % (size_t)kind_block(kind) != 0) return AOTCU_ERR_BAD_ARG;
  size_t rb = kind_row_bytes(kind, cols);
  parallel_rows(rows, [=](size_t r) {
    std::vector<float> x(cols);
    for (size_t c = 0; c < cols; c++) x[c] = offset + amp * uniform_pm1(seed, r * cols + c);
    encode_row(kind, x.data(), cols, out + r * rb);
  });
  return 0;
}

int aotcu_synth_blocks(int kind, size_t n_blocks, uint64_t seed, uint8_t* out) {
  if (kind < AOTCU_Q4_0 || kind > AOTCU_Q6_K || !out) return AOTCU_ERR_BAD_ARG;
  const size_t bs = (size_t)kind_size(kind);
  parallel_rows(n_blocks, [=](size_t b) {
    uint8_t* p = out + b * bs;
    uint64_t ctr = b * 64;
    for (size_t i = 0; i < bs; i += 8) {
      uint64_t r = mix64(seed * 0xD1342543DE82EF95ULL + ctr++);
      memcpy(p + i, &r, bs - i < 8 ? bs - i : 8);
    }
    // f16 scales uniform in [1e-3, 1e-2]
    auto scale = [&]() {
      uint64_t r = mix64(seed * 0xD1342543DE82EF95ULL + ctr++);
      float u = (float)(r >> 40) * (1.0f / 16777216.0f);
      return f32_to_f16(1e-3f + u * 9e-3f);
    };
    if (kind == Q6_K) {
      put16(p + 208, scale());
    } else {
      put16(p, scale());
      if (kind == Q4_K || kind == Q5_K) put16(p + 2, scale());
    }
  });
  return 0;
}

}  // extern "C"
