// Oracle (test infrastructure): block layouts, half-float conversion, activation
// quantizers and row dequantizers. Restates crates/aot-kernels/src/quant.rs.
#include <math.h>
#include <string.h>

#include "oracle_internal.h"

extern "C" {

// quant.rs:46-72
size_t orc_block_size(int kind) {
  switch (kind) {
    case ORC_F32: case ORC_F16: case ORC_BF16: return 1;
    case ORC_Q4_0: case ORC_Q5_0: case ORC_Q8_0: return 32;
    default: return 256;
  }
}

size_t orc_type_size(int kind) {
  static const size_t sz[9] = {4, 2, 2, 18, 22, 34, 144, 176, 210};
  return sz[kind];
}

// quant.rs:70-72
size_t orc_row_bytes(int kind, size_t n) { return n / orc_block_size(kind) * orc_type_size(kind); }

// quant.rs:96-125. Subnormal halves are normalised by shifting until the
// implicit bit appears.
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) {
      bits = sign;
    } else {
      int ex = 113;
      while ((m & 0x400u) == 0) {
        m <<= 1;
        ex -= 1;
      }
      bits = sign | ((uint32_t)ex << 23) | ((m & 0x3FFu) << 13);
    }
  } else if (e == 31) {
    bits = sign | 0x7F800000u | (m << 13);
  } else {
    bits = sign | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

// quant.rs:127-161: round to nearest even, overflow to infinity, flush below
// 2^-25 to zero.
uint16_t orc_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  int e = (int)((x >> 23) & 0xFFu);
  uint32_t mant = x & 0x7FFFFFu;
  if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant != 0 ? 0x200u : 0u));
  e -= 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e < -25) return sign;
  if (e < -14) {
    uint32_t m = mant | 0x800000u;
    uint32_t shift = (uint32_t)(-14 - e) + 13u;
    uint32_t half = 1u << (shift - 1);
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t r = m >> shift;
    if (rem > half || (rem == half && (r & 1u))) r += 1;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(e + 15) << 10) | (mant >> 13);
  uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r += 1;
  return (uint16_t)(sign | r);
}

// quant.rs:163-177
float orc_bf16_to_f32(uint16_t h) {
  uint32_t b = (uint32_t)h << 16;
  float f;
  memcpy(&f, &b, 4);
  return f;
}

uint16_t orc_f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7F800000u) == 0x7F800000u) return (uint16_t)((x >> 16) | ((x & 0x7FFFFFu) ? 0x40u : 0u));
  uint32_t lsb = (x >> 16) & 1u;
  return (uint16_t)((x + 0x7FFFu + lsb) >> 16);
}

// quant.rs:224-228: f32::round is half-away-from-zero, `as i32` saturates.
static inline int round_i(float x) { return (int)roundf(x); }

// quant.rs:231-245
void orc_quantize_q8_0(const float* x, size_t n, orc_block_q8_0* out) {
  size_t nb = n / 32;
  for (size_t i = 0; i < nb; i++) {
    const float* src = x + i * 32;
    float amax = 0.0f;
    for (int j = 0; j < 32; j++) {
      float a = fabsf(src[j]);
      // f32::max ignores a NaN operand.
      if (a > amax || amax != amax) amax = a;
    }
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    out[i].d = d;
    for (int j = 0; j < 32; j++) {
      int q = round_i(src[j] * id);
      q = q < -127 ? -127 : (q > 127 ? 127 : q);
      out[i].qs[j] = (int8_t)q;
    }
  }
}

// quant.rs:248-283
void orc_quantize_q8_k(const float* x, size_t n, orc_block_q8_k* out) {
  size_t nb = n / 256;
  for (size_t i = 0; i < nb; i++) {
    const float* src = x + i * 256;
    orc_block_q8_k* blk = &out[i];
    float amax = 0.0f, mx = 0.0f;
    for (int j = 0; j < 256; j++) {
      float a = fabsf(src[j]);
      if (a > amax) {
        amax = a;
        mx = src[j];
      }
    }
    if (amax == 0.0f) {
      memset(blk, 0, sizeof(*blk));
      continue;
    }
    float iscale = -127.0f / mx;
    for (int j = 0; j < 256; j++) {
      int q = round_i(iscale * src[j]);
      if (q > 127) q = 127;
      blk->qs[j] = (int8_t)q;
    }
    for (int j = 0; j < 16; j++) {
      int s = 0;
      for (int k = 0; k < 16; k++) s += blk->qs[j * 16 + k];
      blk->bsums[j] = (int16_t)s;
    }
    blk->d = 1.0f / iscale;
  }
}

// quant.rs:292-298
void orc_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// quant.rs:300-443, one function per kind.
void orc_dequant_row(int kind, const uint8_t* row, float* out, size_t n) {
  switch (kind) {
    case ORC_F32:
      for (size_t i = 0; i < n; i++) out[i] = rd_f32(row + 4 * i);
      break;
    case ORC_F16:
      for (size_t i = 0; i < n; i++) out[i] = rd_f16(row + 2 * i);
      break;
    case ORC_BF16:
      for (size_t i = 0; i < n; i++) out[i] = orc_bf16_to_f32(rd_u16(row + 2 * i));
      break;
    case ORC_Q4_0:
      for (size_t i = 0; i < n / 32; i++) {
        const uint8_t* b = row + i * 18;
        float* o = out + i * 32;
        float d = rd_f16(b);
        for (int j = 0; j < 16; j++) {
          uint8_t q = b[2 + j];
          o[j] = (float)((int)(q & 0x0F) - 8) * d;
          o[j + 16] = (float)((int)(q >> 4) - 8) * d;
        }
      }
      break;
    case ORC_Q5_0:
      for (size_t i = 0; i < n / 32; i++) {
        const uint8_t* b = row + i * 22;
        float* o = out + i * 32;
        float d = rd_f16(b);
        uint32_t qh = rd_u32(b + 2);
        for (int j = 0; j < 16; j++) {
          uint8_t q = b[6 + j];
          uint32_t lo = (uint32_t)(q & 0x0F) | (((qh >> j) & 1u) << 4);
          uint32_t hi = (uint32_t)(q >> 4) | (((qh >> (j + 16)) & 1u) << 4);
          o[j] = (float)((int)lo - 16) * d;
          o[j + 16] = (float)((int)hi - 16) * d;
        }
      }
      break;
    case ORC_Q8_0:
      for (size_t i = 0; i < n / 32; i++) {
        const uint8_t* b = row + i * 34;
        float* o = out + i * 32;
        float d = rd_f16(b);
        for (int j = 0; j < 32; j++) o[j] = (float)(int8_t)b[2 + j] * d;
      }
      break;
    case ORC_Q4_K:
      for (size_t i = 0; i < n / 256; i++) {
        const uint8_t* b = row + i * 144;
        float* o = out + i * 256;
        float d = rd_f16(b), dmin = rd_f16(b + 2);
        const uint8_t* scales = b + 4;
        const uint8_t* qs = b + 16;
        for (int j = 0; j < 4; j++) {
          uint8_t sc1, m1, sc2, m2;
          orc_scale_min_k4(2 * j, scales, &sc1, &m1);
          orc_scale_min_k4(2 * j + 1, scales, &sc2, &m2);
          float d1 = d * (float)sc1, d2 = d * (float)sc2;
          float mm1 = dmin * (float)m1, mm2 = dmin * (float)m2;
          for (int l = 0; l < 32; l++) {
            uint8_t q = qs[32 * j + l];
            o[64 * j + l] = d1 * (float)(q & 0xF) - mm1;
            o[64 * j + 32 + l] = d2 * (float)(q >> 4) - mm2;
          }
        }
      }
      break;
    case ORC_Q5_K:
      for (size_t i = 0; i < n / 256; i++) {
        const uint8_t* b = row + i * 176;
        float* o = out + i * 256;
        float d = rd_f16(b), dmin = rd_f16(b + 2);
        const uint8_t* scales = b + 4;
        const uint8_t* qh = b + 16;
        const uint8_t* qs = b + 48;
        for (int j = 0; j < 4; j++) {
          uint8_t sc1, m1, sc2, m2;
          orc_scale_min_k4(2 * j, scales, &sc1, &m1);
          orc_scale_min_k4(2 * j + 1, scales, &sc2, &m2);
          float d1 = d * (float)sc1, d2 = d * (float)sc2;
          float mm1 = dmin * (float)m1, mm2 = dmin * (float)m2;
          uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
          for (int l = 0; l < 32; l++) {
            uint8_t q = qs[32 * j + l];
            int h1 = (qh[l] & u1) ? 16 : 0;
            int h2 = (qh[l] & u2) ? 16 : 0;
            o[64 * j + l] = d1 * (float)((q & 0xF) + h1) - mm1;
            o[64 * j + 32 + l] = d2 * (float)((q >> 4) + h2) - mm2;
          }
        }
      }
      break;
    case ORC_Q6_K:
      for (size_t i = 0; i < n / 256; i++) {
        const uint8_t* b = row + i * 210;
        float* o = out + i * 256;
        float d = rd_f16(b + 208);
        for (int h = 0; h < 2; h++) {
          const uint8_t* ql = b + 64 * h;
          const uint8_t* qh = b + 128 + 32 * h;
          const int8_t* sc = (const int8_t*)(b + 192 + 8 * h);
          float* y = o + 128 * h;
          for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l] = d * (float)sc[is] * (float)q1;
            y[l + 32] = d * (float)sc[is + 2] * (float)q2;
            y[l + 64] = d * (float)sc[is + 4] * (float)q3;
            y[l + 96] = d * (float)sc[is + 6] * (float)q4;
          }
        }
      }
      break;
  }
}

}  // extern "C"
