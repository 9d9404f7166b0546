// Oracle (test infrastructure): helpers shared by the oracle's translation units.
#pragma once
#include <string.h>

#include "oracle.h"

// Little-endian field reads; weight bytes are never cast to structs because
// GGUF rows carry no alignment guarantee (crates/aot-kernels/src/quant.rs:3-7).
static inline uint16_t rd_u16(const uint8_t* p) {
  uint16_t v;
  memcpy(&v, p, 2);
  return v;
}
static inline uint32_t rd_u32(const uint8_t* p) {
  uint32_t v;
  memcpy(&v, p, 4);
  return v;
}
static inline float rd_f32(const uint8_t* p) {
  float v;
  memcpy(&v, p, 4);
  return v;
}
static inline float rd_f16(const uint8_t* p) { return orc_f16_to_f32(rd_u16(p)); }

enum orc_act { ORC_ACT_F32 = 0, ORC_ACT_Q8_0 = 1, ORC_ACT_Q8_K = 2 };

// crates/aot-codegen/src/model.rs:88-95
static inline int orc_activation(int kind) {
  if (kind == ORC_Q4_0 || kind == ORC_Q5_0 || kind == ORC_Q8_0) return ORC_ACT_Q8_0;
  if (kind == ORC_Q4_K || kind == ORC_Q5_K || kind == ORC_Q6_K) return ORC_ACT_Q8_K;
  return ORC_ACT_F32;
}

typedef float (*orc_dot_fn)(const uint8_t* w, const void* x, size_t cols);
typedef void (*orc_dot4_fn)(const uint8_t* w, const void* const xs[4], size_t cols, float out[4]);

orc_dot_fn orc_get_dot(int table, int kind);
orc_dot4_fn orc_get_dot4(int table, int kind);

// Fork-join pool (crates/aot-kernels/src/pool.rs).
#ifdef __cplusplus
#include <functional>
void orc_pool_run(orc_pool* p, const std::function<void(int, int)>& f);
void orc_pool_run_chunks(orc_pool* p, size_t n, size_t chunk, const std::function<void(size_t, size_t)>& f);
static inline void orc_split(size_t n, int tid, int nth, size_t* a, size_t* b) {
  size_t chunk = (n + (size_t)nth - 1) / (size_t)nth;
  size_t s = (size_t)tid * chunk, e = ((size_t)tid + 1) * chunk;
  *a = s < n ? s : n;
  *b = e < n ? e : n;
}
#endif
