// Batch-1 matrix-vector products over raw GGUF blocks (the matvec_* /
// matvec2_* / matvec3_* surface of crates/aot-kernels/src/matvec.rs:323-439).
//
// Shape of every kernel here: a CTA owns a contiguous share of the (possibly
// concatenated) row space, streams it tile by tile from HBM into a shared-
// memory ring with 1-D bulk copies (rows are contiguous in GGUF, so a tile of
// rows is one byte range), and threads decode blocks out of shared memory.
// The first tiles are requested before the kernel waits for its predecessor,
// because weights never depend on activations.
//
// Bit-exactness: each (row, block) item yields the f32 term of the reference
// (integers exact, mul/sub unfused); one thread per row then adds the terms in
// block order, which is the reference's `sumf += ...` loop.
#pragma once
#include <cuda_fp16.h>
#include "blockmath.cuh"
#include "device_utils.cuh"
#include "expf_exact.cuh"

namespace aot {

enum GemvEpilogue : int {
  EPI_STORE = 0,     // out[r] = v
  EPI_ACCUM = 1,     // out[r] = out[r] + v           (add_inplace of ops.rs:144-148 folded in)
  EPI_SILU_MUL = 2,  // pair mode: out[r] = silu(g)*u, out2[r] = u   (ops.rs:115-120)
};

struct GemvSeg {
  const uint8_t* w;
  float* out;
  int rows;
  int kind;
};

struct GemvParams {
  GemvSeg seg[3];
  int nseg;
  int pair;          // 1: seg0/seg1 are walked with the same row index (gate/up)
  int cols;
  int span_rows;     // size of the row space the grid splits (concat: sum of rows; pair: rows)
  int rows_per_cta;
  int tile_rows;     // rows of the row space per shared-memory tile
  int stage_bytes;   // bytes reserved per ring stage (multiple of 16)
  int n_stages;
  const void* x;     // activation vectors: block images, reference-layout blocks, or float[]
  int x_image;       // 1: 304-/48-byte block images, 0: BlockQ8_K / BlockQ8_0 as the reference lays them out
  int m;             // number of activation vectors (tokens); outputs are token-major, out[i*rows + r]
  int epilogue;
  int* err;
};

struct U4 {
  uint32_t x, y, z, w;
};
__device__ __forceinline__ U4 lds128(const void* p) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  return U4{v.x, v.y, v.z, v.w};
}
__device__ __forceinline__ uint32_t u4_get(const U4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Shared-memory image of one Q8_K activation block: qs at 0, bsums at 256, d at
// 288, stride 304 (19 x 16 bytes, odd, so 128-bit reads of different blocks by
// neighbouring lanes fall in different bank groups).
constexpr int XK_STRIDE = 304;
constexpr int XK_BSUMS = 256;
constexpr int XK_D = 288;
// Q8_0 activation block image: qs at 0, d at 32, stride 48.
constexpr int X0_STRIDE = 48;
constexpr int X0_D = 32;

__device__ __forceinline__ void load_x_q8k(uint8_t* sx, const void* g, int nb, int image) {
  if (image) {
    const uint4* src4 = reinterpret_cast<const uint4*>(g);
    for (int i = threadIdx.x; i < nb * (XK_STRIDE / 16); i += blockDim.x) reinterpret_cast<uint4*>(sx)[i] = src4[i];
    return;
  }
  const uint32_t* src = reinterpret_cast<const uint32_t*>(g);
  for (int i = threadIdx.x; i < nb * 73; i += blockDim.x) {
    int b = i / 73, w = i - b * 73;
    int off = w == 0 ? XK_D : (w <= 64 ? (w - 1) * 4 : XK_BSUMS + (w - 65) * 4);
    *reinterpret_cast<uint32_t*>(sx + b * XK_STRIDE + off) = src[i];
  }
}
__device__ __forceinline__ void load_x_q80(uint8_t* sx, const void* g, int nb, int image) {
  if (image) {
    const uint4* src4 = reinterpret_cast<const uint4*>(g);
    for (int i = threadIdx.x; i < nb * (X0_STRIDE / 16); i += blockDim.x) reinterpret_cast<uint4*>(sx)[i] = src4[i];
    return;
  }
  const uint32_t* src = reinterpret_cast<const uint32_t*>(g);
  for (int i = threadIdx.x; i < nb * 9; i += blockDim.x) {
    int b = i / 9, w = i - b * 9;
    int off = w == 0 ? X0_D : (w - 1) * 4;
    *reinterpret_cast<uint32_t*>(sx + b * X0_STRIDE + off) = src[i];
  }
}

__device__ __forceinline__ int dp2a_lo(uint32_t a, uint32_t b, int c) { return __dp2a_lo((int)a, (int)b, c); }
__device__ __forceinline__ int dp2a_hi(uint32_t a, uint32_t b, int c) { return __dp2a_hi((int)a, (int)b, c); }

// ---- one (row, block) term, K-quants ------------------------------------------
// wb: the weight block in shared memory (16-byte aligned for Q4_K/Q5_K, 2-byte
// aligned for Q6_K). xb: the Q8_K block image.
template <bool Q5>
__device__ __forceinline__ float term_k4(const uint8_t* wb, const uint8_t* xb) {
  U4 hdr = lds128(wb);
  K4Scales s = k4_unpack(hdr.y, hdr.z, hdr.w);
  float d_w = half_bits_to_float(hdr.x & 0xFFFFu), dmin_w = half_bits_to_float(hdr.x >> 16);
  U4 h0{0, 0, 0, 0}, h1{0, 0, 0, 0};
  const uint8_t* qs = wb + 16;
  if (Q5) {
    h0 = lds128(wb + 16);
    h1 = lds128(wb + 32);
    qs = wb + 48;
  }
  int sumi = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    U4 wa = lds128(qs + 32 * c), wc = lds128(qs + 32 * c + 16);
    U4 y0 = lds128(xb + 64 * c), y1 = lds128(xb + 64 * c + 16), y2 = lds128(xb + 64 * c + 32),
       y3 = lds128(xb + 64 * c + 48);
    int s_lo = 0, s_hi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      uint32_t w = i < 4 ? u4_get(wa, i) : u4_get(wc, i - 4);
      uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
      if (Q5) {
        uint32_t h = i < 4 ? u4_get(h0, i) : u4_get(h1, i - 4);
        lo |= ((h >> (2 * c)) & 0x01010101u) << 4;
        hi |= ((h >> (2 * c + 1)) & 0x01010101u) << 4;
      }
      uint32_t ylo = i < 4 ? u4_get(y0, i) : u4_get(y1, i - 4);
      uint32_t yhi = i < 4 ? u4_get(y2, i) : u4_get(y3, i - 4);
      s_lo = __dp4a((int)lo, (int)ylo, s_lo);
      s_hi = __dp4a((int)hi, (int)yhi, s_hi);
    }
    uint32_t scw = c < 2 ? s.sc_lo : s.sc_hi;
    sumi += byte_of(scw, (2 * c) & 3) * s_lo + byte_of(scw, (2 * c + 1) & 3) * s_hi;
  }
  // summ = sum_j m_j * (bsums[2j] + bsums[2j+1]): each bsums word holds one pair.
  U4 b0 = lds128(xb + XK_BSUMS), b1 = lds128(xb + XK_BSUMS + 16);
  uint32_t m01 = __byte_perm(s.m_lo, 0, 0x1100), m23 = __byte_perm(s.m_lo, 0, 0x3322);
  uint32_t m45 = __byte_perm(s.m_hi, 0, 0x1100), m67 = __byte_perm(s.m_hi, 0, 0x3322);
  int summ = 0;
  summ = dp2a_lo(b0.x, m01, summ);
  summ = dp2a_hi(b0.y, m01, summ);
  summ = dp2a_lo(b0.z, m23, summ);
  summ = dp2a_hi(b0.w, m23, summ);
  summ = dp2a_lo(b1.x, m45, summ);
  summ = dp2a_hi(b1.y, m45, summ);
  summ = dp2a_lo(b1.z, m67, summ);
  summ = dp2a_hi(b1.w, m67, summ);
  float d_x = *reinterpret_cast<const float*>(xb + XK_D);
  return k4_term(d_w, dmin_w, d_x, sumi, summ);
}

__device__ __forceinline__ float term_q6k(const uint8_t* wb, const uint8_t* xb, int* sumi_out = nullptr) {
  // Aligned word stream with a funnel shift for blocks that start 2 bytes into a word.
  const uint32_t sh = ((uint32_t)(uintptr_t)wb & 2u) * 8u;
  const uint32_t* p = reinterpret_cast<const uint32_t*>((uintptr_t)wb & ~(uintptr_t)3);
  auto wload = [&](int k) -> uint32_t { return funnel_r(p[k], p[k + 1], sh); };
  uint32_t scw[4] = {wload(48), wload(49), wload(50), wload(51)};
  int total = 0;
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      U4 y1 = lds128(xb + 128 * n + 16 * half), y2 = lds128(xb + 128 * n + 32 + 16 * half),
         y3 = lds128(xb + 128 * n + 64 + 16 * half), y4 = lds128(xb + 128 * n + 96 + 16 * half);
      int a1 = 0, a2 = 0, a3 = 0, a4 = 0;
#pragma unroll
      for (int ii = 0; ii < 4; ii++) {
        int i = 4 * half + ii;
        uint32_t l0 = wload(16 * n + i), l32 = wload(16 * n + 8 + i), h = wload(32 + 8 * n + i);
        uint32_t q1 = (l0 & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
        uint32_t q2 = (l32 & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
        uint32_t q3 = ((l0 >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
        uint32_t q4 = ((l32 >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
        a1 = __dp4a((int)q1, (int)u4_get(y1, ii), a1);
        a2 = __dp4a((int)q2, (int)u4_get(y2, ii), a2);
        a3 = __dp4a((int)q3, (int)u4_get(y3, ii), a3);
        a4 = __dp4a((int)q4, (int)u4_get(y4, ii), a4);
      }
      int g = 8 * n + half;
      total += (int)(int8_t)byte_of(scw[g >> 2], g & 3) * a1;
      total += (int)(int8_t)byte_of(scw[(g + 2) >> 2], (g + 2) & 3) * a2;
      total += (int)(int8_t)byte_of(scw[(g + 4) >> 2], (g + 4) & 3) * a3;
      total += (int)(int8_t)byte_of(scw[(g + 6) >> 2], (g + 6) & 3) * a4;
    }
  }
  // -32 * sum_g sc_g * bsums[g]
  U4 b0 = lds128(xb + XK_BSUMS), b1 = lds128(xb + XK_BSUMS + 16);
  int bias = 0;
  bias = dp2a_lo(b0.x, scw[0], bias);
  bias = dp2a_hi(b0.y, scw[0], bias);
  bias = dp2a_lo(b0.z, scw[1], bias);
  bias = dp2a_hi(b0.w, scw[1], bias);
  bias = dp2a_lo(b1.x, scw[2], bias);
  bias = dp2a_hi(b1.y, scw[2], bias);
  bias = dp2a_lo(b1.z, scw[3], bias);
  bias = dp2a_hi(b1.w, scw[3], bias);
  int sumi = total - 32 * bias;
  if (sumi_out) *sumi_out = sumi;
  float d_w = half_bits_to_float(wload(52) & 0xFFFFu);
  float d_x = *reinterpret_cast<const float*>(xb + XK_D);
  return q6k_term(d_w, d_x, sumi);
}

__device__ __forceinline__ float term_kq(int kind, const uint8_t* wb, const uint8_t* xb) {
  if (kind == Q4_K) return term_k4<false>(wb, xb);
  if (kind == Q5_K) return term_k4<true>(wb, xb);
  return term_q6k(wb, xb);
}

// ---- tile bookkeeping -----------------------------------------------------------
// A tile is up to three byte ranges ("parts"), one per weight matrix it touches.
struct TilePart {
  const uint8_t* src;  // first byte in global memory
  uint32_t len;        // bytes
  uint32_t soff;       // offset of the 16-byte aligned slot inside the stage
  int seg;
  int row0;            // first row inside the segment
  int rows;
};

// Parts of the tile that covers rows [t0, t1) of the row space.
template <class OpT>
__device__ __forceinline__ int tile_parts(const OpT& P, int t0, int t1, const size_t row_bytes[3], TilePart parts[3]) {
  int n = 0;
  uint32_t soff = 0;
  if (P.pair) {
    for (int s = 0; s < 2; s++) {
      TilePart& tp = parts[n++];
      tp.seg = s;
      tp.row0 = t0;
      tp.rows = t1 - t0;
      tp.src = P.seg[s].w + (size_t)t0 * row_bytes[s];
      tp.len = (uint32_t)((size_t)(t1 - t0) * row_bytes[s]);
      tp.soff = soff;
      soff += bulk_superset_bytes(tp.src, tp.len) + 16;
    }
    return n;
  }
  int base = 0;
  for (int s = 0; s < P.nseg; s++) {
    int a = max(t0, base), b = min(t1, base + P.seg[s].rows);
    if (a < b) {
      TilePart& tp = parts[n++];
      tp.seg = s;
      tp.row0 = a - base;
      tp.rows = b - a;
      tp.src = P.seg[s].w + (size_t)(a - base) * row_bytes[s];
      tp.len = (uint32_t)((size_t)(b - a) * row_bytes[s]);
      tp.soff = soff;
      soff += bulk_superset_bytes(tp.src, tp.len) + 16;
    }
    base += P.seg[s].rows;
  }
  return n;
}

__device__ __forceinline__ float silu_mul_exact(float g, float u) {
  // ops.rs:118-119: v / (1 + exp(-v)) * b
  return fmul(fdiv(g, fadd(1.0f, expf_exact(-g))), u);
}

// ---- K-quant products (Q8_K activations) ---------------------------------------------
// Shared memory: [stages][x image][terms 2 x nb x TRP][barriers]. With m > 1 (prompt
// batches, matmul_* of matvec.rs:479-546) the resident weight tile is applied to
// the m activation vectors one after the other; per token the arithmetic is the
// same code path as m == 1, so batched == single bit for bit.
#ifndef GEMV_THREADS_N
#define GEMV_THREADS_N 256
#endif
constexpr int GEMV_THREADS = GEMV_THREADS_N;
constexpr int GEMV_TRP = 64;  // max rows (over all parts) of one tile

struct TileCtx {
  int c0, c1, n_tiles;
  size_t row_bytes[3];
};

__device__ __forceinline__ void tile_ctx_init(const GemvParams& P, TileCtx& C) {
  for (int s = 0; s < 3; s++) C.row_bytes[s] = s < P.nseg ? kind_row_bytes(P.seg[s].kind, P.cols) : 0;
  C.c0 = blockIdx.x * P.rows_per_cta;
  C.c1 = min(C.c0 + P.rows_per_cta, P.span_rows);
  C.n_tiles = C.c1 > C.c0 ? (C.c1 - C.c0 + P.tile_rows - 1) / P.tile_rows : 0;
}

// Request tile t into its ring stage (one thread).
__device__ __forceinline__ void tile_issue(const GemvParams& P, TileCtx& C, uint8_t* stages, uint64_t* bars, int t) {
  TilePart parts[3];
  int t0 = C.c0 + t * P.tile_rows, t1 = min(t0 + P.tile_rows, C.c1);
  int np = tile_parts(P, t0, t1, C.row_bytes, parts);
  int st = t % P.n_stages;
  uint32_t total = 0;
  for (int i = 0; i < np; i++) total += bulk_superset_bytes(parts[i].src, parts[i].len);
  mbar_expect_tx(&bars[st], total);
  for (int i = 0; i < np; i++)
    bulk_g2s_superset(stages + (size_t)st * P.stage_bytes + parts[i].soff, parts[i].src, parts[i].len, &bars[st]);
}

__global__ void __launch_bounds__(GEMV_THREADS) gemv_q8k_kernel(const GemvParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int nb = P.cols / 256;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  float* terms = reinterpret_cast<float*>(sx + (size_t)nb * XK_STRIDE);
  uint64_t* bars = reinterpret_cast<uint64_t*>(terms + 2 * nb * GEMV_TRP);
  TileCtx C;
  tile_ctx_init(P, C);

  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int t = 0; t < min(C.n_tiles, P.n_stages); t++) tile_issue(P, C, stages, bars, t);
  }
  pdl_launch_dependents();
  // Everything above touches weights only; activations come from the previous kernel.
  pdl_wait();
  const size_t x_stride = (size_t)nb * (P.x_image ? XK_STRIDE : 292);
  if (P.m == 1) {
    load_x_q8k(sx, P.x, nb, P.x_image);
    __syncthreads();
  }

  int flip = 0;
  for (int t = 0; t < C.n_tiles; t++) {
    const int st = t % P.n_stages;
    const uint32_t parity = (uint32_t)(t / P.n_stages) & 1u;
    // Leave together if any thread gave up waiting, so nobody is left at a barrier.
    if (!__syncthreads_and(mbar_wait(&bars[st], parity, P.err) ? 1 : 0)) break;
    TilePart parts[3];
    const int t0 = C.c0 + t * P.tile_rows, t1 = min(t0 + P.tile_rows, C.c1);
    const int np = tile_parts(P, t0, t1, C.row_bytes, parts);
    const int R = t1 - t0;
    for (int tok = 0; tok < P.m; tok++) {
      if (P.m > 1) {
        __syncthreads();
        load_x_q8k(sx, reinterpret_cast<const uint8_t*>(P.x) + (size_t)tok * x_stride, nb, P.x_image);
        __syncthreads();
      }
      float* tt = terms + flip * nb * GEMV_TRP;
      flip ^= 1;
      int trow0 = 0;
      for (int i = 0; i < np; i++) {
        const TilePart& tp = parts[i];
        const int kind = P.seg[tp.seg].kind;
        const int bs = kind_size(kind);
        const uint8_t* base = stages + (size_t)st * P.stage_bytes + tp.soff + ((uintptr_t)tp.src & 15u);
        const int items = tp.rows * nb;
        for (int it = threadIdx.x; it < items; it += GEMV_THREADS) {
          int r = it / nb, b = it - r * nb;
          tt[b * GEMV_TRP + trow0 + r] = term_kq(kind, base + (size_t)it * bs, sx + b * XK_STRIDE);
        }
        trow0 += tp.rows;
      }
      __syncthreads();
      if (threadIdx.x == 0 && tok == P.m - 1 && t + P.n_stages < C.n_tiles) tile_issue(P, C, stages, bars, t + P.n_stages);
      // One thread per row adds the block terms in block order.
      if ((int)threadIdx.x < R) {
        if (P.pair) {
          float g = 0.0f, u = 0.0f;
          for (int b = 0; b < nb; b++) {
            g = fadd(g, tt[b * GEMV_TRP + threadIdx.x]);
            u = fadd(u, tt[b * GEMV_TRP + R + threadIdx.x]);
          }
          const size_t o = (size_t)tok * P.seg[0].rows + t0 + threadIdx.x;
          P.seg[0].out[o] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(g, u) : g;
          P.seg[1].out[o] = u;
        } else {
          float v = 0.0f;
          for (int b = 0; b < nb; b++) v = fadd(v, tt[b * GEMV_TRP + threadIdx.x]);
          int gr = t0 + threadIdx.x, s = 0;
          while (s < P.nseg - 1 && gr >= P.seg[s].rows) {
            gr -= P.seg[s].rows;
            s++;
          }
          float* o = P.seg[s].out + (size_t)tok * P.seg[s].rows + gr;
          *o = P.epilogue == EPI_ACCUM ? fadd(*o, v) : v;
        }
      }
    }
  }
}

// ---- Q4_0 / Q5_0 / Q8_0 products (Q8_0 activations) -------------------------------------
// Thread (row, kk) owns AVX2 lanes kk and kk+4 of the reference kernel (they read
// the same nibble bytes): per block acc = fma(d_w*d_x, float(p), acc) in block
// order (simd_avx2.rs:61-72), then the fixed 8-lane tree (simd_avx2.rs:29-34).
__device__ __forceinline__ uint32_t lds32_unaligned2(const uint8_t* p) {
  // p is 2-byte aligned.
  const uint32_t sh = ((uint32_t)(uintptr_t)p & 2u) * 8u;
  const uint32_t* q = reinterpret_cast<const uint32_t*>((uintptr_t)p & ~(uintptr_t)3);
  return sh ? funnel_r(q[0], q[1], sh) : q[0];
}
__device__ __forceinline__ uint32_t lds16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

__global__ void __launch_bounds__(GEMV_THREADS) gemv_q80_kernel(const GemvParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int nb = P.cols / 32;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  float* pairv = reinterpret_cast<float*>(sx + (((size_t)nb * X0_STRIDE + 15) & ~(size_t)15));  // 2 x TRP
  uint64_t* bars = reinterpret_cast<uint64_t*>(pairv + 2 * GEMV_TRP);
  TileCtx C;
  tile_ctx_init(P, C);

  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int t = 0; t < min(C.n_tiles, P.n_stages); t++) tile_issue(P, C, stages, bars, t);
  }
  pdl_launch_dependents();
  pdl_wait();
  const size_t x_stride = (size_t)nb * (P.x_image ? X0_STRIDE : 36);
  if (P.m == 1) {
    load_x_q80(sx, P.x, nb, P.x_image);
    __syncthreads();
  }

  const int kk = threadIdx.x & 3;
  const int rslot = threadIdx.x >> 2;  // 0..63: row slot inside the tile
  for (int t = 0; t < C.n_tiles; t++) {
    const int st = t % P.n_stages;
    const uint32_t parity = (uint32_t)(t / P.n_stages) & 1u;
    if (!__syncthreads_and(mbar_wait(&bars[st], parity, P.err) ? 1 : 0)) break;
    TilePart parts[3];
    const int t0 = C.c0 + t * P.tile_rows, t1 = min(t0 + P.tile_rows, C.c1);
    const int np = tile_parts(P, t0, t1, C.row_bytes, parts);
    const int R = t1 - t0;
    // This thread's row among the parts (pair mode: rows of both matrices).
    int trow = rslot, pi = -1;
    for (int i = 0; i < np; i++) {
      if (trow < parts[i].rows) {
        pi = i;
        break;
      }
      trow -= parts[i].rows;
    }
    for (int tok = 0; tok < P.m; tok++) {
      if (P.m > 1) {
        __syncthreads();
        load_x_q80(sx, reinterpret_cast<const uint8_t*>(P.x) + (size_t)tok * x_stride, nb, P.x_image);
        __syncthreads();
      }
      float acc_a = 0.0f, acc_b = 0.0f;
      if (pi >= 0) {
        const TilePart& tp = parts[pi];
        const int kind = P.seg[tp.seg].kind;
        const int bs = kind_size(kind);
        const uint8_t* rowp = stages + (size_t)st * P.stage_bytes + tp.soff + ((uintptr_t)tp.src & 15u) +
                              (size_t)trow * C.row_bytes[tp.seg];
        for (int b = 0; b < nb; b++) {
          const uint8_t* wb = rowp + (size_t)b * bs;
          const uint8_t* xb = sx + b * X0_STRIDE;
          float d = fmul(half_bits_to_float(lds16(wb)), *reinterpret_cast<const float*>(xb + X0_D));
          uint32_t ya = *reinterpret_cast<const uint32_t*>(xb + 4 * kk);
          uint32_t yb = *reinterpret_cast<const uint32_t*>(xb + 16 + 4 * kk);
          int pa, pb;
          if (kind == Q8_0) {
            pa = q8_0_lane(lds32_unaligned2(wb + 2 + 4 * kk), ya);
            pb = q8_0_lane(lds32_unaligned2(wb + 18 + 4 * kk), yb);
          } else if (kind == Q4_0) {
            uint32_t q = lds32_unaligned2(wb + 2 + 4 * kk);
            pa = q4_0_lane(q, kk, ya);
            pb = q4_0_lane(q, kk + 4, yb);
          } else {
            uint32_t qh = lds32_unaligned2(wb + 2);
            uint32_t q = lds32_unaligned2(wb + 6 + 4 * kk);
            pa = q5_0_lane(q, qh, kk, ya);
            pb = q5_0_lane(q, qh, kk + 4, yb);
          }
          acc_a = ffma(d, i2f(pa), acc_a);
          acc_b = ffma(d, i2f(pb), acc_b);
        }
      }
      // ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)): the four threads of a row are
      // neighbours in one warp; every lane takes part (idle rows carry zeros).
      float s04 = fadd(acc_a, acc_b);
      float tsum = fadd(s04, __shfl_xor_sync(0xffffffffu, s04, 2));
      float v = fadd(tsum, __shfl_xor_sync(0xffffffffu, tsum, 1));
      if (pi >= 0 && kk == 0) {
        const TilePart& tp = parts[pi];
        if (P.pair) {
          pairv[pi * GEMV_TRP + trow] = v;
        } else {
          float* o = P.seg[tp.seg].out + (size_t)tok * P.seg[tp.seg].rows + tp.row0 + trow;
          *o = P.epilogue == EPI_ACCUM ? fadd(*o, v) : v;
        }
      }
      __syncthreads();
      if (threadIdx.x == 0 && tok == P.m - 1 && t + P.n_stages < C.n_tiles) tile_issue(P, C, stages, bars, t + P.n_stages);
      if (P.pair) {
        if ((int)threadIdx.x < R) {
          float g = pairv[threadIdx.x], u = pairv[GEMV_TRP + threadIdx.x];
          const size_t o = (size_t)tok * P.seg[0].rows + t0 + threadIdx.x;
          P.seg[0].out[o] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(g, u) : g;
          P.seg[1].out[o] = u;
        }
        __syncthreads();
      }
    }
  }
}

// ---- F32 / F16 / BF16 products (f32 activations) --------------------------------------------
// Thread (row, k) owns AVX2 lane k: acc = fma(w[8j+k], x[8j+k], acc) over j in order
// (simd_avx2.rs:433-493), the 8-lane tree, then the unfused scalar tail. Weights
// are read straight from global memory.
__device__ __forceinline__ float load_wf(int kind, const uint8_t* wrow, int j) {
  if (kind == F32) return __ldg(reinterpret_cast<const float*>(wrow) + j);
  const unsigned short h = __ldg(reinterpret_cast<const unsigned short*>(wrow) + j);
  // both conversions are exact (every f16 / bf16 value is an f32 value)
  return kind == F16 ? __half2float(__ushort_as_half(h)) : __uint_as_float((uint32_t)h << 16);
}

// One AVX2 lane chain of a row: acc = fma(w[j], x[j], acc) for j = k, k+8, ... below n8.
// Weights are requested 32 steps ahead of the adds so that enough bytes are in flight.
template <int KIND>
__device__ __forceinline__ float float_lane_chain(const uint8_t* wrow, const float* x, int k, int n8) {
  float acc = 0.0f;
  int j = k;
  for (; j + 8 * 31 < n8; j += 8 * 32) {
    float w[32];
#pragma unroll
    for (int u = 0; u < 32; u++) w[u] = load_wf(KIND, wrow, j + 8 * u);
#pragma unroll
    for (int u = 0; u < 32; u++) acc = ffma(w[u], x[j + 8 * u], acc);
  }
  for (; j < n8; j += 8) acc = ffma(load_wf(KIND, wrow, j), x[j], acc);
  return acc;
}

// The same lane chain for TG activation rows at once: the weights of 16 steps are loaded
// once and applied to every row's own accumulator, each in the order of the single-row chain.
template <int KIND, int TG>
__device__ __forceinline__ void float_lane_chain_multi(const uint8_t* wrow, const float* x, int cols, int k, int n8, int ntok,
                                                       float (&acc)[TG]) {
#pragma unroll
  for (int t = 0; t < TG; t++) acc[t] = 0.0f;
  int j = k;
  for (; j + 8 * 15 < n8; j += 8 * 16) {
    float w[16];
#pragma unroll
    for (int u = 0; u < 16; u++) w[u] = load_wf(KIND, wrow, j + 8 * u);
#pragma unroll
    for (int t = 0; t < TG; t++) {
      if (t < ntok) {
        const float* xt = x + (size_t)t * cols + j;
#pragma unroll
        for (int u = 0; u < 16; u++) acc[t] = ffma(w[u], xt[8 * u], acc[t]);
      }
    }
  }
  for (; j < n8; j += 8) {
    const float w = load_wf(KIND, wrow, j);
#pragma unroll
    for (int t = 0; t < TG; t++)
      if (t < ntok) acc[t] = ffma(w, x[(size_t)t * cols + j], acc[t]);
  }
}

constexpr int FLOAT_TG = 8;  // activation rows handled per pass over a weight row

__global__ void __launch_bounds__(256) gemv_float_kernel(const GemvParams P) {
  pdl_launch_dependents();
  pdl_wait();
  const int k = threadIdx.x & 7;
  const int rows_per_block = blockDim.x >> 3;
  const int n8 = P.cols & ~7;
  // Whole warps (4 rows) stay in or leave the loop together, so the shuffles below
  // always see all 32 lanes.
  for (int gr = blockIdx.x * rows_per_block + (threadIdx.x >> 3); gr < ((P.span_rows + 3) & ~3);
       gr += gridDim.x * rows_per_block) {
    const bool live = gr < P.span_rows;
    int s = 0, r = gr;
    if (live && !P.pair) {
      while (s < P.nseg - 1 && r >= P.seg[s].rows) {
        r -= P.seg[s].rows;
        s++;
      }
    }
    if (P.m == 1) {
      const float* x = reinterpret_cast<const float*>(P.x);
      float res[2] = {0.0f, 0.0f};
      const int nmat = P.pair ? 2 : 1;
      for (int mi = 0; mi < nmat; mi++) {
        const int sg = P.pair ? mi : s;
        const int kind = P.seg[sg].kind;
        const uint8_t* wrow = P.seg[sg].w + (size_t)(live ? r : 0) * kind_row_bytes(kind, P.cols);
        float acc = 0.0f;
        if (live) {
          if (kind == F16) acc = float_lane_chain<F16>(wrow, x, k, n8);
          else if (kind == BF16) acc = float_lane_chain<BF16>(wrow, x, k, n8);
          else acc = float_lane_chain<F32>(wrow, x, k, n8);
        }
        float s1 = fadd(acc, __shfl_xor_sync(0xffffffffu, acc, 4));  // a_k + a_{k+4}
        float t1 = fadd(s1, __shfl_xor_sync(0xffffffffu, s1, 2));
        float sum = fadd(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
        if (live && k == 0) {
          for (int j = n8; j < P.cols; j++) sum = fadd(sum, fmul(load_wf(kind, wrow, j), x[j]));
        }
        res[mi] = sum;
      }
      if (live && k == 0) {
        if (P.pair) {
          P.seg[0].out[r] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(res[0], res[1]) : res[0];
          P.seg[1].out[r] = res[1];
        } else {
          float* o = P.seg[s].out + r;
          *o = P.epilogue == EPI_ACCUM ? fadd(*o, res[0]) : res[0];
        }
      }
      continue;
    }
    // several activation rows: groups of FLOAT_TG rows share one pass over the weight row
    for (int tok0 = 0; tok0 < P.m; tok0 += FLOAT_TG) {
      const int ntok = min(FLOAT_TG, P.m - tok0);
      const float* x = reinterpret_cast<const float*>(P.x) + (size_t)tok0 * P.cols;
      float res[2][FLOAT_TG];
      const int nmat = P.pair ? 2 : 1;
      for (int mi = 0; mi < nmat; mi++) {
        const int sg = P.pair ? mi : s;
        const int kind = P.seg[sg].kind;
        const uint8_t* wrow = P.seg[sg].w + (size_t)(live ? r : 0) * kind_row_bytes(kind, P.cols);
        float acc[FLOAT_TG];
#pragma unroll
        for (int t = 0; t < FLOAT_TG; t++) acc[t] = 0.0f;
        if (live) {
          if (kind == F16) float_lane_chain_multi<F16, FLOAT_TG>(wrow, x, P.cols, k, n8, ntok, acc);
          else if (kind == BF16) float_lane_chain_multi<BF16, FLOAT_TG>(wrow, x, P.cols, k, n8, ntok, acc);
          else float_lane_chain_multi<F32, FLOAT_TG>(wrow, x, P.cols, k, n8, ntok, acc);
        }
#pragma unroll
        for (int t = 0; t < FLOAT_TG; t++) {
          float s1 = fadd(acc[t], __shfl_xor_sync(0xffffffffu, acc[t], 4));  // a_k + a_{k+4}
          float t1 = fadd(s1, __shfl_xor_sync(0xffffffffu, s1, 2));
          float sum = fadd(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
          if (live && k == 0 && t < ntok) {
            for (int j = n8; j < P.cols; j++) sum = fadd(sum, fmul(load_wf(kind, wrow, j), x[(size_t)t * P.cols + j]));
          }
          res[mi][t] = sum;
        }
      }
      if (live && k == 0) {
#pragma unroll
        for (int t = 0; t < FLOAT_TG; t++) {
          if (t < ntok) {
            const int tok = tok0 + t;
            if (P.pair) {
              const size_t o = (size_t)tok * P.seg[0].rows + r;
              P.seg[0].out[o] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(res[0][t], res[1][t]) : res[0][t];
              P.seg[1].out[o] = res[1][t];
            } else {
              float* o = P.seg[s].out + (size_t)tok * P.seg[s].rows + r;
              *o = P.epilogue == EPI_ACCUM ? fadd(*o, res[0][t]) : res[0][t];
            }
          }
        }
      }
    }
  }
}

}  // namespace aot
