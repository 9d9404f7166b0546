// Prompt chunks: K-quant weight matrices applied to m (8..64) activation rows at once with
// int8 tensor-core tiles (the reference's batched micro-kernels, crates/aot-kernels/src/
// matvec.rs:412-560, which reuse one decoded weight block for several tokens).
//
// Bit-identity with the one-token product comes for free: inside a 256-weight super-block
// everything is integer arithmetic (exact in any order), and the f32 block terms are added in
// block order per (row, token) by the one thread that owns that output element.
//
// A CTA works on one group of 16 tokens (two MMA column groups) whose Q8_K images it stages
// in shared memory once, and on TPC row tiles of 16 weight rows at a time; the KS warps of a
// tile split the tile's super-blocks between them. For every 32-weight sub-block (16-weight
// for Q6_K) a warp issues one mma.sync m16n8k32 (m16n8k16) u8 x s8 -> s32 per column group,
// starting from zero: the per-sub-block scale differs per row, so the accumulator has to be
// read out after every K = 32 and is folded into the block's integer sum with one integer
// multiply-add per output element. Each warp leaves the f32 term of each of its blocks in
// shared memory; after a barrier the terms of an output element are added in block order.
// Weight nibbles are unpacked in registers straight from global memory, fetched one block
// ahead (each 32-byte sector is used completely by the quad that reads it).
#pragma once
#include <cuda_fp16.h>

#include "blockmath.cuh"
#include "device_utils.cuh"
#include "gemv.cuh"

namespace aot {

constexpr int GEMM_WARPS = 8;   // warps per CTA
constexpr int GEMM_MAX_KB = 8;  // super-blocks per staged activation chunk, at most
constexpr int GEMM_MAX_M = 64;

struct GemmParams {
  GemvSeg seg[3];
  int nseg, pair, cols, m, epilogue;
  const uint8_t* x;   // [m][cols/256] Q8_K images (304 bytes) or reference-layout BlockQ8_K (292 bytes)
  int x_image;
  int n_groups;       // token groups of 16 tokens; CTA c works on group c % n_groups
  int n_tiles;        // 16-row tiles over all matrices (pair mode: of one matrix)
  int ks;             // warps that split one tile's super-blocks (a divisor of the CTA's warps)
  int kc;             // super-blocks staged at a time (all of them when they fit)
  int tiles_before[4];  // first tile index of each matrix (pair mode: one list for both)
};

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Loads from a shared-space address.
__device__ __forceinline__ uint32_t gm_lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void gm_lds64(uint32_t a, uint32_t& x, uint32_t& y) {
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a));
}
__device__ __forceinline__ U4 gm_lds128(uint32_t a) {
  U4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// A 32-bit word at a 2-byte aligned global address.
__device__ __forceinline__ uint32_t ldg32_a2(const uint8_t* p) {
  if (((uintptr_t)p & 2u) == 0) return __ldg(reinterpret_cast<const uint32_t*>(p));
  const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
  return (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
}

// The words of one super-block that a thread needs for its two rows (row g and row g+8 of
// the tile; g = lane/4, q = lane%4), fetched one block ahead of their use.
//   Q4_K / Q5_K: [0..3] d|dmin + packed scales, [4..11] nibble words (pair c: 4+2c holds
//                weights k = 8q..8q+3, 5+2c k = 8q+4..8q+7), [12..13] fifth-bit words (Q5_K)
//   Q6_K:        [0..3] low nibbles l, [4..7] low nibbles l+32, [8..11] high bits
//                (index 2n+hh), [12..15] scales, [16] d
struct WFrag {
  uint32_t w[2][17];
};

__device__ __forceinline__ void gemm_load_frag(int kind, const uint8_t* wa, const uint8_t* wb, WFrag& f) {
  const int q = threadIdx.x & 3;
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const uint8_t* p = r ? wb : wa;
    if (kind == Q6_K) {
#pragma unroll
      for (int i = 0; i < 4; i++) {  // i = 2n + hh
        const int lo = 64 * (i >> 1) + 16 * (i & 1) + 4 * q;
        f.w[r][i] = ldg32_a2(p + lo);
        f.w[r][4 + i] = ldg32_a2(p + lo + 32);
        f.w[r][8 + i] = ldg32_a2(p + 128 + 32 * (i >> 1) + 16 * (i & 1) + 4 * q);
        f.w[r][12 + i] = ldg32_a2(p + 192 + 4 * i);
      }
      f.w[r][16] = ldg32_a2(p + 206) >> 16;
    } else {
      const uint4 h = __ldg(reinterpret_cast<const uint4*>(p));
      f.w[r][0] = h.x; f.w[r][1] = h.y; f.w[r][2] = h.z; f.w[r][3] = h.w;
      const int qoff = kind == Q5_K ? 48 : 16;
      // lane q takes bytes 8q..8q+7 of every 32-byte nibble run: weights k = 8q..8q+7 of both
      // sub-blocks of the pair (the activation fragment uses the same k order)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p + qoff + 32 * c) + q);
        f.w[r][4 + 2 * c] = v.x;
        f.w[r][5 + 2 * c] = v.y;
      }
      if (kind == Q5_K) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p + 16) + q);
        f.w[r][12] = v.x;
        f.w[r][13] = v.y;
      }
    }
  }
}

// One 16-row tile of one matrix against NT token groups: adds the f32 term of one
// super-block into acc.v[t][i] (i: 0 = row g / token 2q, 1 = row g / token 2q+1, 2 = row
// g+8 / token 2q, 3 = row g+8 / token 2q+1). Called in block order.
// `xs` is the shared-space address of the block's images, layout [token][304].
template <int NT>
struct TileAcc {
  float v[NT][4];
};

template <int NT, bool Q5>
__device__ __forceinline__ void gemm_block_k4(const WFrag& f, uint32_t xs, int tok0, TileAcc<NT>& acc) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const K4Scales sa = k4_unpack(f.w[0][1], f.w[0][2], f.w[0][3]), sb = k4_unpack(f.w[1][1], f.w[1][2], f.w[1][3]);
  int sumi[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int i = 0; i < 4; i++) sumi[t][i] = 0;
  }
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const uint32_t qa0 = f.w[0][4 + 2 * c], qa1 = f.w[0][5 + 2 * c], qb0 = f.w[1][4 + 2 * c], qb1 = f.w[1][5 + 2 * c];
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
      const int j = 2 * c + hi;  // sub-block
      uint32_t a0 = (hi ? qa0 >> 4 : qa0) & 0x0F0F0F0Fu, a2 = (hi ? qa1 >> 4 : qa1) & 0x0F0F0F0Fu;
      uint32_t a1 = (hi ? qb0 >> 4 : qb0) & 0x0F0F0F0Fu, a3 = (hi ? qb1 >> 4 : qb1) & 0x0F0F0F0Fu;
      if (Q5) {
        a0 |= ((f.w[0][12] >> j) & 0x01010101u) << 4;
        a2 |= ((f.w[0][13] >> j) & 0x01010101u) << 4;
        a1 |= ((f.w[1][12] >> j) & 0x01010101u) << 4;
        a3 |= ((f.w[1][13] >> j) & 0x01010101u) << 4;
      }
      const int sca = byte_of(j < 4 ? sa.sc_lo : sa.sc_hi, j & 3), scb = byte_of(j < 4 ? sb.sc_lo : sb.sc_hi, j & 3);
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const uint32_t xa = xs + (uint32_t)(tok0 + 8 * t + g) * XK_STRIDE + 32 * j + 8 * q;
        uint32_t y0, y1;
        gm_lds64(xa, y0, y1);  // activations k = 8q..8q+3 and 8q+4..8q+7, matching the weight words
        int cc[4];
        mma_u8s8_k32(cc, a0, a1, a2, a3, y0, y1);
        sumi[t][0] += sca * cc[0];
        sumi[t][1] += sca * cc[1];
        sumi[t][2] += scb * cc[2];
        sumi[t][3] += scb * cc[3];
      }
    }
  }
  // mins x activation sub-block sums (each sub-block is two 16-element sums of the image)
  const uint32_t ma01 = __byte_perm(sa.m_lo, 0, 0x1100), ma23 = __byte_perm(sa.m_lo, 0, 0x3322);
  const uint32_t ma45 = __byte_perm(sa.m_hi, 0, 0x1100), ma67 = __byte_perm(sa.m_hi, 0, 0x3322);
  const uint32_t mb01 = __byte_perm(sb.m_lo, 0, 0x1100), mb23 = __byte_perm(sb.m_lo, 0, 0x3322);
  const uint32_t mb45 = __byte_perm(sb.m_hi, 0, 0x1100), mb67 = __byte_perm(sb.m_hi, 0, 0x3322);
  const float da = half_bits_to_float((uint16_t)(f.w[0][0] & 0xFFFFu)), dmina = half_bits_to_float((uint16_t)(f.w[0][0] >> 16));
  const float db = half_bits_to_float((uint16_t)(f.w[1][0] & 0xFFFFu)), dminb = half_bits_to_float((uint16_t)(f.w[1][0] >> 16));
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {  // the thread's two tokens of this group
      const uint32_t xt = xs + (uint32_t)(tok0 + 8 * t + 2 * q + e) * XK_STRIDE;
      const U4 b0 = gm_lds128(xt + XK_BSUMS), b1 = gm_lds128(xt + XK_BSUMS + 16);
      int sma = 0, smb = 0;
      sma = dp2a_lo(b0.x, ma01, sma); sma = dp2a_hi(b0.y, ma01, sma);
      sma = dp2a_lo(b0.z, ma23, sma); sma = dp2a_hi(b0.w, ma23, sma);
      sma = dp2a_lo(b1.x, ma45, sma); sma = dp2a_hi(b1.y, ma45, sma);
      sma = dp2a_lo(b1.z, ma67, sma); sma = dp2a_hi(b1.w, ma67, sma);
      smb = dp2a_lo(b0.x, mb01, smb); smb = dp2a_hi(b0.y, mb01, smb);
      smb = dp2a_lo(b0.z, mb23, smb); smb = dp2a_hi(b0.w, mb23, smb);
      smb = dp2a_lo(b1.x, mb45, smb); smb = dp2a_hi(b1.y, mb45, smb);
      smb = dp2a_lo(b1.z, mb67, smb); smb = dp2a_hi(b1.w, mb67, smb);
      const float dx = __uint_as_float(gm_lds32(xt + XK_D));
      acc.v[t][e] = fadd(acc.v[t][e], k4_term(da, dmina, dx, sumi[t][e], sma));
      acc.v[t][2 + e] = fadd(acc.v[t][2 + e], k4_term(db, dminb, dx, sumi[t][2 + e], smb));
    }
  }
}

// Q6_K: sixteen 16-weight sub-blocks with signed 8-bit scales. Weights are used as
// 0..63 and the -32 offset goes through the activation sums (see blockmath.cuh).
template <int NT>
__device__ __forceinline__ void gemm_block_q6k(const WFrag& f, uint32_t xs, int tok0, TileAcc<NT>& acc) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  int sumi[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int i = 0; i < 4; i++) sumi[t][i] = 0;
  }
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      const int i4 = 2 * n + hh;
      const uint32_t la0 = f.w[0][i4], la32 = f.w[0][4 + i4], hqa = f.w[0][8 + i4];
      const uint32_t lb0 = f.w[1][i4], lb32 = f.w[1][4 + i4], hqb = f.w[1][8 + i4];
#pragma unroll
      for (int qu = 0; qu < 4; qu++) {  // quarter of the 128-weight half
        const uint32_t la = (qu & 1) ? la32 : la0, lb = (qu & 1) ? lb32 : lb0;
        const uint32_t a0 = (((qu & 2) ? la >> 4 : la) & 0x0F0F0F0Fu) | (((hqa >> (2 * qu)) & 0x03030303u) << 4);
        const uint32_t a1 = (((qu & 2) ? lb >> 4 : lb) & 0x0F0F0F0Fu) | (((hqb >> (2 * qu)) & 0x03030303u) << 4);
        const int s = 8 * n + hh + 2 * qu;  // sub-block
        const int ca = (int)(int8_t)byte_of(f.w[0][12 + (s >> 2)], s & 3), cb = (int)(int8_t)byte_of(f.w[1][12 + (s >> 2)], s & 3);
        const int yoff = 128 * n + 32 * qu + 16 * hh + 4 * q;
#pragma unroll
        for (int t = 0; t < NT; t++) {
          const uint32_t xa = xs + (uint32_t)(tok0 + 8 * t + g) * XK_STRIDE + yoff;
          int cc[4];
          mma_u8s8_k16(cc, a0, a1, gm_lds32(xa));
          sumi[t][0] += ca * cc[0];
          sumi[t][1] += ca * cc[1];
          sumi[t][2] += cb * cc[2];
          sumi[t][3] += cb * cc[3];
        }
      }
    }
  }
  const float da = half_bits_to_float((uint16_t)f.w[0][16]), db = half_bits_to_float((uint16_t)f.w[1][16]);
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const uint32_t xt = xs + (uint32_t)(tok0 + 8 * t + 2 * q + e) * XK_STRIDE;
      const U4 b0 = gm_lds128(xt + XK_BSUMS), b1 = gm_lds128(xt + XK_BSUMS + 16);
      int ba = 0, bb = 0;
      ba = dp2a_lo(b0.x, f.w[0][12], ba); ba = dp2a_hi(b0.y, f.w[0][12], ba);
      ba = dp2a_lo(b0.z, f.w[0][13], ba); ba = dp2a_hi(b0.w, f.w[0][13], ba);
      ba = dp2a_lo(b1.x, f.w[0][14], ba); ba = dp2a_hi(b1.y, f.w[0][14], ba);
      ba = dp2a_lo(b1.z, f.w[0][15], ba); ba = dp2a_hi(b1.w, f.w[0][15], ba);
      bb = dp2a_lo(b0.x, f.w[1][12], bb); bb = dp2a_hi(b0.y, f.w[1][12], bb);
      bb = dp2a_lo(b0.z, f.w[1][13], bb); bb = dp2a_hi(b0.w, f.w[1][13], bb);
      bb = dp2a_lo(b1.x, f.w[1][14], bb); bb = dp2a_hi(b1.y, f.w[1][14], bb);
      bb = dp2a_lo(b1.z, f.w[1][15], bb); bb = dp2a_hi(b1.w, f.w[1][15], bb);
      const float dx = __uint_as_float(gm_lds32(xt + XK_D));
      acc.v[t][e] = fadd(acc.v[t][e], q6k_term(da, dx, sumi[t][e] - 32 * ba));
      acc.v[t][2 + e] = fadd(acc.v[t][2 + e], q6k_term(db, dx, sumi[t][2 + e] - 32 * bb));
    }
  }
}

template <int NT>
__device__ __forceinline__ void gemm_block(int kind, const WFrag& f, uint32_t xs, int tok0, TileAcc<NT>& acc) {
  if (kind == Q4_K) gemm_block_k4<NT, false>(f, xs, tok0, acc);
  else if (kind == Q6_K) gemm_block_q6k<NT>(f, xs, tok0, acc);
  else gemm_block_k4<NT, true>(f, xs, tok0, acc);
}

// Stage the activation images of super-blocks [b0, b0 + kb_n) for tokens [t0, t0 + nt8) into
// `dst` ([kb][slot][304]); slots beyond token m-1 repeat the last token (their results are
// dropped).
__device__ __forceinline__ void gemm_stage_x(uint32_t dst, const uint8_t* x, int x_image, int nb, int b0, int kb_n, int t0,
                                             int nt8, int m) {
  if (x_image) {
    const int pieces = kb_n * nt8 * (XK_STRIDE / 16);
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
      const int kb = i / (nt8 * (XK_STRIDE / 16)), r = i - kb * (nt8 * (XK_STRIDE / 16));
      const int slot = r / (XK_STRIDE / 16), p = r - slot * (XK_STRIDE / 16);
      const int ts = min(t0 + slot, m - 1);
      cp_async16(dst + (uint32_t)((kb * nt8 + slot) * XK_STRIDE + 16 * p),
                 x + ((size_t)ts * nb + (size_t)(b0 + kb)) * XK_STRIDE + 16 * p);
    }
  } else {
    // BlockQ8_K {f32 d; i8 qs[256]; i16 bsums[16]} (quant.rs:8-14), word by word into the image
    // layout, with plain loads (four in flight per thread)
    const int pieces = kb_n * nt8 * 73;
    for (int i0 = threadIdx.x; i0 < pieces; i0 += 4 * blockDim.x) {
      uint32_t v[4];
      uint32_t da[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + u * blockDim.x;
        if (i < pieces) {
          const int kb = i / (nt8 * 73), r = i - kb * (nt8 * 73);
          const int slot = r / 73, w = r - slot * 73;
          const int ts = min(t0 + slot, m - 1);
          const int off = w == 0 ? XK_D : (w <= 64 ? (w - 1) * 4 : XK_BSUMS + (w - 65) * 4);
          da[u] = dst + (uint32_t)((kb * nt8 + slot) * XK_STRIDE + off);
          v[u] = __ldg(reinterpret_cast<const uint32_t*>(x + ((size_t)ts * nb + (size_t)(b0 + kb)) * 292) + w);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (i0 + u * (int)blockDim.x < pieces) asm volatile("st.shared.u32 [%0], %1;" ::"r"(da[u]), "r"(v[u]) : "memory");
      }
    }
  }
}

constexpr int GEMM_NT = 2;             // MMA column groups (of 8 tokens) per CTA
constexpr int GEMM_TOK = 8 * GEMM_NT;  // tokens per CTA

template <bool PAIR>
__global__ void __launch_bounds__(GEMM_WARPS * 32, 2) gemm_q8k_mma_kernel(const GemmParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int NT = GEMM_NT, NT8 = GEMM_TOK, n_mat = PAIR ? 2 : 1, EPL = NT * 4;  // EPL: outputs per lane
  const int nb = P.cols >> 8, kc = P.kc;
  const int n_chunks = (nb + kc - 1) / kc;
  const int n_warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int ks = P.ks, tpc = n_warps / ks;   // k-parts per tile, tiles per CTA
  const int tile_i = warp / ks, part = warp - tile_i * ks;
  // [images: kc x 16 tokens x 304][terms: tpc x n_mat x kc x 256 floats]
  const uint32_t ximg = smem_addr(smem);
  float* terms = reinterpret_cast<float*>(smem + (size_t)kc * NT8 * XK_STRIDE);
  const int tg = (int)blockIdx.x % P.n_groups, cta_in_group = (int)blockIdx.x / P.n_groups;
  const int ctas_per_group = (int)gridDim.x / P.n_groups;
  const int tokg = tg * NT8;  // first token of the group
  const int per_round = ctas_per_group * tpc;
  const int n_rounds = (P.n_tiles + per_round - 1) / per_round;
  const int per_part = EPL / ks > 0 ? EPL / ks : 1;  // outputs per lane this warp sums
  pdl_launch_dependents();
  for (int round = 0; round < n_rounds; round++) {
    const int tile_raw = (round * ctas_per_group + cta_in_group) * tpc + tile_i;
    const bool active = tile_raw < P.n_tiles;
    const int tile = active ? tile_raw : 0;
    int s = 0;
    if (!PAIR) {
      while (s < P.nseg - 1 && tile >= P.tiles_before[s + 1]) s++;
    }
    const int r0 = (tile - P.tiles_before[s]) * 16;
    // rows of this thread (clamped: a ragged last tile recomputes the last row)
    const uint8_t* wrow[n_mat][2];
    int kind[n_mat];
    uint32_t rbytes[n_mat];
#pragma unroll
    for (int mt = 0; mt < n_mat; mt++) {
      const GemvSeg& sg = P.seg[PAIR ? mt : s];
      kind[mt] = sg.kind;
      rbytes[mt] = (uint32_t)kind_size(sg.kind);
      const size_t row_bytes = (size_t)rbytes[mt] * nb;
      wrow[mt][0] = sg.w + (size_t)min(r0 + g, sg.rows - 1) * row_bytes;
      wrow[mt][1] = sg.w + (size_t)min(r0 + g + 8, sg.rows - 1) * row_bytes;
    }
    // Within a chunk of kc super-blocks this warp takes blocks part, part + ks, ...;
    // weights are fetched one (block, matrix) step ahead of their use, across chunks too.
    WFrag cur, nxt;
    if (active && part < nb) gemm_load_frag(kind[0], wrow[0][0] + (size_t)part * rbytes[0], wrow[0][1] + (size_t)part * rbytes[0], cur);
    float sum0[EPL], sum1[EPL];  // running sums of this thread's outputs (first / second matrix)
#pragma unroll
    for (int e = 0; e < EPL; e++) sum0[e] = sum1[e] = 0.0f;
    for (int ch = 0; ch < n_chunks; ch++) {
      const int b0 = ch * kc, b1 = min(b0 + kc, nb);
      // Weights do not depend on the previous kernel; activations and outputs do.
      if (round == 0 && ch == 0) pdl_wait();
      if (n_chunks > 1 || round == 0) {
        // (with one chunk the images of the token group stay for all rounds)
        gemm_stage_x(ximg, P.x, P.x_image, nb, b0, b1 - b0, tokg, NT8, P.m);
        cp_async_commit();
        cp_async_wait<0>();
      }
      __syncthreads();  // images are in place; the terms of the previous chunk have been consumed
      if (active) {
        for (int b = b0 + part; b < b1; b += ks) {
          const uint32_t xb = ximg + (uint32_t)((b - b0) * NT8) * XK_STRIDE;
#pragma unroll
          for (int mt = 0; mt < n_mat; mt++) {
            int nbk = b;
            if (mt + 1 == n_mat) {
              nbk = b + ks;
              if (nbk >= b1) nbk = b1 + part;  // first block of this warp in the next chunk
            }
            const int nmt = mt + 1 < n_mat ? mt + 1 : 0;
            if (nbk < nb)
              gemm_load_frag(kind[nmt], wrow[nmt][0] + (size_t)nbk * rbytes[nmt], wrow[nmt][1] + (size_t)nbk * rbytes[nmt], nxt);
            TileAcc<NT> term;
#pragma unroll
            for (int t = 0; t < NT; t++) {
#pragma unroll
              for (int i = 0; i < 4; i++) term.v[t][i] = 0.0f;
            }
            gemm_block<NT>(kind[mt], cur, xb, 0, term);
            float4* dst = reinterpret_cast<float4*>(terms + ((size_t)(tile_i * n_mat + mt) * kc + (b - b0)) * (32 * EPL) + lane * EPL);
#pragma unroll
            for (int t = 0; t < NT; t++) dst[t] = make_float4(term.v[t][0], term.v[t][1], term.v[t][2], term.v[t][3]);
            cur = nxt;
          }
        }
      }
      __syncthreads();  // all terms of the chunk are written; the images may be replaced
      if (active) {
        // The terms of an output element are added in block order by one thread; the ks
        // warps of a tile share the tile's outputs.
#pragma unroll
        for (int e = 0; e < EPL; e++) {
          if (e >= part * per_part && e < (part + 1) * per_part) {
            const float* tp = terms + (size_t)(tile_i * n_mat) * kc * (32 * EPL) + lane * EPL + e;
            for (int b = 0; b < b1 - b0; b++) {
              sum0[e] = fadd(sum0[e], tp[(size_t)b * (32 * EPL)]);
              if (PAIR) sum1[e] = fadd(sum1[e], tp[(size_t)(kc + b) * (32 * EPL)]);
            }
          }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int e = 0; e < EPL; e++) {
        if (e >= part * per_part && e < (part + 1) * per_part) {
          const int t = e >> 2, i = e & 3;
          const int row = r0 + g + (i >> 1) * 8, tok = tokg + 8 * t + 2 * q + (i & 1);
          const GemvSeg& sg = P.seg[PAIR ? 0 : s];
          if (row < sg.rows && tok < P.m) {
            const size_t o = (size_t)tok * sg.rows + row;
            if (PAIR) {
              P.seg[0].out[o] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(sum0[e], sum1[e]) : sum0[e];
              P.seg[1].out[o] = sum1[e];
            } else {
              sg.out[o] = P.epilogue == EPI_ACCUM ? fadd(sg.out[o], sum0[e]) : sum0[e];
            }
          }
        }
      }
    }
  }
}

}  // namespace aot
