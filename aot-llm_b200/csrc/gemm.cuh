// Prompt chunks: K-quant weight matrices applied to m (8..64) activation rows at once with
// int8 tensor-core tiles (the reference's batched micro-kernels, crates/aot-kernels/src/
// matvec.rs:412-560, which reuse one decoded weight block for several tokens).
//
// Bit-identity with the one-token product comes for free: inside a 256-weight super-block
// everything is integer arithmetic (exact in any order), and the f32 block terms are added in
// block order per (row, token) by the one thread that owns that output element.
//
// A warp owns a tile of 16 weight rows and NT groups of 8 tokens. For every 32-weight
// sub-block (16-weight for Q6_K) it issues one mma.sync m16n8k32 (m16n8k16) u8 x s8 -> s32
// per token group, starting from zero: the per-sub-block scale differs per row, so the
// accumulator has to be read out after every K = 32 and is folded into the block's integer
// sum with one integer multiply-add per output element. Weight nibbles are unpacked in
// registers straight from global memory (each 32-byte sector is used completely by the
// quad that reads it); the activation images of the current K chunk sit in shared memory,
// double buffered with cp.async.
#pragma once
#include <cuda_fp16.h>

#include "blockmath.cuh"
#include "device_utils.cuh"
#include "gemv.cuh"

namespace aot {

constexpr int GEMM_WARPS = 8;   // warps per CTA
constexpr int GEMM_KB = 2;      // super-blocks per staged activation chunk
constexpr int GEMM_MAX_M = 64;

struct GemmParams {
  GemvSeg seg[3];
  int nseg, pair, cols, m, epilogue;
  const uint8_t* x;   // [m][cols/256] Q8_K images (304 bytes) or reference-layout BlockQ8_K (292 bytes)
  int x_image;
  int m_pad;          // token slots staged per chunk: n_groups * NT * 8 (>= m)
  int n_groups;       // token groups of 8*NT per tile
  int n_items;        // (row tile, token group) pairs
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
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
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
__device__ __forceinline__ U4 gm_lds128(uint32_t a) {
  U4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// A 32-bit word at a 2-byte aligned global address.
__device__ __forceinline__ uint32_t ldg32_a2(const uint8_t* p) {
  const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
  return (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
}

// One 16-row tile of one matrix against NT token groups: adds, per super-block and in
// block order, the f32 terms into acc[t][i] (i: 0 = row g / token 2q, 1 = row g / token
// 2q+1, 2 = row g+8 / token 2q, 3 = row g+8 / token 2q+1; g = lane/4, q = lane%4).
// `xs` is the shared-space address of the chunk buffer, layout [kb][token][304].
template <int NT>
struct TileAcc {
  float v[NT][4];
};

template <int NT, bool Q5>
__device__ __forceinline__ void gemm_block_k4(const uint8_t* wa, const uint8_t* wb, uint32_t xs, int tok0, TileAcc<NT>& acc) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const uint4 ha = __ldg(reinterpret_cast<const uint4*>(wa)), hb = __ldg(reinterpret_cast<const uint4*>(wb));
  const K4Scales sa = k4_unpack(ha.y, ha.z, ha.w), sb = k4_unpack(hb.y, hb.z, hb.w);
  constexpr int QOFF = Q5 ? 48 : 16;
  uint32_t hqa0 = 0, hqa1 = 0, hqb0 = 0, hqb1 = 0;
  if (Q5) {
    hqa0 = __ldg(reinterpret_cast<const uint32_t*>(wa + 16) + q);
    hqa1 = __ldg(reinterpret_cast<const uint32_t*>(wa + 32) + q);
    hqb0 = __ldg(reinterpret_cast<const uint32_t*>(wb + 16) + q);
    hqb1 = __ldg(reinterpret_cast<const uint32_t*>(wb + 32) + q);
  }
  int sumi[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int i = 0; i < 4; i++) sumi[t][i] = 0;
  }
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const uint32_t qa0 = __ldg(reinterpret_cast<const uint32_t*>(wa + QOFF + 32 * c) + q);
    const uint32_t qa1 = __ldg(reinterpret_cast<const uint32_t*>(wa + QOFF + 32 * c + 16) + q);
    const uint32_t qb0 = __ldg(reinterpret_cast<const uint32_t*>(wb + QOFF + 32 * c) + q);
    const uint32_t qb1 = __ldg(reinterpret_cast<const uint32_t*>(wb + QOFF + 32 * c + 16) + q);
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
      const int j = 2 * c + hi;  // sub-block
      uint32_t a0 = (hi ? qa0 >> 4 : qa0) & 0x0F0F0F0Fu, a2 = (hi ? qa1 >> 4 : qa1) & 0x0F0F0F0Fu;
      uint32_t a1 = (hi ? qb0 >> 4 : qb0) & 0x0F0F0F0Fu, a3 = (hi ? qb1 >> 4 : qb1) & 0x0F0F0F0Fu;
      if (Q5) {
        a0 |= ((hqa0 >> j) & 0x01010101u) << 4;
        a2 |= ((hqa1 >> j) & 0x01010101u) << 4;
        a1 |= ((hqb0 >> j) & 0x01010101u) << 4;
        a3 |= ((hqb1 >> j) & 0x01010101u) << 4;
      }
      const int sca = byte_of(j < 4 ? sa.sc_lo : sa.sc_hi, j & 3), scb = byte_of(j < 4 ? sb.sc_lo : sb.sc_hi, j & 3);
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const uint32_t xa = xs + (uint32_t)(tok0 + 8 * t + g) * XK_STRIDE + 32 * j + 4 * q;
        int cc[4];
        mma_u8s8_k32(cc, a0, a1, a2, a3, gm_lds32(xa), gm_lds32(xa + 16));
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
  const float da = half_bits_to_float((uint16_t)(ha.x & 0xFFFFu)), dmina = half_bits_to_float((uint16_t)(ha.x >> 16));
  const float db = half_bits_to_float((uint16_t)(hb.x & 0xFFFFu)), dminb = half_bits_to_float((uint16_t)(hb.x >> 16));
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
__device__ __forceinline__ void gemm_block_q6k(const uint8_t* wa, const uint8_t* wb, uint32_t xs, int tok0, TileAcc<NT>& acc) {
  const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  int sumi[NT][4];
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int i = 0; i < 4; i++) sumi[t][i] = 0;
  }
  uint32_t sca[4], scb[4];  // scales, four per word
#pragma unroll
  for (int k = 0; k < 4; k++) {
    sca[k] = ldg32_a2(wa + 192 + 4 * k);
    scb[k] = ldg32_a2(wb + 192 + 4 * k);
  }
#pragma unroll
  for (int n = 0; n < 2; n++) {
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      const int lo = 64 * n + 16 * hh + 4 * q, ho = 128 + 32 * n + 16 * hh + 4 * q;
      const uint32_t la0 = ldg32_a2(wa + lo), la32 = ldg32_a2(wa + lo + 32), hqa = ldg32_a2(wa + ho);
      const uint32_t lb0 = ldg32_a2(wb + lo), lb32 = ldg32_a2(wb + lo + 32), hqb = ldg32_a2(wb + ho);
#pragma unroll
      for (int qu = 0; qu < 4; qu++) {  // quarter of the 128-weight half
        const uint32_t la = (qu & 1) ? la32 : la0, lb = (qu & 1) ? lb32 : lb0;
        const uint32_t a0 = ((qu & 2) ? la >> 4 : la) & 0x0F0F0F0Fu | (((hqa >> (2 * qu)) & 0x03030303u) << 4);
        const uint32_t a1 = ((qu & 2) ? lb >> 4 : lb) & 0x0F0F0F0Fu | (((hqb >> (2 * qu)) & 0x03030303u) << 4);
        const int s = 8 * n + hh + 2 * qu;  // sub-block
        const int ca = (int)(int8_t)byte_of(sca[s >> 2], s & 3), cb = (int)(int8_t)byte_of(scb[s >> 2], s & 3);
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
  const float da = half_bits_to_float((uint16_t)(ldg32_a2(wa + 208 - 2) >> 16));
  const float db = half_bits_to_float((uint16_t)(ldg32_a2(wb + 208 - 2) >> 16));
#pragma unroll
  for (int t = 0; t < NT; t++) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const uint32_t xt = xs + (uint32_t)(tok0 + 8 * t + 2 * q + e) * XK_STRIDE;
      const U4 b0 = gm_lds128(xt + XK_BSUMS), b1 = gm_lds128(xt + XK_BSUMS + 16);
      int ba = 0, bb = 0;
      ba = dp2a_lo(b0.x, sca[0], ba); ba = dp2a_hi(b0.y, sca[0], ba);
      ba = dp2a_lo(b0.z, sca[1], ba); ba = dp2a_hi(b0.w, sca[1], ba);
      ba = dp2a_lo(b1.x, sca[2], ba); ba = dp2a_hi(b1.y, sca[2], ba);
      ba = dp2a_lo(b1.z, sca[3], ba); ba = dp2a_hi(b1.w, sca[3], ba);
      bb = dp2a_lo(b0.x, scb[0], bb); bb = dp2a_hi(b0.y, scb[0], bb);
      bb = dp2a_lo(b0.z, scb[1], bb); bb = dp2a_hi(b0.w, scb[1], bb);
      bb = dp2a_lo(b1.x, scb[2], bb); bb = dp2a_hi(b1.y, scb[2], bb);
      bb = dp2a_lo(b1.z, scb[3], bb); bb = dp2a_hi(b1.w, scb[3], bb);
      const float dx = __uint_as_float(gm_lds32(xt + XK_D));
      acc.v[t][e] = fadd(acc.v[t][e], q6k_term(da, dx, sumi[t][e] - 32 * ba));
      acc.v[t][2 + e] = fadd(acc.v[t][2 + e], q6k_term(db, dx, sumi[t][2 + e] - 32 * bb));
    }
  }
}

template <int NT>
__device__ __forceinline__ void gemm_block(int kind, const uint8_t* wa, const uint8_t* wb, uint32_t xs, int tok0,
                                           TileAcc<NT>& acc) {
  if (kind == Q4_K) gemm_block_k4<NT, false>(wa, wb, xs, tok0, acc);
  else if (kind == Q6_K) gemm_block_q6k<NT>(wa, wb, xs, tok0, acc);
  else gemm_block_k4<NT, true>(wa, wb, xs, tok0, acc);
}

// Stage the activation images of super-blocks [b0, b0 + kb_n) for all m_pad tokens into
// `dst` ([kb][token][304]); rows beyond m repeat the last token (their results are dropped).
__device__ __forceinline__ void gemm_stage_x(uint32_t dst, const uint8_t* x, int x_image, int nb, int b0, int kb_n, int m,
                                             int m_pad) {
  if (x_image) {
    const int pieces = kb_n * m_pad * (XK_STRIDE / 16);
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
      const int kb = i / (m_pad * (XK_STRIDE / 16)), r = i - kb * (m_pad * (XK_STRIDE / 16));
      const int tok = r / (XK_STRIDE / 16), p = r - tok * (XK_STRIDE / 16);
      const int ts = tok < m ? tok : m - 1;
      cp_async16(dst + (uint32_t)((kb * m_pad + tok) * XK_STRIDE + 16 * p),
                 x + ((size_t)ts * nb + (size_t)(b0 + kb)) * XK_STRIDE + 16 * p);
    }
  } else {
    // BlockQ8_K {f32 d; i8 qs[256]; i16 bsums[16]} (quant.rs:8-14), word by word into the image layout
    const int pieces = kb_n * m_pad * 73;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
      const int kb = i / (m_pad * 73), r = i - kb * (m_pad * 73);
      const int tok = r / 73, w = r - tok * 73;
      const int ts = tok < m ? tok : m - 1;
      const int off = w == 0 ? XK_D : (w <= 64 ? (w - 1) * 4 : XK_BSUMS + (w - 65) * 4);
      cp_async4(dst + (uint32_t)((kb * m_pad + tok) * XK_STRIDE + off), x + ((size_t)ts * nb + (size_t)(b0 + kb)) * 292 + 4 * w);
    }
  }
}

template <int NT, bool PAIR>
__global__ void __launch_bounds__(GEMM_WARPS * 32) gemm_q8k_mma_kernel(const GemmParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int nb = P.cols >> 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const uint32_t buf_bytes = (uint32_t)(GEMM_KB * P.m_pad * XK_STRIDE);
  const uint32_t sbase = smem_addr(smem);
  const int n_chunks = (nb + GEMM_KB - 1) / GEMM_KB;
  const int per_round = gridDim.x * GEMM_WARPS;
  const int n_rounds = (P.n_items + per_round - 1) / per_round;
  pdl_launch_dependents();
  pdl_wait();
  for (int round = 0; round < n_rounds; round++) {
    // this warp's (row tile, token group)
    const int item = (round * (int)gridDim.x + (int)blockIdx.x) * GEMM_WARPS + warp;
    const bool active = item < P.n_items;
    const int tile = active ? item / P.n_groups : 0;
    const int tok0 = active ? (item - tile * P.n_groups) * 8 * NT : 0;
    int s = 0;
    if (!PAIR) {
      while (s < P.nseg - 1 && tile >= P.tiles_before[s + 1]) s++;
    }
    const int r0 = (tile - P.tiles_before[s]) * 16;
    constexpr int n_mat = PAIR ? 2 : 1;
    TileAcc<NT> acc[n_mat];
#pragma unroll
    for (int mt = 0; mt < n_mat; mt++) {
#pragma unroll
      for (int t = 0; t < NT; t++) {
#pragma unroll
        for (int i = 0; i < 4; i++) acc[mt].v[t][i] = 0.0f;
      }
    }
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
    __syncthreads();  // the previous round is done with both chunk buffers
    gemm_stage_x(sbase, P.x, P.x_image, nb, 0, min(GEMM_KB, nb), P.m, P.m_pad);
    cp_async_commit();
    for (int ch = 0; ch < n_chunks; ch++) {
      const int b0 = ch * GEMM_KB, kb_n = min(GEMM_KB, nb - b0);
      if (ch + 1 < n_chunks) {
        gemm_stage_x(sbase + ((ch + 1) & 1) * buf_bytes, P.x, P.x_image, nb, b0 + GEMM_KB, min(GEMM_KB, nb - b0 - GEMM_KB), P.m,
                     P.m_pad);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (active) {
        const uint32_t xs = sbase + (ch & 1) * buf_bytes;
        for (int kb = 0; kb < kb_n; kb++) {
          const int b = b0 + kb;
          const uint32_t xb = xs + (uint32_t)(kb * P.m_pad) * XK_STRIDE;
          gemm_block<NT>(kind[0], wrow[0][0] + (size_t)b * rbytes[0], wrow[0][1] + (size_t)b * rbytes[0], xb, tok0, acc[0]);
          if (PAIR)
            gemm_block<NT>(kind[n_mat - 1], wrow[n_mat - 1][0] + (size_t)b * rbytes[n_mat - 1],
                           wrow[n_mat - 1][1] + (size_t)b * rbytes[n_mat - 1], xb, tok0, acc[n_mat - 1]);
        }
      }
      __syncthreads();  // everyone is done with this buffer before it is refilled
    }
    if (active) {
#pragma unroll
      for (int t = 0; t < NT; t++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int row = r0 + g + (i >> 1) * 8, tok = tok0 + 8 * t + 2 * q + (i & 1);
          const GemvSeg& sg = P.seg[PAIR ? 0 : s];
          if (row < sg.rows && tok < P.m) {
            const size_t o = (size_t)tok * sg.rows + row;
            if (PAIR) {
              const float gate = acc[0].v[t][i], up = acc[n_mat - 1].v[t][i];
              P.seg[0].out[o] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(gate, up) : gate;
              P.seg[1].out[o] = up;
            } else {
              const float v = acc[0].v[t][i];
              sg.out[o] = P.epilogue == EPI_ACCUM ? fadd(sg.out[o], v) : v;
            }
          }
        }
      }
    }
  }
}

}  // namespace aot
