// Products of Q4_0 / Q5_0 / Q8_0 matrices with Q8_0 activation rows, streamed by column
// chunks (matvec.rs:170-262: eight AVX2 lane accumulators per row, one fma per 32-weight
// block, the horizontal sum of simd_avx2.rs:29-34 at the end).
//
// A row's result is eight sequential chains of nb = cols / 32 fused multiply-adds, so the
// work that can run at once is (rows on the SM) x 8 chains. Keeping whole rows in shared
// memory leaves too few of them there (a 14336-column Q8_0 row is 15 KB). This kernel keeps
// a group of 60 or 120 rows resident as column chunks instead: for every four rows of the
// group ("quad") the producer warp requests the next 16 blocks as one 2-D tensor copy
// (cp.async.bulk.tensor over this GPU's own memory, no multicast) into a ring stage; lane
// (g, k) of consumer warp w owns chain k of row g of the warp's quad (of its two quads, for
// N = 2 rows per lane) from the first chunk to the last, with the accumulators in registers.
// A chunk row is 288 / 352 / 544 bytes (32 or 96 modulo 128), so the four rows a warp reads
// in one instruction fall into different banks, and all of them read the same activation
// words (a broadcast). Several activation rows (NT > 1) meet every block while its weights
// are in registers; their images' chunk travels with the stage as one more tensor copy.
#pragma once
#include <cuda.h>

#include "mega.cuh"

namespace aot {

constexpr int Q80S_CBLK = 16;     // blocks per chunk
constexpr int Q80S_MAX_TOK = 16;  // activation rows per launch (accumulators live in registers)

template <int KIND>
struct Q80Kind {
  static constexpr int BS = KIND == Q4_0 ? 18 : (KIND == Q5_0 ? 22 : 34);
  static constexpr int CB = Q80S_CBLK * BS;  // bytes of a chunk row: a multiple of 16, and 32 or 96 modulo 128
  static_assert(CB % 16 == 0 && (CB % 128 == 32 || CB % 128 == 96), "chunk rows must be TMA-aligned and spread over the banks");
};
constexpr int q80s_chunk_bytes(int kind) { return Q80S_CBLK * (kind == Q4_0 ? 18 : (kind == Q5_0 ? 22 : 34)); }

struct Q80StreamParams {
  alignas(64) CUtensorMap map[3];  // per matrix: u32 elements, [rows][row_bytes / 4], box [4][CB / 4]
  alignas(64) CUtensorMap xmap;    // NT > 1: the activation images as u32 [m][nb * 12], box [16][16 blocks]
  GemvSeg seg[3];
  int nseg, pair, cols, epilogue;
  int quad_base, quad_rem;  // quads (four rows of the row space; pair rows in pair mode) split over the grid
  const void* x;            // NT = 1: the activation row, block images (x_image) or reference-layout blocks
  int x_image, m;
  int qw, ts;  // consumer warps per token group (each owns NR quads of a stage), token groups (qw * ts <= consumer warps)
  int n_stages;
  int* err;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
               : "memory");
}

// Lane k's four weights of a block as signed bytes (the operand of its dp4a): the integers
// q4_0_lane / q5_0_lane / q8_0_lane form.
template <int KIND>
__device__ __forceinline__ int q80_lane_word(uint32_t wb, int k) {
  if (KIND == Q8_0) return (int)lds32_a2s(wb + 2 + 4 * k);
  if (KIND == Q4_0) {
    const uint32_t qs4 = lds32_a2s(wb + 2 + 4 * (k & 3));
    const uint32_t v = (k < 4 ? qs4 : (qs4 >> 4)) & 0x0F0F0F0Fu;
    return (int)(((v | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
  }
  const uint32_t qs4 = lds32_a2s(wb + 6 + 4 * (k & 3)), qh = lds32_a2s(wb + 2);
  uint32_t v = (k < 4 ? qs4 : (qs4 >> 4)) & 0x0F0F0F0Fu;
  const uint32_t hb = (qh >> (4 * k)) & 0xFu;
  v |= ((hb & 1u) << 4) | ((hb & 2u) << 11) | ((hb & 4u) << 18) | ((hb & 8u) << 25);
  return (int)(((v | 0x80808080u) - 0x10101010u) ^ 0x80808080u);
}

// Quad of the row space -> (matrix, first row inside it). Every matrix has a multiple of four rows.
__device__ __forceinline__ void q80s_locate(const Q80StreamParams& P, int quad, int& sg, int& lr) {
  sg = 0;
  lr = 4 * quad;
  if (!P.pair)
    while (sg < P.nseg - 1 && lr >= P.seg[sg].rows) {
      lr -= P.seg[sg].rows;
      sg++;
    }
}

template <int KIND, int NR, int NT>
__global__ void __launch_bounds__(MEGA_THREADS, 1) q80_stream_kernel(const __grid_constant__ Q80StreamParams P) {
  using K = Q80Kind<KIND>;
  constexpr int BS = K::BS, CB = K::CB, CBLK = Q80S_CBLK;
  constexpr int QUAD = 4 * CB;
  // several activation rows: their images travel with the stage, one chunk (16 blocks of 16
  // rows) per stage, so neither the row length nor the number of rows is bounded by shared memory
  constexpr bool XS = NT > 1;
  constexpr int XROW = Q80S_CBLK * X0_STRIDE;        // bytes of one activation row's chunk
  constexpr int XBYTES = XS ? Q80S_MAX_TOK * XROW : 0;
  const int SLOTS = P.qw * NR;  // quads per stage
  const int WBYTES = SLOTS * QUAD;
  const int STAGE = WBYTES + XBYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages: weight quads (, activation chunk)][activation images of a single row][barriers][abort]
  const int nb = P.cols >> 5;
  uint8_t* const stages = smem;
  uint8_t* const sx = stages + (size_t)P.n_stages * STAGE;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(sx + (XS ? 0 : (((size_t)nb * X0_STRIDE + 127) & ~(size_t)127)));
  volatile int* const abort = reinterpret_cast<volatile int*>(bars + 16);
  Ring R;
  R.stages = stages;
  R.full = bars;
  R.empty = bars + 8;
  R.desc = nullptr;
  R.n_stages = P.n_stages;
  R.stage_bytes = STAGE;
  R.abort = abort;
  R.err = P.err;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) {
      mbar_init(&R.full[s], 1);
      mbar_init(&R.empty[s], MEGA_CONSUMER_WARPS);
    }
    *abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = (int)blockIdx.x;
  const int q0 = cta * P.quad_base + min(cta, P.quad_rem), q1 = q0 + P.quad_base + (cta < P.quad_rem ? 1 : 0);
  // quads of the row space a group covers: a pair quad fills two slots (gate, up)
  const int qpg = P.pair ? SLOTS / 2 : SLOTS;
  const int n_groups = (q1 - q0 + qpg - 1) / qpg;
  const int n_chunks = (nb + CBLK - 1) / CBLK;
  // slot s = (warp s / NR, quad of the lane s % NR) -> matrix and first row
  auto slot_quad = [&](int gq, int s, int& sg, int& lr) -> bool {
    const int quad = P.pair ? gq + s / NR : gq + s;
    if (quad >= q1) return false;
    q80s_locate(P, quad, sg, lr);
    if (P.pair) sg = s % NR;
    return true;
  };
  pdl_launch_dependents();
  if (warp == MEGA_CONSUMER_WARPS) {
    // weights do not depend on the previous kernel: stream them right away (the activation
    // chunks of several rows do, and go with them)
    if (XS) pdl_wait();
    RingPos pp{0, 0u};
    uint32_t tiles_issued = 0;
#pragma unroll 1
    for (int grp = 0; grp < n_groups; grp++) {
      int sg = 0, lr = 0;
      const bool mine = lane < SLOTS && (NR == 2 || !P.pair) && slot_quad(q0 + grp * qpg, lane, sg, lr);
      const uint32_t total = __popc(__ballot_sync(0xffffffffu, mine)) * (uint32_t)QUAD + (uint32_t)XBYTES;
#pragma unroll 1
      for (int c = 0; c < n_chunks; c++) {
        int ok = 1;
        if (lane == 0) ok = ring_wait(R, &R.empty[pp.st], pp.parity ^ 1u) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, ok, 0)) {
          if (lane == 0) produce_drain(R, pp, tiles_issued);
          return;
        }
        if (mine)
          tma_load_2d(smem_addr(stages + (size_t)pp.st * STAGE + lane * QUAD), &P.map[sg], c * (CB / 4), lr, &R.full[pp.st]);
        if (XS && lane == 31) tma_load_2d(smem_addr(stages + (size_t)pp.st * STAGE + WBYTES), &P.xmap, c * (XROW / 4), 0, &R.full[pp.st]);
        __syncwarp();
        if (lane == 0) mbar_expect_tx(&R.full[pp.st], total);
        tiles_issued++;
        pp.advance(R.n_stages);
      }
    }
    if (lane == 0) produce_drain(R, pp, tiles_issued);
    return;
  }
  pdl_wait();
  if (!XS) {
    CtaGroup cg{(int)threadIdx.x, MEGA_CONSUMER_WARPS * 32, 1};
    if (P.x_image) {
      const uint4* src4 = reinterpret_cast<const uint4*>(P.x);
      for (int i = cg.tid; i < nb * (X0_STRIDE / 16); i += cg.nthreads) reinterpret_cast<uint4*>(sx)[i] = src4[i];
    } else {
      // BlockQ8_0 {f32 d; i8 qs[32]} (quant.rs:16-20) -> image {qs; d}
      const uint32_t* src = reinterpret_cast<const uint32_t*>(P.x);
      for (int i = cg.tid; i < nb * 9; i += cg.nthreads) {
        const int bi = i / 9, w = i - bi * 9;
        *reinterpret_cast<uint32_t*>(sx + bi * X0_STRIDE + (w == 0 ? X0_D : (w - 1) * 4)) = src[i];
      }
    }
    cg.sync();
  }
  const int k = lane & 7, g = lane >> 3;
  // token group tg (activation rows tok0 .. tok0 + NT - 1), quads wq * NR .. of every stage
  const int tg = warp / P.qw, wq = warp - tg * P.qw, tok0 = tg * NT;
  // distance between activation rows, and this token group's first row (inside the stage when streamed)
  const uint32_t xs = XS ? (uint32_t)XROW : (uint32_t)nb * X0_STRIDE, sxa = XS ? (uint32_t)tok0 * xs : smem_addr(sx);
  RingPos cp{0, 0u};
#pragma unroll 1
  for (int grp = 0; grp < n_groups; grp++) {
    // this lane's rows: matrix, row, place in the stage
    int sgi[NR], lri[NR];
    bool live[NR];
    bool any_live = false;
#pragma unroll
    for (int nr = 0; nr < NR; nr++) {
      sgi[nr] = 0;
      lri[nr] = 0;
      live[nr] = tg < P.ts && (NR == 2 || !P.pair) && slot_quad(q0 + grp * qpg, wq * NR + nr, sgi[nr], lri[nr]);
      lri[nr] += g;
      any_live = any_live || live[nr];
    }
    float acc[NR][NT];
#pragma unroll
    for (int nr = 0; nr < NR; nr++)
#pragma unroll
      for (int t = 0; t < NT; t++) acc[nr][t] = 0.0f;
#pragma unroll 1
    for (int c = 0; c < n_chunks; c++) {
      if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
      const uint32_t wrow0 = smem_addr(stages + (size_t)cp.st * STAGE) + (uint32_t)(wq * NR) * QUAD + (uint32_t)g * CB;
      const int nblk = any_live ? min(CBLK, nb - c * CBLK) : 0;  // a warp without rows only keeps the ring turning
      const uint32_t xc = XS ? smem_addr(stages + (size_t)cp.st * STAGE) + (uint32_t)WBYTES + sxa : sxa + (uint32_t)c * (CBLK * X0_STRIDE);
#pragma unroll(NT == 1 ? 4 : 1)
      for (int jb = 0; jb < nblk; jb++) {
        const uint32_t xb = xc + (uint32_t)jb * X0_STRIDE;
        float dw[NR];
        int w4[NR];
#pragma unroll
        for (int nr = 0; nr < NR; nr++) {
          const uint32_t wb = wrow0 + (uint32_t)nr * QUAD + (uint32_t)jb * BS;
          uint32_t h;
          asm("ld.shared.u16 %0, [%1];" : "=r"(h) : "r"(wb));
          dw[nr] = half_bits_hw(h);
          w4[nr] = q80_lane_word<KIND>(wb, k);
        }
#pragma unroll
        for (int t = 0; t < NT; t++) {
          {  // rows past the launch's last are zeros in the box: their sums are dropped below
            const uint32_t xt = xb + (uint32_t)t * xs;
            const int y = (int)rd_lds32(xt + 4 * k);
            const float dx = __uint_as_float(rd_lds32(xt + X0_D));
#pragma unroll
            for (int nr = 0; nr < NR; nr++) acc[nr][t] = ffma(fmul(dw[nr], dx), i2f(__dp4a(w4[nr], y, 0)), acc[nr][t]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&R.empty[cp.st]);
      cp.advance(R.n_stages);
    }
    // ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)) over a row's eight lanes, then the epilogue
#pragma unroll
    for (int t = 0; t < NT; t++) {
      if (NT == 1 || tok0 + t < P.m) {
        float v[NR];
#pragma unroll
        for (int nr = 0; nr < NR; nr++) {
          float a = acc[nr][t];
          a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 4));
          a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 2));
          v[nr] = fadd(a, __shfl_xor_sync(0xffffffffu, a, 1));
        }
        if (k == 0) {
          if (NR == 2 && P.pair) {
            if (live[0]) {
              const size_t r = (size_t)(tok0 + t) * P.seg[0].rows + lri[0];
              P.seg[0].out[r] = P.epilogue == EPI_SILU_MUL ? silu_mul_exact(v[0], v[NR - 1]) : v[0];
              P.seg[1].out[r] = v[NR - 1];
            }
          } else {
#pragma unroll
            for (int nr = 0; nr < NR; nr++) {
              if (live[nr]) {
                float* o = P.seg[sgi[nr]].out + (size_t)(tok0 + t) * P.seg[sgi[nr]].rows + lri[nr];
                *o = P.epilogue == EPI_ACCUM ? fadd(__ldcg(o), v[nr]) : v[nr];
              }
            }
          }
        }
      }
    }
  }
}

}  // namespace aot
