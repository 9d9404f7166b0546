// Products of F16 / BF16 / F32 matrices with f32 activation rows, streamed by column chunks
// (simd_avx2.rs:433-493: eight AVX2 lane accumulators per row, acc_k = fma(w[8j+k], x[8j+k],
// acc_k) for j in order, then the horizontal sum of simd_avx2.rs:29-34).
//
// The structure of q80stream.cuh: a group of 60 or 120 rows stays resident as 288- or 544-byte
// column chunks, one 2-D tensor copy per four rows ("quad") and chunk, and lane (g, k) of a
// consumer warp owns chain k of row g of the warp's quad(s) from the first chunk to the
// last. The activation rows are f32 in global memory, so their chunk travels with the
// stage as one more tensor copy (box: chunk columns by 1 or 16 rows; rows past the launch's
// last are filled with zeros and their results dropped), and no length of row or number of
// rows has to fit in shared memory. Columns in eights only (the scalar tail of an odd
// length is left to gemv_float_kernel).
#pragma once
#include <cuda.h>

#include "mega.cuh"
#include "q80stream.cuh"

namespace aot {

// bytes of a chunk row (32 modulo 128): 544 for a single activation row (larger copies: the copy
// engine's rate of requests is what limits a pure stream), 288 for several (the stage also holds
// 16 rows of activations, and the arithmetic sets the pace)
constexpr int FS_CB_ONE = 544, FS_CB_MANY = 288;
inline int fs_chunk_bytes(size_t m) { return m == 1 ? FS_CB_ONE : FS_CB_MANY; }
constexpr int FS_MAX_TOK = 16;   // activation rows per launch

struct FloatStreamParams {
  alignas(64) CUtensorMap map[3];  // per matrix: u32 elements, [rows][row_bytes / 4], box [4][chunk bytes / 4]
  alignas(64) CUtensorMap xmap;    // activations: f32 [m][cols], box [1 or 16][chunk columns, at most 136]
  GemvSeg seg[3];
  int nseg, pair, cols, epilogue;
  int quad_base, quad_rem;  // quads (four rows of the row space; pair rows in pair mode) split over the grid
  int m;                    // activation rows of this launch
  int qw, ts;               // consumer warps per token group (each owns NR quads of a stage), token groups
  int n_stages;
  int* err;
};

template <int KIND, int NR, int NT>
__global__ void __launch_bounds__(MEGA_THREADS, 1) float_stream_kernel(const __grid_constant__ FloatStreamParams P) {
  constexpr int FS_CB = NT == 1 ? FS_CB_ONE : FS_CB_MANY;
  constexpr int ES = KIND == F32 ? 4 : 2;       // bytes per weight
  constexpr int CCOLS = FS_CB / ES;             // columns per chunk
  constexpr int CSTEPS = CCOLS / 8;             // AVX2 steps per chunk
  constexpr int QUAD = 4 * FS_CB;
  constexpr int XROW = CCOLS * 4;               // bytes of an activation row's chunk
  // a tensor box holds at most 256 elements per row: the 272-column chunk of a single row comes as two copies
  constexpr int NXC = CCOLS > 256 ? 2 : 1, XBOX = CCOLS / NXC;
  constexpr int XROWS = NT == 1 ? 1 : FS_MAX_TOK;   // rows of the activation box
  static_assert(NXC == 1 || XROWS == 1, "split activation boxes are single rows");
  constexpr int XCOPY = (XROWS * XBOX * 4 + 127) & ~127;
  const int SLOTS = P.qw * NR;                  // quads per stage
  const int WBYTES = SLOTS * QUAD;
  const int STAGE = WBYTES + NXC * XCOPY;
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages: weight quads, activation chunk][barriers][abort]
  uint8_t* const stages = smem;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(stages + (size_t)P.n_stages * STAGE);
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
  const int qpg = P.pair ? SLOTS / 2 : SLOTS;
  const int n_groups = (q1 - q0 + qpg - 1) / qpg;
  const int n_chunks = (P.cols + CCOLS - 1) / CCOLS;
  // slot s = (warp s / NR, quad of the lane s % NR) -> matrix and first row
  auto slot_quad = [&](int gq, int s, int& sg, int& lr) -> bool {
    const int quad = P.pair ? gq + s / NR : gq + s;
    if (quad >= q1) return false;
    sg = 0;
    lr = 4 * quad;
    if (P.pair) {
      sg = s % NR;
    } else {
      while (sg < P.nseg - 1 && lr >= P.seg[sg].rows) {
        lr -= P.seg[sg].rows;
        sg++;
      }
    }
    return true;
  };
  pdl_launch_dependents();
  if (warp == MEGA_CONSUMER_WARPS) {
    // the activation rows are the previous kernel's output
    pdl_wait();
    RingPos pp{0, 0u};
    uint32_t tiles_issued = 0;
#pragma unroll 1
    for (int grp = 0; grp < n_groups; grp++) {
      int sg = 0, lr = 0;
      const bool mine = lane < SLOTS && (NR == 2 || !P.pair) && slot_quad(q0 + grp * qpg, lane, sg, lr);
      const uint32_t total = __popc(__ballot_sync(0xffffffffu, mine)) * (uint32_t)QUAD + (uint32_t)(XROWS * XROW);
#pragma unroll 1
      for (int c = 0; c < n_chunks; c++) {
        int ok = 1;
        if (lane == 0) ok = ring_wait(R, &R.empty[pp.st], pp.parity ^ 1u) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, ok, 0)) {
          if (lane == 0) produce_drain(R, pp, tiles_issued);
          return;
        }
        uint8_t* const stage = stages + (size_t)pp.st * STAGE;
        if (mine) tma_load_2d(smem_addr(stage + lane * QUAD), &P.map[sg], c * (FS_CB / 4), lr, &R.full[pp.st]);
        if (lane >= 32 - NXC) tma_load_2d(smem_addr(stage + WBYTES + (31 - lane) * XCOPY), &P.xmap, c * CCOLS + (31 - lane) * XBOX, 0, &R.full[pp.st]);
        __syncwarp();
        if (lane == 0) mbar_expect_tx(&R.full[pp.st], total);
        tiles_issued++;
        pp.advance(R.n_stages);
      }
    }
    if (lane == 0) produce_drain(R, pp, tiles_issued);
    return;
  }
  pdl_wait();  // residual adds read what the previous kernel wrote
  const int k = lane & 7, g = lane >> 3;
  // token group tg (activation rows tok0 .. tok0 + NT - 1), quads wq * NR .. of every stage
  const int tg = warp / P.qw, wq = warp - tg * P.qw, tok0 = tg * NT;
  RingPos cp{0, 0u};
#pragma unroll 1
  for (int grp = 0; grp < n_groups; grp++) {
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
      const uint32_t stage = smem_addr(stages + (size_t)cp.st * STAGE);
      const uint32_t wrow0 = stage + (uint32_t)(wq * NR) * QUAD + (uint32_t)g * FS_CB + (uint32_t)k * ES;
      const uint32_t xrow0 = stage + (uint32_t)WBYTES + (uint32_t)tok0 * XROW + (uint32_t)k * 4;
      const int nsteps = any_live ? min(CSTEPS, (P.cols - c * CCOLS) >> 3) : 0;  // a warp without rows only keeps the ring turning
#pragma unroll(NT == 1 ? 6 : 1)
      for (int j = 0; j < nsteps; j++) {
        float w[NR];
#pragma unroll
        for (int nr = 0; nr < NR; nr++) {
          const uint32_t wa = wrow0 + (uint32_t)nr * QUAD + (uint32_t)j * (8 * ES);
          if (KIND == F32) {
            w[nr] = __uint_as_float(rd_lds32(wa));
          } else {
            uint32_t h;
            asm("ld.shared.u16 %0, [%1];" : "=r"(h) : "r"(wa));
            // both conversions are exact (every f16 / bf16 value is an f32 value)
            w[nr] = KIND == F16 ? half_bits_hw(h) : __uint_as_float(h << 16);
          }
        }
#pragma unroll
        for (int t = 0; t < NT; t++) {
          const float x = __uint_as_float(rd_lds32(xrow0 + (uint32_t)t * XROW + (uint32_t)j * 32 + (NXC == 2 && j >= CSTEPS / 2 ? XCOPY - XBOX * 4 : 0)));
#pragma unroll
          for (int nr = 0; nr < NR; nr++) acc[nr][t] = ffma(w[nr], x, acc[nr][t]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&R.empty[cp.st]);
      cp.advance(R.n_stages);
    }
    // ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)) over a row's eight lanes, then the epilogue
#pragma unroll
    for (int t = 0; t < NT; t++) {
      float v[NR];
#pragma unroll
      for (int nr = 0; nr < NR; nr++) {
        float a = acc[nr][t];
        a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 4));
        a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 2));
        v[nr] = fadd(a, __shfl_xor_sync(0xffffffffu, a, 1));
      }
      if (k == 0 && tok0 + t < P.m) {
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

}  // namespace aot
