// Prompt chunks (8..64 activation rows) against Q4_K / Q5_K matrices on the fifth-generation
// tensor cores: tcgen05.mma kind::i8 with int32 accumulators in tensor memory
// (matmul_rows of crates/aot-kernels/src/matvec.rs:479-522; the x4 micro-kernels of
// simd_avx2.rs:340-384 are its CPU counterpart).
//
// The obstacle to one contraction per 256-weight super-block is the 6-bit scale of every
// 32-weight sub-block: sumi = sum_j sc_j * (q_j . y_j), and sc * q does not fit eight bits.
// The scale is split instead of the product: sc = 8 * s_hi + s_lo with both digits in 0..7,
// so s_hi * q and s_lo * q are at most 7 * 31 = 217 and fit an unsigned byte. A CUDA-core
// pass turns the raw nibbles into two operand tiles A_hi = s_hi * q and A_lo = s_lo * q (one
// 32-bit multiply per four weights and digit), the tensor core accumulates both over the
// whole super-block, and sumi = 8 * acc_hi + acc_lo is the reference's integer, bit for
// bit. The accumulators are read out once per super-block, not once per sub-block.
//
// One CTA owns tiles of 128 weight rows (M) x up to 64 tokens (N). Warp roles:
//   warps 0..7   fill: per 64-weight chunk, turn raw GGUF bytes (requested one super-block
//                ahead) and Q8_K activations into the operand tiles of a ring stage
//                (canonical K-major layout without swizzle: 8 rows x 16 bytes core matrices);
//   warps 8..15  epilogue: tcgen05.ld the two accumulators of a finished super-block,
//                form the reference's f32 term (d_w*d_x)*sumi - (dmin_w*d_x)*summ and add
//                it to the row's running sum in block order (the order of the single-row
//                products, so batched == single bit for bit, dots.rs:205-266);
//   warp 16      one thread issues the MMAs and commits them to mbarriers.
// Two accumulator sets (256 tensor-memory columns) let the epilogue of one super-block run
// under the MMAs of the next. Every wait is bounded; on expiry the error word is set and
// the CTA drains, frees its tensor memory and returns.
#pragma once
#include "blockmath.cuh"
#include "device_utils.cuh"
#include "gemv.cuh"

namespace aot {

constexpr int TC_ROWS = 128;             // weight rows per tile (MMA M)
constexpr int TC_TOK = 64;               // tokens per tile (MMA N)
constexpr int TC_FILL_WARPS = 8;
constexpr int TC_EPI_WARPS = 8;
constexpr int TC_THREADS = (TC_FILL_WARPS + TC_EPI_WARPS + 1) * 32;
constexpr int TC_STAGES = 4;
constexpr int TC_A_TILE = TC_ROWS * 32;  // one digit, one K = 32 step: 4 KB
constexpr int TC_B_TILE = TC_TOK * 32;   // 2 KB
// stage: [A_hi step 0][A_lo step 0][A_hi step 1][A_lo step 1][B step 0][B step 1]
constexpr int TC_STAGE_BYTES = 4 * TC_A_TILE + 2 * TC_B_TILE;
// side data of one super-block: per weight row {d, dmin, mins 0..3, mins 4..7}, per token
// {d_x, pad, pad, pad, four words of sub-block sums}
constexpr int TC_SIDE_BYTES = TC_ROWS * 16 + TC_TOK * 32;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 2 * TC_SIDE_BYTES + 256;
constexpr int TC_TMEM_COLS = 256;        // two sets of (acc_hi, acc_lo) x 64 columns

struct GemmTcParams {
  GemvSeg seg[3];
  int nseg, cols, m, epilogue;
  const uint8_t* prep[3];  // prepared operands of each matrix (k4_prepare_kernel); gemm_k4_prep_kernel only
  const uint8_t* x;  // [m][cols/256] Q8_K images (304 bytes) or reference-layout BlockQ8_K (292 bytes)
  int x_image;
  int tiles_before[4];  // first tile of each matrix in the concatenated tile space
  int n_tiles;
  int* err;
  // parity export (one matrix): integers per (token, row, block) before any float arithmetic, or null
  int* dbg_sumi;
  int* dbg_summ;
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_dst)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// All MMAs this thread issued so far arrive on `bar` when they have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Shared-memory operand descriptor: K-major, no swizzle, core matrices of 8 rows x 16 bytes
// stored back to back; the second 16-byte K chunk of a row group lies 128 bytes after the
// first (leading byte offset), the next group of 8 rows 256 bytes on (stride byte offset).
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(256 >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor: D = s32, A = unsigned 8-bit, B = signed 8-bit, both K-major,
// N = 64, M = 128.
constexpr uint32_t TC_IDESC = (2u << 4) | (0u << 7) | (1u << 10) | ((TC_TOK >> 3) << 17) | ((TC_ROWS >> 4) << 24);
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 consecutive columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, int (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Generic-proxy stores to shared memory become visible to the tensor core's reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Bounded wait on an mbarrier phase; `abort` is a shared flag of the CTA.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* err) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
  }
  *abort = 1;
  if (err) atomicOr(err, DEVERR_MBAR_TIMEOUT);
  return false;
}

// 16 bytes from global memory at an address that is 16-byte aligned (block images) or only
// 4-byte aligned (reference-layout blocks).
__device__ __forceinline__ uint4 ldg16_any(const uint8_t* p) {
  if (((uintptr_t)p & 15u) == 0) return __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
  return make_uint4(__ldg(q), __ldg(q + 1), __ldg(q + 2), __ldg(q + 3));
}

// Offset of byte k (0..31) of row r inside a K = 32 operand tile.
__device__ __forceinline__ uint32_t tc_tile_off(int r, int kchunk) { return (uint32_t)((r & 7) * 16 + (r >> 3) * 256 + kchunk * 128); }

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_k4_tc_kernel(const GemmTcParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][side data x 2][barriers][tmem base][abort]
  uint8_t* const stages = smem;
  uint8_t* const side = smem + TC_STAGES * TC_STAGE_BYTES;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(side + 2 * TC_SIDE_BYTES);
  uint64_t* const full = bars;                   // [TC_STAGES] fill -> MMA
  uint64_t* const empty = bars + TC_STAGES;      // [TC_STAGES] MMA -> fill
  uint64_t* const acc_full = bars + 2 * TC_STAGES;       // [2] MMA -> epilogue
  uint64_t* const acc_empty = bars + 2 * TC_STAGES + 2;  // [2] epilogue -> MMA and fill
  uint64_t* const side_full = bars + 2 * TC_STAGES + 4;  // [2] fill -> epilogue: side data of the super-block written
  uint64_t* const drain = bars + 2 * TC_STAGES + 6;      // all MMAs of the CTA have completed
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 7);
  volatile int* const abort = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; s++) {
      mbar_init(&full[s], TC_FILL_WARPS / 2);  // the four warps whose threads own the chunk
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], TC_EPI_WARPS);
      mbar_init(&side_full[b], TC_FILL_WARPS);
    }
    mbar_init(drain, 1);
    *abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) tc_alloc(tmem_slot, TC_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  const int nb = P.cols >> 8, m = P.m;
  const size_t x_block = P.x_image ? XK_STRIDE : 292;  // bytes of one activation block
  const int x_qs = P.x_image ? 0 : 4, x_bs = P.x_image ? XK_BSUMS : 260, x_d = P.x_image ? XK_D : 0;

  if (warp < TC_FILL_WARPS) {
    // ---- fill warps ---------------------------------------------------------------------------
    // Thread (row r, chunk pair cp) turns chunks 2cp and 2cp+1 of every super-block of its
    // row into operand tiles. Its 64 raw bytes of the next super-block are requested while
    // the current one is processed, so the fill does not run at memory latency.
    const int f = threadIdx.x;          // 0..255
    const int r = f & 127, cp = f >> 7;
    uint32_t blk = 0;                   // super-block counter (accumulator set = blk & 1)
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      int sg = 0;
      while (sg < P.nseg - 1 && tile >= P.tiles_before[sg + 1]) sg++;
      const GemvSeg& S = P.seg[sg];
      const bool q5 = S.kind == Q5_K;
      const int bs = q5 ? 176 : 144, qoff = (q5 ? 48 : 16) + 64 * cp;
      const size_t row_bytes = (size_t)nb * bs;
      const int row0 = (tile - P.tiles_before[sg]) * TC_ROWS;
      const int rr = min(row0 + r, S.rows - 1);  // rows past the matrix repeat its last row; their results are dropped
      const uint8_t* wrow = S.w + (size_t)rr * row_bytes;
      // Weights (header, scales and this thread's 64 quant bytes) are requested one super-block
      // ahead, the activations of a chunk one chunk ahead, so that the fill does not run at
      // memory latency.
      auto fetch_w = [&](int b, uint4& hdr, uint4 (&q)[4]) {
        const uint8_t* wb = wrow + (size_t)b * bs;
        hdr = __ldg(reinterpret_cast<const uint4*>(wb));
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = __ldg(reinterpret_cast<const uint4*>(wb + qoff) + i);
      };
      // this thread's two 16-byte parts (items r and r + 128 of 256) of chunk c of block b
      auto fetch_x = [&](int b, int c, uint4 (&xa)[2]) {
#pragma unroll
        for (int k = 0; k < 2; k++) {
          const int item = r + 128 * k, tok = item >> 2, part = item & 3;
          xa[k] = make_uint4(0, 0, 0, 0);
          if (tok < m) xa[k] = ldg16_any(P.x + ((size_t)tok * nb + b) * x_block + x_qs + 64 * c + 16 * part);
        }
      };
      uint4 n_hdr, n_q[4], n_xa[2];
      fetch_w(0, n_hdr, n_q);
      fetch_x(0, 2 * cp, n_xa);
      for (int b = 0; b < nb; b++, blk++) {
        const uint8_t* wb = wrow + (size_t)b * bs;
        const uint4 hdr = n_hdr;
        uint4 qv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) qv[i] = n_q[i];
        if (b + 1 < nb) fetch_w(b + 1, n_hdr, n_q);
        uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0;
        if (q5) {
          h0 = __ldg(reinterpret_cast<const uint4*>(wb + 16));
          h1 = __ldg(reinterpret_cast<const uint4*>(wb + 16) + 1);
        }
        // token side data (threads cp == 1, r < tokens): requested now, written after the chunks
        uint32_t t_dx = 0;
        uint4 t_bs0 = make_uint4(0, 0, 0, 0), t_bs1 = t_bs0;
        if (cp == 1 && r < m) {
          const uint8_t* xb = P.x + ((size_t)r * nb + b) * x_block;
          t_dx = __ldg(reinterpret_cast<const uint32_t*>(xb + x_d));
          const uint32_t* bsw = reinterpret_cast<const uint32_t*>(xb + x_bs);
          t_bs0 = make_uint4(__ldg(bsw), __ldg(bsw + 1), __ldg(bsw + 2), __ldg(bsw + 3));
          t_bs1 = make_uint4(__ldg(bsw + 4), __ldg(bsw + 5), __ldg(bsw + 6), __ldg(bsw + 7));
        }
        const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
        const int buf = blk & 1;
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
          const int c = 2 * cp + cc;
          const uint32_t it = blk * 4 + (uint32_t)c;  // stage use counter
          const int st = it % TC_STAGES;
          uint4 xa[2] = {n_xa[0], n_xa[1]};
          // the next chunk this thread fills: the other one of this block, or the first of the next
          if (cc == 0) fetch_x(b, c + 1, n_xa);
          else if (b + 1 < nb) fetch_x(b + 1, 2 * cp, n_xa);
          if (!tc_wait(&empty[st], ((it / TC_STAGES) & 1u) ^ 1u, abort, P.err)) goto fill_done;
          uint8_t* stg = stages + st * TC_STAGE_BYTES;
          const uint32_t qw[8] = {qv[2 * cc].x, qv[2 * cc].y, qv[2 * cc].z, qv[2 * cc].w,
                                  qv[2 * cc + 1].x, qv[2 * cc + 1].y, qv[2 * cc + 1].z, qv[2 * cc + 1].w};
          const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
          // A: sub-blocks j = 2c (low nibbles, step 0) and 2c + 1 (high nibbles, step 1) of row r
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int j = 2 * c + half;
            const int sc = byte_of(j < 4 ? ks.sc_lo : ks.sc_hi, j & 3);
            const uint32_t s_hi = (uint32_t)sc >> 3, s_lo = (uint32_t)sc & 7u;
            uint32_t dh[8], dl[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
              uint32_t n = (qw[i] >> (4 * half)) & 0x0F0F0F0Fu;
              if (q5) n |= ((hw[i] >> j) & 0x01010101u) << 4;
              dh[i] = n * s_hi;  // every byte stays below 256: no carry between bytes
              dl[i] = n * s_lo;
            }
            uint8_t* a_hi = stg + (2 * half) * TC_A_TILE;
            uint8_t* a_lo = a_hi + TC_A_TILE;
            *reinterpret_cast<uint4*>(a_hi + tc_tile_off(r, 0)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
            *reinterpret_cast<uint4*>(a_hi + tc_tile_off(r, 1)) = make_uint4(dh[4], dh[5], dh[6], dh[7]);
            *reinterpret_cast<uint4*>(a_lo + tc_tile_off(r, 0)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
            *reinterpret_cast<uint4*>(a_lo + tc_tile_off(r, 1)) = make_uint4(dl[4], dl[5], dl[6], dl[7]);
          }
          // B: parts 0,1 of a token -> step 0 (the low-nibble sub-block), parts 2,3 -> step 1
#pragma unroll
          for (int k = 0; k < 2; k++) {
            const int item = r + 128 * k, tok = item >> 2, part = item & 3;
            *reinterpret_cast<uint4*>(stg + 4 * TC_A_TILE + (part >> 1) * TC_B_TILE + tc_tile_off(tok, part & 1)) = xa[k];
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive_cta(&full[st]);
        }
        // side data of the super-block, read by the epilogue after the block's last MMA: the
        // accumulator set's previous user must be done with it
        if (!tc_wait(&acc_empty[buf], ((blk >> 1) & 1u) ^ 1u, abort, P.err)) goto fill_done;
        {
          uint8_t* sd = side + buf * TC_SIDE_BYTES;
          if (cp == 0) {
            const float d = half_bits_to_float(hdr.x & 0xFFFFu), dmin = half_bits_to_float(hdr.x >> 16);
            *reinterpret_cast<uint4*>(sd + r * 16) = make_uint4(__float_as_uint(d), __float_as_uint(dmin), ks.m_lo, ks.m_hi);
          } else if (r < TC_TOK) {
            // sums of the eight 32-element sub-blocks: bsums[2j] + bsums[2j+1], as 16-bit pairs
            const uint32_t bw[8] = {t_bs0.x, t_bs0.y, t_bs0.z, t_bs0.w, t_bs1.x, t_bs1.y, t_bs1.z, t_bs1.w};
            uint32_t sp[8];
#pragma unroll
            for (int j = 0; j < 8; j++) sp[j] = (uint32_t)(((int)(short)(bw[j] & 0xFFFF) + ((int)bw[j] >> 16)) & 0xFFFF);
            *reinterpret_cast<uint4*>(sd + TC_ROWS * 16 + r * 32) = make_uint4(t_dx, 0, 0, 0);
            *reinterpret_cast<uint4*>(sd + TC_ROWS * 16 + r * 32 + 16) =
                make_uint4(sp[0] | (sp[1] << 16), sp[2] | (sp[3] << 16), sp[4] | (sp[5] << 16), sp[6] | (sp[7] << 16));
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_cta(&side_full[buf]);
        }
      }
    }
  fill_done:;
  } else if (warp < TC_FILL_WARPS + TC_EPI_WARPS) {
    // ---- epilogue warps -----------------------------------------------------------------------
    const int ew = warp - TC_FILL_WARPS;       // 0..7
    const int quarter = warp & 3;              // tensor-memory lanes 32*quarter .. +31 belong to this warp
    const int col0 = (ew >> 2) * 32;           // the 32 tokens this warp finishes
    const int r = quarter * 32 + lane;         // weight row of the tile
    uint32_t blk = 0;
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      int sg = 0;
      while (sg < P.nseg - 1 && tile >= P.tiles_before[sg + 1]) sg++;
      const GemvSeg& S = P.seg[sg];
      const int row = (tile - P.tiles_before[sg]) * TC_ROWS + r;
      float acc[32];
#pragma unroll
      for (int t = 0; t < 32; t++) acc[t] = 0.0f;
      for (int b = 0; b < nb; b++, blk++) {
        const int buf = blk & 1;
        if (!tc_wait(&side_full[buf], (blk >> 1) & 1u, abort, P.err)) goto epi_done;
        if (!tc_wait(&acc_full[buf], (blk >> 1) & 1u, abort, P.err)) goto epi_done;
        tc_fence_after();
        int hi[32], lo[32];
        const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 2 * TC_TOK + col0);
        tc_ld32(taddr, hi);
        tc_ld32(taddr + TC_TOK, lo);
        tc_wait_ld();
        const uint8_t* sd = side + buf * TC_SIDE_BYTES;
        const uint4 ri = *reinterpret_cast<const uint4*>(sd + r * 16);
        const float d_w = __uint_as_float(ri.x), dmin_w = __uint_as_float(ri.y);
#pragma unroll
        for (int t = 0; t < 32; t++) {
          const uint8_t* ti = sd + TC_ROWS * 16 + (col0 + t) * 32;
          const float d_x = *reinterpret_cast<const float*>(ti);
          const uint4 sp = *reinterpret_cast<const uint4*>(ti + 16);
          // matvec.rs:89-103: summ = sum_j m_j * (bsums[2j] + bsums[2j+1])
          int summ = __dp2a_lo((int)sp.x, (int)ri.z, 0);   // sums 0,1 x mins 0,1
          summ = __dp2a_hi((int)sp.y, (int)ri.z, summ);    // sums 2,3 x mins 2,3
          summ = __dp2a_lo((int)sp.z, (int)ri.w, summ);
          summ = __dp2a_hi((int)sp.w, (int)ri.w, summ);
          const int sumi = hi[t] * 8 + lo[t];
          if (P.dbg_sumi && row < S.rows && col0 + t < m) {
            const size_t di = ((size_t)(col0 + t) * S.rows + row) * nb + b;
            P.dbg_sumi[di] = sumi;
            P.dbg_summ[di] = summ;
          }
          acc[t] = fadd(acc[t], k4_term(d_w, dmin_w, d_x, sumi, summ));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(&acc_empty[buf]);
      }
      if (row < S.rows) {
#pragma unroll
        for (int t = 0; t < 32; t++) {
          if (col0 + t < m) {
            float* o = S.out + (size_t)(col0 + t) * S.rows + row;
            *o = P.epilogue == EPI_ACCUM ? fadd(*o, acc[t]) : acc[t];
          }
        }
      }
    }
  epi_done:;
  } else if (lane == 0) {
    // ---- MMA issue (one thread) ----------------------------------------------------------------
    uint32_t it = 0, blk = 0;
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      for (int b = 0; b < nb; b++, blk++) {
        const int buf = blk & 1;
        if (!tc_wait(&acc_empty[buf], ((blk >> 1) & 1u) ^ 1u, abort, P.err)) goto mma_done;
        tc_fence_after();
        const uint32_t d_hi = tmem + (uint32_t)(buf * 2 * TC_TOK), d_lo = d_hi + TC_TOK;
        for (int c = 0; c < 4; c++, it++) {
          const int st = it % TC_STAGES;
          if (!tc_wait(&full[st], (it / TC_STAGES) & 1u, abort, P.err)) goto mma_done;
          tc_fence_after();
          const uint32_t sa = smem_addr(stages + st * TC_STAGE_BYTES);
#pragma unroll
          for (int step = 0; step < 2; step++) {
            const uint64_t db = tc_desc(sa + 4 * TC_A_TILE + step * TC_B_TILE);
            const uint32_t accum = (c | step) != 0 ? 1u : 0u;
            tc_mma_i8(d_hi, tc_desc(sa + (2 * step) * TC_A_TILE), db, accum);
            tc_mma_i8(d_lo, tc_desc(sa + (2 * step + 1) * TC_A_TILE), db, accum);
          }
          tc_commit(&empty[st]);  // the stage may be refilled once these MMAs have read it
        }
        tc_commit(&acc_full[buf]);
      }
    }
  mma_done:
    // Tensor memory is freed after the CTA-wide barrier below: every MMA issued above has to
    // be complete by then, also when a wait gave up half way through a super-block.
    tc_commit(drain);
    for (uint32_t k = 0; k < (1u << 20); ++k)
      if (mbar_try_wait(drain, 0)) break;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(tmem, TC_TMEM_COLS);
}


// ---- prepared operands ----------------------------------------------------------------------
// The digit tiles depend only on the weights, so they can be formed once per model instead of
// once per launch: k4_prepare_kernel writes, for every tile of 128 rows and every
// super-block, the four chunks' operand tiles exactly as a ring stage holds them (4 x 16 KB)
// followed by the rows' side data (2 KB). gemm_k4_prep_kernel then fetches a chunk's tiles
// with one bulk copy onto the stage's mbarrier and streams 2.06 bytes per weight from HBM
// instead of unpacking nibbles; the price is memory (3.7 x the Q4_K bytes), which a 180 GB
// part has. Warp roles there: 16 worker warps (place the activations of the next
// super-block, then read out the accumulators of the current one: 32 rows x 16 tokens per
// warp), one thread that issues the bulk copies, one that issues the MMAs. Measured on the
// gate/up pair of the TinyLlama shape (88 tiles, M = 64): 27 us against 41 us for the
// unpacking kernel. Of those, copies and MMAs are hidden (removing either changes the time
// by about 1 us); the accumulator read-out and f32 terms are 8 us, placing and fetching
// activations 5 us, and the mbarrier hand-overs of a super-block about 0.85 us each with
// everything else removed, so a tile of eight super-blocks cannot finish in less than
// about 11 us however fast the operands arrive. That is why launches of few tiles gain
// nothing here and stay on the mma.sync kernel.
constexpr int TC_PREP_CHUNK = 4 * TC_A_TILE;                       // 16 KB
constexpr int TC_PREP_BLOCK = 4 * TC_PREP_CHUNK + TC_ROWS * 16;    // 66 KB
__host__ __device__ inline size_t tc_prep_bytes(size_t rows, size_t cols) {
  return ((rows + TC_ROWS - 1) / TC_ROWS) * (cols / 256) * (size_t)TC_PREP_BLOCK;
}
constexpr int TP_WORKERS = 16;
constexpr int TP_THREADS = (TP_WORKERS + 2) * 32;
constexpr int TP_STAGES = 8;                   // operands arrive at HBM latency: a deeper ring
constexpr int TP_SMEM_BYTES = TP_STAGES * TC_STAGE_BYTES + 2 * TC_SIDE_BYTES + 256;

// The operand tiles of chunk c (sub-blocks 2c: low nibbles, K step 0; 2c + 1: high nibbles,
// K step 1) of weight row r, written at `a`. qa, qb: the chunk's 32 quant bytes; h0, h1: the
// super-block's 32 high-bit bytes (Q5_K).
__device__ __forceinline__ void tc_write_a(uint8_t* a, int r, int c, const uint4& qa, const uint4& qb, const uint4& h0, const uint4& h1,
                                           const K4Scales& ks, bool q5) {
  const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
  const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int j = 2 * c + half;
    const int sc = byte_of(j < 4 ? ks.sc_lo : ks.sc_hi, j & 3);
    const uint32_t s_hi = (uint32_t)sc >> 3, s_lo = (uint32_t)sc & 7u;
    uint32_t dh[8], dl[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      uint32_t n = (qw[i] >> (4 * half)) & 0x0F0F0F0Fu;
      if (q5) n |= ((hw[i] >> j) & 0x01010101u) << 4;
      dh[i] = n * s_hi;  // every byte stays below 256: no carry between bytes
      dl[i] = n * s_lo;
    }
    uint8_t* a_hi = a + (2 * half) * TC_A_TILE;
    uint8_t* a_lo = a_hi + TC_A_TILE;
    *reinterpret_cast<uint4*>(a_hi + tc_tile_off(r, 0)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
    *reinterpret_cast<uint4*>(a_hi + tc_tile_off(r, 1)) = make_uint4(dh[4], dh[5], dh[6], dh[7]);
    *reinterpret_cast<uint4*>(a_lo + tc_tile_off(r, 0)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
    *reinterpret_cast<uint4*>(a_lo + tc_tile_off(r, 1)) = make_uint4(dl[4], dl[5], dl[6], dl[7]);
  }
}

// Prepared operands of one matrix: block (tile, b) by CTA tile * nb + b, thread (row r, chunk
// pair cp).
__global__ void __launch_bounds__(256) k4_prepare_kernel(const uint8_t* w, int kind, int rows, int cols, uint8_t* out) {
  const int nb = cols >> 8, tile = blockIdx.x / nb, b = blockIdx.x - tile * nb;
  const int r = threadIdx.x & 127, cp = threadIdx.x >> 7;
  const bool q5 = kind == Q5_K;
  const int bs = q5 ? 176 : 144, qoff = (q5 ? 48 : 16) + 64 * cp;
  const int row = tile * TC_ROWS + r;
  uint8_t* dst = out + (size_t)blockIdx.x * TC_PREP_BLOCK;
  if (row >= rows) {
    // rows past the matrix: zero operands (their results are dropped)
    for (int cc = 0; cc < 2; cc++)
      for (int t = 0; t < 4; t++)
        for (int k = 0; k < 2; k++)
          *reinterpret_cast<uint4*>(dst + (2 * cp + cc) * TC_PREP_CHUNK + t * TC_A_TILE + tc_tile_off(r, k)) = make_uint4(0, 0, 0, 0);
    if (cp == 0) *reinterpret_cast<uint4*>(dst + 4 * TC_PREP_CHUNK + r * 16) = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint8_t* wb = w + (size_t)row * nb * bs + (size_t)b * bs;
  const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(wb));
  uint4 qv[4];
#pragma unroll
  for (int i = 0; i < 4; i++) qv[i] = __ldg(reinterpret_cast<const uint4*>(wb + qoff) + i);
  uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0;
  if (q5) {
    h0 = __ldg(reinterpret_cast<const uint4*>(wb + 16));
    h1 = __ldg(reinterpret_cast<const uint4*>(wb + 16) + 1);
  }
  const K4Scales ks = k4_unpack(hdr.y, hdr.z, hdr.w);
#pragma unroll
  for (int cc = 0; cc < 2; cc++) tc_write_a(dst + (2 * cp + cc) * TC_PREP_CHUNK, r, 2 * cp + cc, qv[2 * cc], qv[2 * cc + 1], h0, h1, ks, q5);
  if (cp == 0) {
    const float d = half_bits_to_float(hdr.x & 0xFFFFu), dmin = half_bits_to_float(hdr.x >> 16);
    *reinterpret_cast<uint4*>(dst + 4 * TC_PREP_CHUNK + r * 16) = make_uint4(__float_as_uint(d), __float_as_uint(dmin), ks.m_lo, ks.m_hi);
  }
}

// 16 consecutive columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tc_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(TP_THREADS, 1) gemm_k4_prep_kernel(const GemmTcParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][side data x 2][barriers][tmem base][abort]
  uint8_t* const stages = smem;
  uint8_t* const side = smem + TP_STAGES * TC_STAGE_BYTES;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(side + 2 * TC_SIDE_BYTES);
  uint64_t* const full = bars;                           // [TP_STAGES] copy + activations -> MMA
  uint64_t* const empty = bars + TP_STAGES;              // [TP_STAGES] MMA -> producer and workers
  uint64_t* const acc_full = bars + 2 * TP_STAGES;       // [2] MMA -> workers
  uint64_t* const acc_empty = bars + 2 * TP_STAGES + 2;  // [2] workers -> MMA, producer, workers
  uint64_t* const side_full = bars + 2 * TP_STAGES + 4;  // [2] side data of the super-block written
  uint64_t* const drain = bars + 2 * TP_STAGES + 6;      // all MMAs of the CTA have completed
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TP_STAGES + 7);
  volatile int* const abort = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < TP_STAGES; s++) {
      mbar_init(&full[s], TP_WORKERS / 2 + 1);  // the eight warps that place the chunk's activations + the copy
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], TP_WORKERS);
      mbar_init(&side_full[b], TP_WORKERS + 1);
    }
    mbar_init(drain, 1);
    *abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) tc_alloc(tmem_slot, TC_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  const int nb = P.cols >> 8, m = P.m;
  const size_t x_block = P.x_image ? XK_STRIDE : 292;  // bytes of one activation block
  const int x_qs = P.x_image ? 0 : 4, x_bs = P.x_image ? XK_BSUMS : 260, x_d = P.x_image ? XK_D : 0;

  if (warp < TP_WORKERS) {
    // ---- worker warps ---------------------------------------------------------------------------
    const int t = threadIdx.x;                      // 0..511
    const int item = t & 255, fh = t >> 8;          // activation part `item` of chunks 2 fh and 2 fh + 1
    const int ftok = item >> 2, part = item & 3;
    const int quarter = warp & 3;                   // tensor-memory lanes 32 quarter .. + 31 belong to this warp
    const int col0 = (warp >> 2) * 16;              // the 16 tokens this warp finishes
    const int r = quarter * 32 + lane;              // weight row of the tile
    uint32_t blk = 0;
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      int sg = 0;
      while (sg < P.nseg - 1 && tile >= P.tiles_before[sg + 1]) sg++;
      const GemvSeg& S = P.seg[sg];
      const int row = (tile - P.tiles_before[sg]) * TC_ROWS + r;
      // this thread's activation pieces and (threads 0..63) its token's side data of block b
      auto fetch = [&](int b, uint4 (&xa)[2], uint32_t& dx, uint4& b0, uint4& b1) {
#pragma unroll
        for (int k = 0; k < 2; k++) {
          xa[k] = make_uint4(0, 0, 0, 0);
          if (ftok < m) xa[k] = ldg16_any(P.x + ((size_t)ftok * nb + b) * x_block + x_qs + 64 * (2 * fh + k) + 16 * part);
        }
        dx = 0;
        b0 = make_uint4(0, 0, 0, 0);
        b1 = b0;
        if (t < m) {
          const uint8_t* xb = P.x + ((size_t)t * nb + b) * x_block;
          dx = __ldg(reinterpret_cast<const uint32_t*>(xb + x_d));
          const uint32_t* bsw = reinterpret_cast<const uint32_t*>(xb + x_bs);
          b0 = make_uint4(__ldg(bsw), __ldg(bsw + 1), __ldg(bsw + 2), __ldg(bsw + 3));
          b1 = make_uint4(__ldg(bsw + 4), __ldg(bsw + 5), __ldg(bsw + 6), __ldg(bsw + 7));
        }
      };
      // places the activations and token side data of super-block (tile, b), counter value fb
      auto fill = [&](uint32_t fb, const uint4 (&xa)[2], uint32_t dx, const uint4& b0, const uint4& b1) -> bool {
        const int buf = fb & 1;
        if (!tc_wait(&acc_empty[buf], ((fb >> 1) & 1u) ^ 1u, abort, P.err)) return false;
        uint8_t* sd = side + buf * TC_SIDE_BYTES;
        if (t < TC_TOK) {
          // sums of the eight 32-element sub-blocks: bsums[2j] + bsums[2j+1], as 16-bit pairs
          const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          uint32_t sp[8];
#pragma unroll
          for (int j = 0; j < 8; j++) sp[j] = (uint32_t)(((int)(short)(bw[j] & 0xFFFF) + ((int)bw[j] >> 16)) & 0xFFFF);
          *reinterpret_cast<uint4*>(sd + TC_ROWS * 16 + t * 32) = make_uint4(dx, 0, 0, 0);
          *reinterpret_cast<uint4*>(sd + TC_ROWS * 16 + t * 32 + 16) =
              make_uint4(sp[0] | (sp[1] << 16), sp[2] | (sp[3] << 16), sp[4] | (sp[5] << 16), sp[6] | (sp[7] << 16));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(&side_full[buf]);
#pragma unroll
        for (int k = 0; k < 2; k++) {
          const uint32_t it = fb * 4 + (uint32_t)(2 * fh + k);
          const int st = it % TP_STAGES;
          if (!tc_wait(&empty[st], ((it / TP_STAGES) & 1u) ^ 1u, abort, P.err)) return false;
          uint8_t* stg = stages + st * TC_STAGE_BYTES;
          *reinterpret_cast<uint4*>(stg + 4 * TC_A_TILE + (part >> 1) * TC_B_TILE + tc_tile_off(ftok, part & 1)) = xa[k];
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive_cta(&full[st]);
        }
        return true;
      };
      uint4 c_xa[2], n_xa[2], c_b0, c_b1, n_b0, n_b1;
      uint32_t c_dx, n_dx;
      fetch(0, c_xa, c_dx, c_b0, c_b1);
      if (nb > 1) fetch(1, n_xa, n_dx, n_b0, n_b1);
      if (!fill(blk, c_xa, c_dx, c_b0, c_b1)) goto work_done;
      float acc[16];
#pragma unroll
      for (int k = 0; k < 16; k++) acc[k] = 0.0f;
      for (int b = 0; b < nb; b++, blk++) {
        if (b + 1 < nb) {
          // the next super-block's activations go in before this one's accumulators come out
          c_xa[0] = n_xa[0]; c_xa[1] = n_xa[1]; c_dx = n_dx; c_b0 = n_b0; c_b1 = n_b1;
          if (b + 2 < nb) fetch(b + 2, n_xa, n_dx, n_b0, n_b1);
          if (!fill(blk + 1, c_xa, c_dx, c_b0, c_b1)) goto work_done;
        }
        const int buf = blk & 1;
        if (!tc_wait(&side_full[buf], (blk >> 1) & 1u, abort, P.err)) goto work_done;
        if (!tc_wait(&acc_full[buf], (blk >> 1) & 1u, abort, P.err)) goto work_done;
        tc_fence_after();
        int hi[16], lo[16];
        const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 2 * TC_TOK + col0);
        tc_ld16(taddr, hi);
        tc_ld16(taddr + TC_TOK, lo);
        tc_wait_ld();
        const uint8_t* sd = side + buf * TC_SIDE_BYTES;
        const uint4 ri = *reinterpret_cast<const uint4*>(sd + r * 16);
        const float d_w = __uint_as_float(ri.x), dmin_w = __uint_as_float(ri.y);
#pragma unroll
        for (int k = 0; k < 16; k++) {
          const uint8_t* ti = sd + TC_ROWS * 16 + (col0 + k) * 32;
          const float d_x = *reinterpret_cast<const float*>(ti);
          const uint4 sp = *reinterpret_cast<const uint4*>(ti + 16);
          // matvec.rs:89-103: summ = sum_j m_j * (bsums[2j] + bsums[2j+1])
          int summ = __dp2a_lo((int)sp.x, (int)ri.z, 0);
          summ = __dp2a_hi((int)sp.y, (int)ri.z, summ);
          summ = __dp2a_lo((int)sp.z, (int)ri.w, summ);
          summ = __dp2a_hi((int)sp.w, (int)ri.w, summ);
          const int sumi = hi[k] * 8 + lo[k];
          if (P.dbg_sumi && row < S.rows && col0 + k < m) {
            const size_t di = ((size_t)(col0 + k) * S.rows + row) * nb + b;
            P.dbg_sumi[di] = sumi;
            P.dbg_summ[di] = summ;
          }
          acc[k] = fadd(acc[k], k4_term(d_w, dmin_w, d_x, sumi, summ));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(&acc_empty[buf]);
      }
      if (row < S.rows) {
#pragma unroll
        for (int k = 0; k < 16; k++) {
          if (col0 + k < m) {
            float* o = S.out + (size_t)(col0 + k) * S.rows + row;
            *o = P.epilogue == EPI_ACCUM ? fadd(*o, acc[k]) : acc[k];
          }
        }
      }
    }
  work_done:;
  } else if (warp == TP_WORKERS && lane == 0) {
    // ---- MMA issue (one thread) ----------------------------------------------------------------
    uint32_t it = 0, blk = 0;
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      for (int b = 0; b < nb; b++, blk++) {
        const int buf = blk & 1;
        if (!tc_wait(&acc_empty[buf], ((blk >> 1) & 1u) ^ 1u, abort, P.err)) goto mma_done;
        tc_fence_after();
        const uint32_t d_hi = tmem + (uint32_t)(buf * 2 * TC_TOK), d_lo = d_hi + TC_TOK;
        for (int c = 0; c < 4; c++, it++) {
          const int st = it % TP_STAGES;
          if (!tc_wait(&full[st], (it / TP_STAGES) & 1u, abort, P.err)) goto mma_done;
          tc_fence_after();
          const uint32_t sa = smem_addr(stages + st * TC_STAGE_BYTES);
#pragma unroll
          for (int step = 0; step < 2; step++) {
            const uint64_t db = tc_desc(sa + 4 * TC_A_TILE + step * TC_B_TILE);
            const uint32_t accum = (c | step) != 0 ? 1u : 0u;
            tc_mma_i8(d_hi, tc_desc(sa + (2 * step) * TC_A_TILE), db, accum);
            tc_mma_i8(d_lo, tc_desc(sa + (2 * step + 1) * TC_A_TILE), db, accum);
          }
          tc_commit(&empty[st]);  // the stage may be refilled once these MMAs have read it
        }
        tc_commit(&acc_full[buf]);
      }
    }
  mma_done:
    // Tensor memory is freed after the CTA-wide barrier below: every MMA issued above has to
    // be complete by then, also when a wait gave up half way through a super-block.
    tc_commit(drain);
    for (uint32_t k = 0; k < (1u << 20); ++k)
      if (mbar_try_wait(drain, 0)) break;
  } else if (warp == TP_WORKERS + 1 && lane == 0) {
    // ---- producer (one thread): bulk copies of the prepared operands ------------------------------
    uint32_t it = 0, blk = 0;
    for (int tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
      int sg = 0;
      while (sg < P.nseg - 1 && tile >= P.tiles_before[sg + 1]) sg++;
      const uint8_t* pw = P.prep[sg] + (size_t)(tile - P.tiles_before[sg]) * nb * TC_PREP_BLOCK;
      for (int b = 0; b < nb; b++, blk++) {
        const int buf = blk & 1;
        const uint8_t* pb = pw + (size_t)b * TC_PREP_BLOCK;
        if (!tc_wait(&acc_empty[buf], ((blk >> 1) & 1u) ^ 1u, abort, P.err)) goto prod_done;
        mbar_expect_tx(&side_full[buf], TC_ROWS * 16);
        bulk_g2s(side + buf * TC_SIDE_BYTES, pb + 4 * TC_PREP_CHUNK, TC_ROWS * 16, &side_full[buf]);
        for (int c = 0; c < 4; c++, it++) {
          const int st = it % TP_STAGES;
          if (!tc_wait(&empty[st], ((it / TP_STAGES) & 1u) ^ 1u, abort, P.err)) goto prod_done;
          mbar_expect_tx(&full[st], TC_PREP_CHUNK);
          bulk_g2s(stages + st * TC_STAGE_BYTES, pb + (size_t)c * TC_PREP_CHUNK, TC_PREP_CHUNK, &full[st]);
        }
      }
    }
  prod_done:
    // A wait gave up with bulk copies possibly still in flight towards this CTA's shared
    // memory: give them time to land before the CTA may exit (bounded; never taken in a
    // healthy run).
    if (*abort) {
      const long long t0 = clock64();
      for (uint32_t k = 0; k < (1u << 20) && clock64() - t0 < 400000; ++k) {
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(tmem, TC_TMEM_COLS);
}

}  // namespace aot
