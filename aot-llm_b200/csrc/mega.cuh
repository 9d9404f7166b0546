// One decode step (crates/aot-codegen/src/emit.rs:243-333, 466-486) as a single
// persistent kernel: one CTA per SM, a producer warp that streams this CTA's
// share of every weight matrix of the step through a shared-memory ring with 1-D
// bulk copies (it runs ahead across phases, because weights never depend on
// activations) and consumer warps that do the arithmetic. Activation vectors pass
// from one phase to the next as tagged 64-bit words (value + phase tag in one store),
// so a consumer starts as soon as the words it needs have arrived; the only grid-wide
// barrier left is the one in front of the argmax. All results are bit-identical to the
// reference's CPU path (see blockmath.cuh, seqsum.cuh, expf_exact.cuh).
#pragma once
#include <cuda_fp16.h>

#include "blockmath.cuh"
#include "device_utils.cuh"
#include "expf_exact.cuh"
#include "gemv.cuh"
#include "groupsum.cuh"
#include "ops.cuh"
#include "rowdot.cuh"
#include "rowwide.cuh"
#include "seqsum.cuh"

namespace aot {

// 512 threads (15 consumer warps and the producer warp) leave 128 registers per thread:
// measured faster than 640 or 768 threads, whose register budgets spill in the row products.
#ifndef MEGA_THREADS_N
#define MEGA_THREADS_N 512
#endif
// The gate and up rows of a pair go through the arithmetic side by side when the register
// budget allows it (128 registers per thread up to 512 threads, 80 at 768).
#ifndef MEGA_PAIR_INTERLEAVE
#define MEGA_PAIR_INTERLEAVE (MEGA_THREADS_N <= 512)
#endif

// ---- tagged activation words ---------------------------------------------------------------
// Activation vectors that cross CTAs inside the step travel as 64-bit words {f32 value,
// 32-bit tag}. A writer stores value and tag with one 8-byte store; a reader polls the word
// until it carries the tag of the phase it expects. Data and "ready" arrive together, so
// no fence, counter or grid-wide barrier sits between a matrix product and its consumers:
// one trip through L2 instead of the three of a fence + flag + data scheme (measured:
// about 7 K cycles per hand-over with per-CTA flags, most of it the two fences).
// A reader asks for all of its words at once and asks again, for all of them, until every
// tag matches; examining them one after the other would cost one L2 round trip per word
// that was still missing at the first look.
// Tags are unique per (launch, phase): (launch count << 11) | phase id, phase id >= 1;
// a zeroed buffer therefore never matches.
//
// Every wait is bounded: `abort` points at two shared words of the CTA, [0] = a wait of this
// CTA has given up, [1] = polls (about a microsecond each) before a wait gives up. The host
// raises the limit when several GPUs step together: a rank whose host thread is late must
// not make its peers give up.
typedef unsigned long long LLWord;

__device__ __forceinline__ void ll_store(LLWord* p, float v, uint32_t tag) {
  const LLWord w = ((LLWord)tag << 32) | (LLWord)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ LLWord ll_load(const LLWord* p) {
  LLWord w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ void ll_load2(const LLWord* p, LLWord& a, LLWord& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// Value of a word whose tag may be ignored (this CTA wrote it in an earlier phase).
__device__ __forceinline__ float ll_value(const LLWord* p) { return __uint_as_float((uint32_t)ll_load(p)); }

// A wait gave up: the CTA's abort flag and the device error word are set; every later wait
// then returns at once, so the kernel drains.
__device__ __noinline__ void ll_give_up(volatile int* abort, int* err) {
  if (!*abort) {
    *abort = 1;
    if (err) atomicOr(err, DEVERR_GRID_TIMEOUT);
  }
}
// One word.
__device__ __forceinline__ float ll_wait(const LLWord* p, uint32_t tag, volatile int* abort, int* err) {
  LLWord w = ll_load(p);
  if ((uint32_t)(w >> 32) != tag) {
    const uint32_t limit = (uint32_t)abort[1];
    for (uint32_t it = 0;; ++it) {
      w = ll_load(p);
      if ((uint32_t)(w >> 32) == tag) break;
      if (it >= limit || *abort) {
        ll_give_up(abort, err);
        break;
      }
    }
  }
  return __uint_as_float((uint32_t)w);
}
// Eight consecutive words (64-byte aligned), requested together in every round.
__device__ __forceinline__ void ll_wait8(const LLWord* p, uint32_t tag, float (&v)[8], volatile int* abort, int* err) {
  LLWord w[8];
  const uint32_t limit = (uint32_t)abort[1];
  for (uint32_t it = 0;; ++it) {
#pragma unroll
    for (int i = 0; i < 4; i++) ll_load2(p + 2 * i, w[2 * i], w[2 * i + 1]);
    bool all = true;
#pragma unroll
    for (int i = 0; i < 8; i++) all = all && (uint32_t)(w[i] >> 32) == tag;
    if (all) break;
    if (it >= limit || *abort) {
      ll_give_up(abort, err);
      break;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) v[i] = __uint_as_float((uint32_t)w[i]);
}

// Rows [c0, c1) of a vector of `span` rows that belong to this CTA: an even split with
// the remainder spread over the first CTAs, so every CTA owns a row when span >= gridDim.x.
__device__ __forceinline__ void cta_rows(int span, int& c0, int& c1) {
  const int base = span / (int)gridDim.x, rem = span - base * (int)gridDim.x, b = (int)blockIdx.x;
  c0 = b * base + min(b, rem);
  c1 = c0 + base + (b < rem ? 1 : 0);
}

// ---- tagged words across GPUs -----------------------------------------------------------------
// Row-sharded models (each GPU holds some heads and some FFN rows) produce partial rows of
// attn_output and ffn_down. A rank stores its partial of row i as a tagged word into slot
// [product][its rank][i] of every rank's inbox (plain 8-byte stores to peer memory over
// NVLink); the CTA that owns row i on each rank waits for the world's words, adds them in
// rank order (so every rank gets the same bits) and publishes the new residual row locally.
constexpr int TP_MAX_WORLD = 8;  // ranks of one exchange (one NVSwitch domain)
struct TpExchange {
  int world, rank, dim;
  int head_sharded;  // the output head is split by vocabulary rows: ranks exchange their best (logit, id)
  int head_row0;     // first vocabulary row of this rank's slice
  int arg_off;       // word offset of the [world][2] argmax slots behind the partial rows
  int pad_[2];       // keeps the members behind this struct on their former 16-byte phase
  LLWord* inbox[TP_MAX_WORLD];  // inbox of rank d (peer mapping), layout [2 products][world][dim], then [world][2]
};

__device__ __forceinline__ void ll_store_sys(LLWord* p, float v, uint32_t tag) {
  const LLWord w = ((LLWord)tag << 32) | (LLWord)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ float ll_wait_sys(const LLWord* p, uint32_t tag, volatile int* abort, int* err) {
  LLWord w;
  uint32_t it = 0;
  const uint32_t limit = (uint32_t)abort[1];
  for (;;) {
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    if ((uint32_t)(w >> 32) == tag) break;
    if (++it >= limit || ((it & 31u) == 31u && *abort)) {
      if (!*abort) {
        *abort = 1;
        if (err) atomicOr(err, DEVERR_GRID_TIMEOUT);
      }
      break;
    }
  }
  return __uint_as_float((uint32_t)w);
}

// The one-kernel step walks all of its code once per layer, so the code has to stay inside
// the SM's instruction cache: everything large that is used from more than one place is
// kept out of line.
__device__ __noinline__ float silu_mul_call(float g, float u) { return fmul(fdiv(g, fadd(1.0f, expf_exact(-g))), u); }
__device__ __noinline__ float group_seq_sum_call(const float* p, int n, SeqSumScratch* sc, int tid, int nthreads, int bar_id,
                                                 unsigned long long* prof) {
  return group_seq_sum(p, n, sc, CtaGroup{tid, nthreads, bar_id}, prof);
}
__device__ __noinline__ float dequant_elem_call(int kind, const uint8_t* row, size_t e) { return dequant_elem(kind, row, e); }

// ---- step description (built once by the host, lives in global memory) ------------------
// One matrix-product phase as both the producer and the consumers see it. The row
// space (concatenated rows, or shared rows in pair mode) is split evenly over the
// grid; a CTA walks its share in tiles of `tile_rows` rows.
struct MegaOp {
  GemvSeg seg[3];
  uint32_t row_bytes[3];
  int nseg, pair, cols, span_rows, rows_per_cta, tile_rows, epilogue;
  int ll;  // outputs are tagged words (seg[].out points at LLWord), not plain floats
  int cta_base, cta_rem;  // span_rows / grid and span_rows % grid: CTA b owns cta_base (+1 when b < cta_rem) rows
  // derived by the host so that no consumer warp divides: blocks per row, stride of a row's
  // terms in the warp's strip, units a strip holds, tiles of a CTA with cta_base / cta_base + 1 rows
  int nb, tstride, cap, n_tiles_lo, n_tiles_hi;
  // parity export (single plain matrix only): integer block sums per (row, block), or null
  int* dbg_sumi;
  int* dbg_summ;
};

struct StepLayer {
  const float* attn_norm;
  const float* ffn_norm;
  const float* q_norm;
  const float* k_norm;
  MegaOp qkv, wo, gu, down;
};

struct StepParams {
  int dim, hidden, n_layer, n_head, n_kv_head, head_dim, rot_dim, vocab, n_ctx;
  float eps;
  int qk_norm, neox;
  const StepLayer* layers;
  const float* output_norm;
  const MegaOp* out_op;
  const uint8_t* token_embd;
  int embd_kind;
  size_t embd_row_bytes;
  LLWord *xl, *ql, *kl, *vl, *attl, *hbl;  // tagged activation vectors (residual, q, k, v, attention out, hidden)
  float *x;                                // plain copy of the final residual stream, for readers outside the kernel
  float *logits, *k_cache, *v_cache;
  unsigned* epoch;                         // launch count; bumped by CTA 0 when the kernel ends
  TpExchange tp;                           // world > 1: this GPU holds one shard of the model
  const float* rope_table;
  int* step;  // {token, pos, n_generated}
  int* history;
  int history_cap;
  int* out_token;
  int want_logits, with_argmax;
  unsigned* grid_bar;  // arrival counter, zero at launch
  int* err;
  int n_stages, stage_bytes;
  int scratch_bytes;   // f32 scratch region (norm rows, attention)
  int small_floats;    // floats of the scratch region's head (norm rows; q, k, v, squares, scores); the rest stages K and V rows
  int stage_floats;    // floats of the K/V staging area
  int v_chunk;         // positions per staged K or V chunk when a head's rows do not fit the staging area
  int fast;            // FastBits: which sequential f32 loops may be reordered
  int spin_limit;      // polls before a tagged-word wait gives up
  int table_bytes;     // bytes of the StepLayer table staged in shared memory (n_layer + 1 entries)
  unsigned long long* prof;  // optional: cycles per phase, accumulated by one CTA
  int prof_cta;
  unsigned long long* timeline;  // optional: [grid][16] global-timer stamps at the phase boundaries of one layer
  int timeline_layer;
  LLWord* scl;  // [n_head][n_ctx] attention scores, when several CTAs share a head
};

// ---- shared-memory ring --------------------------------------------------------------------
// What a ring stage holds, written by the producer warp before it arms the stage and read
// by the consumers after the stage's barrier completes: up to three parts (segments of a
// concatenated row space, or the gate and up rows of a pair), each a run of whole rows, and
// one record per unit (a row, or a gate/up row pair) with everything a consumer warp needs:
// the producer's 32 lanes do the index arithmetic off the consumers' path.
struct TileUnit {
  uint32_t row[2];  // shared address of the unit's row(s), weight kind in bits 24..31
  float* out;       // where the row's result goes (first matrix of a pair)
};
constexpr int TILE_MAX_UNITS = 32;
struct TileDesc {
  uint32_t base[3];  // shared address of the part's first row
  int row0[3];       // index of that row inside its segment
  int rows[3];
  int seg[3];
  int u0, n_units;   // CTA-relative index of the tile's first unit, and the number of units
  int pad[2];
  uint8_t first[32];  // per consumer warp: its first unit in this tile (then every n_warps-th)
  TileUnit unit[TILE_MAX_UNITS];
};
static_assert(sizeof(TileDesc) == 608, "TileDesc layout");

struct Ring {
  uint8_t* stages;
  uint64_t* full;
  uint64_t* empty;
  TileDesc* desc;
  int n_stages, stage_bytes;
  volatile int* abort;  // set when any bounded wait of this CTA expired
  int* err;
};

// Position of a producer or consumer in the ring: stage index and use parity.
struct RingPos {
  int st;
  uint32_t parity;
  __device__ __forceinline__ void advance(int n_stages) {
    if (++st == n_stages) {
      st = 0;
      parity ^= 1u;
    }
  }
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool ring_wait(const Ring& R, uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*R.abort) return false;
  }
  *R.abort = 1;
  if (R.err) atomicOr(R.err, DEVERR_MBAR_TIMEOUT);
  return false;
}

// Rows [c0, c1) of the op's row space that belong to this CTA.
__device__ __forceinline__ void op_cta_rows(const MegaOp& op, int& c0, int& c1) {
  const int b = (int)blockIdx.x;
  c0 = b * op.cta_base + min(b, op.cta_rem);
  c1 = c0 + op.cta_base + (b < op.cta_rem ? 1 : 0);
}

// Before a CTA returns, every bulk copy it requested into its shared memory must have
// landed: the producer (lane 0) waits, with a limit, for the last arrival it armed on each
// stage. After a normal run they have all completed long ago; this matters when a wait
// gave up and the consumers left tiles unread.
__device__ __forceinline__ void produce_drain(const Ring& R, const RingPos& pp, uint32_t tiles_issued) {
  for (int st = 0; st < R.n_stages; st++) {
    if ((uint32_t)st >= tiles_issued) break;  // never armed
    const uint32_t parity = st < pp.st ? pp.parity : pp.parity ^ 1u;  // parity of the stage's last use
    for (uint32_t it = 0; it < (1u << 20); ++it)
      if (mbar_try_wait(&R.full[st], parity)) break;
  }
}

// Producer side (the whole producer warp): request every tile of this CTA's share of `op`
// and describe it for the consumers. Lane 0 waits for the stage and issues the copies, part
// by part; every lane then writes one unit record; the stage's single arrival, which
// carries the byte count of all copies, comes last (a barrier's pending byte count may run
// negative in between).
__device__ __forceinline__ void produce_op(const MegaOp& op, const Ring& R, RingPos& pp, int n_consumers, uint32_t& tiles_issued) {
  const int lane = threadIdx.x & 31;
  int c0, c1;
  op_cta_rows(op, c0, c1);
  const int nseg = op.nseg, pair = op.pair, tile_rows = op.tile_rows;
#pragma unroll 1
  for (int t0 = c0; t0 < c1; t0 += tile_rows) {
    int ok = 1;
    if (lane == 0) ok = ring_wait(R, &R.empty[pp.st], pp.parity ^ 1u) ? 1 : 0;
    if (!__shfl_sync(0xffffffffu, ok, 0)) return;
    const int t1 = min(t0 + tile_rows, c1);
    TileDesc& D = R.desc[pp.st];
    uint8_t* const stage = R.stages + (size_t)pp.st * R.stage_bytes;
    // parts: the two matrices of a pair share the row range; concatenated segments split it
    // (every lane computes them; lane 0 issues the copies)
    uint32_t total = 0, off = 0;
    int np = 0, base = 0;
    // this lane's unit: rows [t0 + lane] of the row space
    const int my = t0 + lane;
    uint32_t my_row[2] = {0u, 0u};
    float* my_out = nullptr;
#pragma unroll 1
    for (int sgi = 0; sgi < nseg; sgi++) {
      const int rows = op.seg[sgi].rows;
      const int a = pair ? t0 : max(t0, base) - base, b = pair ? t1 : min(t1, base + rows) - base;
      if (a < b) {
        const uint32_t rb = op.row_bytes[sgi];
        const uint8_t* src = op.seg[sgi].w + (size_t)a * rb;
        const uint32_t len = (uint32_t)(b - a) * rb, sup = bulk_superset_bytes(src, len);
        const uint32_t pbase = smem_addr(stage + off) + ((uint32_t)(uintptr_t)src & 15u);
        if (lane == 0) {
          D.base[np] = pbase;
          D.row0[np] = a;
          D.rows[np] = b - a;
          D.seg[np] = sgi;
          bulk_g2s_superset(stage + off, src, len, &R.full[pp.st]);
        }
        // does this lane's unit lie in the part?
        const int lr = pair ? lane : my - base - a;
        if (lr >= 0 && lr < b - a && my < t1) {
          my_row[pair ? sgi : 0] = (pbase + (uint32_t)lr * rb) | ((uint32_t)op.seg[sgi].kind << 24);
          if (!pair || sgi == 0)
            my_out = op.ll ? reinterpret_cast<float*>(reinterpret_cast<LLWord*>(op.seg[sgi].out) + a + lr) : op.seg[sgi].out + a + lr;
        }
        off += sup + 16;
        total += sup;
        np++;
      }
      base += rows;
    }
    if (lane == 0) {
      for (int i = np; i < 3; i++) D.rows[i] = 0;
      D.u0 = t0 - c0;
      D.n_units = t1 - t0;
    }
    if (my < t1) {
      TileUnit U;
      U.row[0] = my_row[0];
      U.row[1] = my_row[1];
      U.out = my_out;
      D.unit[lane] = U;
    }
    if (lane < n_consumers) {
      const int f = (lane - (t0 - c0) % n_consumers + n_consumers) % n_consumers;
      D.first[lane] = (uint8_t)(f < t1 - t0 ? f : 255);
    }
    __syncwarp();
    if (lane == 0) mbar_expect_tx(&R.full[pp.st], total);
    tiles_issued++;
    pp.advance(R.n_stages);
  }
}

// Consumer side (every consumer warp). The rows (gate/up row pairs in pair mode) of this
// CTA's share are dealt to the warps round robin, continuing across tiles, and a warp takes
// a whole row: four lanes per super-block with the activation slices in registers
// (rowdot.cuh); the gate and up rows of a pair go through the arithmetic side by side.
// Block terms are parked in the warp's strip `wterms`; when the strip is full or the
// product ends, lane i adds the terms of parked row i in block order and runs the epilogue
// (residual add, SiLU gate, exchange with the other ranks). `sx` holds the Q8_K images of
// the activation vector; `op` lives in shared memory.
constexpr int WARP_TERMS_FLOATS = 128;  // strip per consumer warp

// Lane i finishes parked unit i: `my_out` is the address of its output word, `my_old` the
// residual value asked for when the unit was parked (ACCUM into tagged words only).
template <bool TP>
__device__ __forceinline__ void warp_flush(const MegaOp& op, const float* wterms, int pend, int nb, int tstride, uint32_t tag,
                                           const TpExchange* tpx, int which, float* my_out, float my_old, float* part, int part_row0) {
  __syncwarp();
  const int lane = threadIdx.x & 31;
  if (op.pair) {
    // lanes 0..15 add the gate rows, lanes 16..31 the matching up rows
    const int i = lane & 15, mt = lane >> 4;
    float v = 0.0f;
    if (i < pend) v = terms_seq_sum(wterms + (2 * i + mt) * tstride, nb);
    const float up = __shfl_down_sync(0xffffffffu, v, 16);
    if (lane < pend) {
      const float hv = op.epilogue == EPI_SILU_MUL ? silu_mul_call(v, up) : v;
      if (op.ll) {
        ll_store(reinterpret_cast<LLWord*>(my_out), hv, tag);
      } else {
        *my_out = hv;
        op.seg[1].out[my_out - op.seg[0].out] = up;
      }
    }
  } else if (lane < pend) {
    const float v = terms_seq_sum(wterms + lane * tstride, nb);
    if (TP && op.ll && tpx && op.epilogue == EPI_ACCUM) {
      // a partial row of a sharded product: parked for the CTA's hand-over to the ranks, which
      // sends the CTA's rows as contiguous words (a warp's own rows are n_warps apart: one
      // 8-byte NVLink write each would cost a packet per row and rank)
      part[(int)(reinterpret_cast<LLWord*>(my_out) - reinterpret_cast<LLWord*>(op.seg[0].out)) - part_row0] = v;
    } else if (op.ll) {
      // a residual row is only ever written by its owner, so its old value needs no tag check
      ll_store(reinterpret_cast<LLWord*>(my_out), op.epilogue == EPI_ACCUM ? fadd(my_old, v) : v, tag);
    } else {
      *my_out = op.epilogue == EPI_ACCUM ? fadd(__ldcg(my_out), v) : v;
    }
  }
  __syncwarp();
}

template <bool TP = false>
__device__ __forceinline__ void consume_op(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, float* wterms, int warp,
                                           int n_warps, uint32_t tag, const TpExchange* tpx = nullptr, int which = 0,
                                           SubProf sp = SubProf{nullptr, 0}, float* part = nullptr, int part_row0 = 0) {
  sp.last = clock64();
  const int pair = op.pair, nb = op.nb, ll = op.ll;
  const int lane = threadIdx.x & 31;
  const int mats = pair ? 2 : 1;
  const int tstride = op.tstride;  // odd, so the lane-parallel reads of the flush spread over the banks
  const int cap = op.cap;
  const uint32_t sxa = smem_addr(sx);
  const bool accum_ll = !pair && ll && op.epilogue == EPI_ACCUM && !(TP && tpx);
  YCache yc;
  yc.lay = YL_NONE;
  yc.g0 = -1;
  int pend = 0;
  float* my_out = nullptr;
  float my_old = 0.0f;
  const int n_tiles = (int)blockIdx.x < op.cta_rem ? op.n_tiles_hi : op.n_tiles_lo;
#pragma unroll 1
  for (int tile = 0; tile < n_tiles; tile++) {
    sp.mark(18);
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    sp.mark(25);
    const TileDesc& D = R.desc[cp.st];
    const int n_units = D.n_units;
#pragma unroll 1
    for (int i = D.first[warp]; i < n_units; i += n_warps) {
      const TileUnit U = D.unit[i];
      if (lane == pend) {
        // this lane will finish the unit: note where its result goes
        my_out = U.out;
        if (accum_ll) my_old = ll_value(reinterpret_cast<const LLWord*>(my_out));
      }
      float* const tdst = wterms + pend * mats * tstride;
      const int kind = (int)(U.row[0] >> 24);
      sp.mark(18);
      if (pair) {
#if MEGA_PAIR_INTERLEAVE
        const uint32_t rows2[2] = {U.row[0] & 0xFFFFFFu, U.row[1] & 0xFFFFFFu};
        float* const t2[2] = {tdst, tdst + tstride};
        warp_rows_terms<2>(kind, rows2, sxa, nb, yc, t2);
#else
#pragma unroll 1
        for (int mt = 0; mt < 2; mt++) {
          const uint32_t rows1[1] = {U.row[mt] & 0xFFFFFFu};
          float* const t1[1] = {tdst + mt * tstride};
          warp_rows_terms<1>(kind, rows1, sxa, nb, yc, t1);
        }
#endif
      } else {
        const uint32_t rows1[1] = {U.row[0] & 0xFFFFFFu};
        float* const t1[1] = {tdst};
        const int drow[1] = {op.dbg_sumi ? (int)(U.out - op.seg[0].out) : 0};
        warp_rows_terms<1>(kind, rows1, sxa, nb, yc, t1, op.dbg_sumi, op.dbg_summ, drow);
      }
      sp.mark(27);
      if (++pend == cap) {
        warp_flush<TP>(op, wterms, pend, nb, tstride, tag, tpx, which, my_out, my_old, part, part_row0);
        pend = 0;
        sp.mark(30);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
  sp.mark(18);
  if (pend) warp_flush<TP>(op, wterms, pend, nb, tstride, tag, tpx, which, my_out, my_old, part, part_row0);
  sp.mark(30);
}

// ---- grid-wide barrier for the consumer warps ---------------------------------------------
// Arrival counter in global memory, zero at launch, never reset: barrier number k
// completes when it reaches k * gridDim.x. The spin is bounded; when it gives up the
// error word is set and every later barrier returns at once, so the kernel drains.
__device__ __forceinline__ bool grid_sync(const StepParams& P, const CtaGroup& g, unsigned& target, volatile int* abort) {
  g.sync();
  if (g.tid == 0) {
    target += gridDim.x;
    if (!*abort) {
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.grid_bar) : "memory");
      bool ok = false;
      for (uint32_t it = 0; it < (1u << 24); ++it) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.grid_bar) : "memory");
        if (v >= target) {
          ok = true;
          break;
        }
        if ((it & 1023u) == 1023u && *(volatile int*)P.err) break;
      }
      if (!ok) {
        *abort = 1;
        atomicOr(P.err, DEVERR_GRID_TIMEOUT);
      }
    }
  }
  g.sync();
  return !*abort;
}

// ---- activation phases -----------------------------------------------------------------------
struct MegaSmem {
  uint8_t* sx;          // Q8_K images of the current activation vector
  float* scr;           // f32 scratch
  SeqSumScratch* ss;
  float* red;           // 64 floats: per-warp partials of a reduction; partial rows parked for the cross-rank hand-over
  volatile int* abort;  // this CTA gave up on a bounded wait
  int* err;             // device error word
};

// Which of the reference's sequential f32 loops may be evaluated in another order
// (StepParams::fast). 0 reproduces every loop bit for bit; each bit trades one loop for a
// tree or split form whose result differs in the last bits only.
enum FastBits : int {
  FAST_NORM_SUM = 1,     // sum of squares of rmsnorm (ops.rs:10-13)
  FAST_SOFTMAX_SUM = 2,  // softmax denominator (ops.rs:103-107)
};

// Sum of the `nw` per-warp partials in red[0..nw), the same order in every thread.
__device__ __forceinline__ float red_sum(const float* red, int nw) {
  float s = 0.0f;
  for (int w = 0; w < nw; w++) s = fadd(s, red[w]);
  return s;
}

// quant.rs:248-283 for the 256 values a warp holds (lane l: elements 8l..8l+7), written as
// a block image.
__device__ __forceinline__ void quantize_block_call(float v0, float v1, float v2, float v3, float v4, float v5, float v6, float v7,
                                                    uint8_t* dst) {
  const float v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
  warp_quantize_q8k_vals(v, dst, 1);
}

// x -> rmsnorm -> Q8_K images in shared memory (ops.rs:7-18 then quant.rs:248-283).
// `src` holds tagged words other CTAs publish under `tag`; for the embedding the row is
// already in scr[0..n). `mirror`, when given, receives a plain copy of the row. The warp
// that owns a super-block keeps its 256 values in registers from the load to the quantized
// image (at most two super-blocks per warp: n <= 512 * warps).
__device__ __forceinline__ void phase_norm_quant(const LLWord* src, uint32_t tag, bool src_in_scr, float* mirror, const float* w,
                                                 int n, float eps, int fast, const MegaSmem& M, const CtaGroup& g,
                                                 SubProf sp = SubProf{nullptr, 0}, unsigned long long* walker_prof = nullptr) {
  sp.last = clock64();
  float* row = M.scr;
  float* sq = M.scr + n;
  const int warp = g.tid >> 5, nw = g.nthreads >> 5, lane = g.tid & 31, nblk = n >> 8;
  float v[2][8];
  float4 w0[2], w1[2];
  float part = 0.0f;
#pragma unroll
  for (int k = 0; k < 2; k++) {
    const int b = warp + k * nw;
    if (b < nblk) {
      // the norm weights are requested before the wait on the row
      w0[k] = __ldg(reinterpret_cast<const float4*>(w + b * 256 + 8 * lane));
      w1[k] = __ldg(reinterpret_cast<const float4*>(w + b * 256 + 8 * lane) + 1);
    }
  }
#pragma unroll
  for (int k = 0; k < 2; k++) {
    const int b = warp + k * nw;
    if (b < nblk) {
      const int e0 = b * 256 + 8 * lane;
      if (src_in_scr) {
        const float4 a0 = *reinterpret_cast<const float4*>(row + e0), a1 = *reinterpret_cast<const float4*>(row + e0 + 4);
        v[k][0] = a0.x; v[k][1] = a0.y; v[k][2] = a0.z; v[k][3] = a0.w;
        v[k][4] = a1.x; v[k][5] = a1.y; v[k][6] = a1.z; v[k][7] = a1.w;
      } else {
        ll_wait8(src + e0, tag, v[k], M.abort, M.err);
      }
      if (mirror) {
        *reinterpret_cast<float4*>(mirror + e0) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
        *reinterpret_cast<float4*>(mirror + e0 + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
      }
      if (fast & FAST_NORM_SUM) {
#pragma unroll
        for (int i = 0; i < 8; i++) part = fadd(part, fmul(v[k][i], v[k][i]));
      } else {
        *reinterpret_cast<float4*>(sq + e0) =
            make_float4(fmul(v[k][0], v[k][0]), fmul(v[k][1], v[k][1]), fmul(v[k][2], v[k][2]), fmul(v[k][3], v[k][3]));
        *reinterpret_cast<float4*>(sq + e0 + 4) =
            make_float4(fmul(v[k][4], v[k][4]), fmul(v[k][5], v[k][5]), fmul(v[k][6], v[k][6]), fmul(v[k][7], v[k][7]));
      }
    }
  }
  sp.mark(16);
  float ss;
  if (fast & FAST_NORM_SUM) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = fadd(part, __shfl_xor_sync(0xffffffffu, part, o));
    if (lane == 0) M.red[warp] = part;
    g.sync();
    ss = red_sum(M.red, nw);
  } else {
    ss = group_seq_sum_call(sq, n, M.ss, g.tid, g.nthreads, g.bar_id, walker_prof ? walker_prof : sp.prof);  // opens with a barrier
    sp.last = clock64();
  }
  sp.mark(17);
  const float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)n), eps)));
#pragma unroll
  for (int k = 0; k < 2; k++) {
    const int b = warp + k * nw;
    if (b < nblk)
      quantize_block_call(fmul(fmul(v[k][0], r), w0[k].x), fmul(fmul(v[k][1], r), w0[k].y), fmul(fmul(v[k][2], r), w0[k].z),
                          fmul(fmul(v[k][3], r), w0[k].w), fmul(fmul(v[k][4], r), w1[k].x), fmul(fmul(v[k][5], r), w1[k].y),
                          fmul(fmul(v[k][6], r), w1[k].z), fmul(fmul(v[k][7], r), w1[k].w), M.sx + b * XK_STRIDE);
  }
  g.sync();
  sp.mark(19);
}

// A vector other CTAs publish under `tag` -> Q8_K images.
__device__ __forceinline__ void phase_quant(const LLWord* src, uint32_t tag, int n, const MegaSmem& M, const CtaGroup& g) {
  const int warp = g.tid >> 5, nw = g.nthreads >> 5, lane = g.tid & 31;
  for (int b = warp; b < n / 256; b += nw) {
    float v[8];
    ll_wait8(src + b * 256 + 8 * lane, tag, v, M.abort, M.err);
    quantize_block_call(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], M.sx + b * XK_STRIDE);
  }
  g.sync();
}

// Stage rows [c0, c0 + cn) of one KV head (row `pos` comes from `cur`, the row of the token
// being decoded, which is not in the cache yet) into `buf` with row stride `stride` floats.
// Cached rows travel with cp.async (no registers, completion by cp.async.wait_group), so
// the next chunk loads while the current one is consumed.
__device__ __forceinline__ void stage_kv_rows(float* buf, int stride, const float* cache, size_t kvd, int head_off, int hd4,
                                              int c0, int cn, int pos, const float* cur, int tid, int T) {
  for (int j = tid; j < cn * hd4; j += T) {
    const int t = j / hd4, i4 = j - t * hd4, tt = c0 + t;
    float* dst = buf + t * stride + 4 * i4;
    if (tt == pos) *reinterpret_cast<float4*>(dst) = reinterpret_cast<const float4*>(cur)[i4];
    else asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(cache + (size_t)tt * kvd + head_off + 4 * i4) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// Sum of p[0..n) (shared memory, written by any thread of the group) returned to every
// thread: in the reference's sequential order, or as a tree when `tree` is set. Longer
// sequential sums go through the chunked algorithm of groupsum.cuh; up to SEQ_CHAIN_MAX
// terms one thread's plain add chain (4 cycles per term) is quicker than its set-up.
constexpr int SEQ_CHAIN_MAX = 256;
__device__ __forceinline__ float cta_sum(const float* p, int n, bool tree, const MegaSmem& M, const CtaGroup& g) {
  if (!tree && n > SEQ_CHAIN_MAX) return group_seq_sum_call(p, n, M.ss, g.tid, g.nthreads, g.bar_id, nullptr);
  g.sync();
  if (tree) {
    float a = 0.0f;
    for (int i = g.tid; i < n; i += g.nthreads) a = fadd(a, p[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fadd(a, __shfl_xor_sync(0xffffffffu, a, o));
    if ((g.tid & 31) == 0) M.red[g.tid >> 5] = a;
    g.sync();
    return red_sum(M.red, g.nthreads >> 5);
  }
  if (g.tid == 0) {
    float s = 0.0f;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
      const float4 a = *reinterpret_cast<const float4*>(p + i), b = *reinterpret_cast<const float4*>(p + i + 4);
      s = fadd(s, a.x); s = fadd(s, a.y); s = fadd(s, a.z); s = fadd(s, a.w);
      s = fadd(s, b.x); s = fadd(s, b.y); s = fadd(s, b.z); s = fadd(s, b.w);
    }
    for (; i < n; i++) s = fadd(s, p[i]);
    M.red[40] = s;
  }
  g.sync();
  return M.red[40];
}

// Softmax over sc[0..n) in place (ops.rs:98-112): `lmax` is this thread's maximum of the
// scores it wrote. Ends with the scaled values written; callers put a barrier before
// other threads read them.
__device__ __forceinline__ void softmax_rows(float* sc, int n, float lmax, int fast, const MegaSmem& M, const CtaGroup& g) {
  const int tid = g.tid, T = g.nthreads;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
  if ((tid & 31) == 0) M.red[tid >> 5] = lmax;
  g.sync();
  float mx = M.red[0];
  for (int w = 1; w < (T >> 5); w++) mx = fmaxf(mx, M.red[w]);
  for (int t = tid; t < n; t += T) sc[t] = expf_exact(fsub(sc[t], mx));
  const float sum = cta_sum(sc, n, (fast & FAST_SOFTMAX_SUM) != 0, M, g);  // opens with a barrier
  const float inv = fdiv(1.0f, sum);
  g.sync();
  for (int t = tid; t < n; t += T) sc[t] = fmul(sc[t], inv);
}

// o + sum over t < cn of a[t] * v[t * stride], positions in order (ops.rs:208-214): eight
// products, then their adds; the add chain is the only dependent work and the compiler's
// own unrolling of this plain loop overlaps the loads of later rounds with it (measured:
// 8 cycles per term against 12 to 14 for hand-pipelined or non-unrolled forms). `a` is
// 16-byte aligned.
__device__ __forceinline__ float value_mix(float o, const float* a, const float* v, int stride, int cn) {
  int t = 0;
  for (; t + 8 <= cn; t += 8) {
    const float4 x = *reinterpret_cast<const float4*>(a + t), y = *reinterpret_cast<const float4*>(a + t + 4);
    const float p0 = fmul(x.x, v[(t + 0) * stride]), p1 = fmul(x.y, v[(t + 1) * stride]);
    const float p2 = fmul(x.z, v[(t + 2) * stride]), p3 = fmul(x.w, v[(t + 3) * stride]);
    const float p4 = fmul(y.x, v[(t + 4) * stride]), p5 = fmul(y.y, v[(t + 5) * stride]);
    const float p6 = fmul(y.z, v[(t + 6) * stride]), p7 = fmul(y.w, v[(t + 7) * stride]);
    o = fadd(o, p0); o = fadd(o, p1); o = fadd(o, p2); o = fadd(o, p3);
    o = fadd(o, p4); o = fadd(o, p5); o = fadd(o, p6); o = fadd(o, p7);
  }
  for (; t < cn; t++) o = fadd(o, fmul(a[t], v[t * stride]));
  return o;
}

// Which of `nd` head dimensions this thread mixes, or -1: the dimensions are spread over
// the group's warps, 8 (or 16, or 32) lanes of each, so that the per-warp instruction
// streams run on all four schedulers instead of one or two.
__device__ __forceinline__ int mix_dim(int tid, int T, int nd) {
  const int nwarps = T >> 5;
  const int per = 8 * nwarps >= nd ? 8 : (16 * nwarps >= nd ? 16 : 32);
  const int lane = tid & 31, d = (tid >> 5) * per + lane;
  return lane < per && d < nd ? d : -1;
}

// q.k over one head (ops.rs:160-166): products first (independent), then the adds in
// element order. `kchunk(j)` returns float4 chunk j of the cached row; hd4 is even. A plain
// loop: the compiler's unrolling overlaps later loads with the add chain.
template <class KChunk>
__device__ __forceinline__ float qk_dot(const float4* qt, KChunk kchunk, int hd4) {
  float s = 0.0f;
#pragma unroll 2
  for (int i0 = 0; i0 < hd4; i0 += 2) {
    const float4 k0 = kchunk(i0), q0 = qt[i0], k1 = kchunk(i0 + 1), q1 = qt[i0 + 1];
    const float p0 = fmul(q0.x, k0.x), p1 = fmul(q0.y, k0.y), p2 = fmul(q0.z, k0.z), p3 = fmul(q0.w, k0.w);
    const float p4 = fmul(q1.x, k1.x), p5 = fmul(q1.y, k1.y), p6 = fmul(q1.z, k1.z), p7 = fmul(q1.w, k1.w);
    s = fadd(s, p0); s = fadd(s, p1); s = fadd(s, p2); s = fadd(s, p3);
    s = fadd(s, p4); s = fadd(s, p5); s = fadd(s, p6); s = fadd(s, p7);
  }
  return s;
}

// The cached K and V rows of positions [0, pos) of head h's KV head, requested into the
// staging area long before the attention phase needs them (they do not depend on the token
// being decoded): K rows first, then V rows, hd floats each; the 16-byte chunks of K row t
// are stored at chunk index j ^ (t & 7) so that threads reading different rows hit
// different banks. Returns false, and stages nothing, when the rows do not fit.
__device__ __forceinline__ bool attn_stage_early(const StepParams& P, int li, int h, int pos, float* stg, int tid, int nthreads) {
  const int hd = P.head_dim, n = pos + 1;
  if ((size_t)2 * n * hd > (size_t)P.stage_floats) return false;
  const int kvd = P.n_kv_head * hd, kvh = h / (P.n_head / P.n_kv_head), hd4 = hd >> 2;
  const int mask = (hd & 31) == 0 ? 7 : 0;
  const float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd + kvh * hd;
  const float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd + kvh * hd;
  float* kbuf = stg;
  float* vbuf = stg + (size_t)n * hd;
#pragma unroll 1
  for (int j = tid; j < pos * hd4; j += nthreads) {
    const int t = j / hd4, i4 = j - t * hd4;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(kbuf + t * hd + 4 * (i4 ^ (t & mask)))),
                 "l"(kc + (size_t)t * kvd + 4 * i4)
                 : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(vbuf + t * hd + 4 * i4)), "l"(vc + (size_t)t * kvd + 4 * i4)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  return true;
}

// Scores and value mix of head h when the cached rows pass through two chunk buffers
// (contexts whose rows do not fit the staging area): cached K rows are staged in chunks,
// double buffered, rows padded by one float4 to spread the banks; then the softmax; then
// the V rows the same way. q, k, v of the token being decoded are in sq, sk, sv.
__device__ __forceinline__ void attention_chunked(const StepParams& P, int li, int h, int pos, uint32_t tag_out, const MegaSmem& M,
                                               int tid, int T) {
  const CtaGroup g{tid, T, 1};
  const int hd = P.head_dim, kvd = P.n_kv_head * hd, kvh = h / (P.n_head / P.n_kv_head), n = pos + 1, hd4 = hd >> 2;
  float* sq = M.scr;
  float* sk = sq + hd;
  float* sv = sk + hd;
  float* sc = sv + 3 * hd;
  float* vbuf = M.scr + P.small_floats;
  const float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd;
  const float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd;
  const float scale = 1.0f / sqrtf((float)hd);
  const float4* qt = reinterpret_cast<const float4*>(sq);
  const int kstride = hd + 4, chunk = P.v_chunk, buf_floats = chunk * kstride;
  float lmax = -INFINITY;
  stage_kv_rows(vbuf, kstride, kc, kvd, kvh * hd, hd4, 0, min(chunk, n), pos, sk, tid, T);
#pragma unroll 1
  for (int c0 = 0, ci = 0; c0 < n; c0 += chunk, ci++) {
    const int cn = min(chunk, n - c0);
    float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + chunk < n) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, kstride, kc, kvd, kvh * hd, hd4, c0 + chunk, min(chunk, n - c0 - chunk), pos, sk, tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    for (int t = tid; t < cn; t += T) {
      const float4* kt = reinterpret_cast<const float4*>(cur_buf + t * kstride);
      float s = qk_dot(qt, [&](int j) { return kt[j]; }, hd4);
      s = fmul(s, scale);
      sc[c0 + t] = s;
      lmax = fmaxf(lmax, s);
    }
    g.sync();  // this buffer is refilled two chunks later
  }
  // the first chunk of V rows loads while the softmax runs
  stage_kv_rows(vbuf, hd, vc, kvd, kvh * hd, hd4, 0, min(chunk, n), pos, sv, tid, T);
  softmax_rows(sc, n, lmax, P.fast, M, g);
  float o = 0.0f;
  const int md = mix_dim(tid, T, hd);
#pragma unroll 1
  for (int c0 = 0, ci = 0; c0 < n; c0 += chunk, ci++) {
    const int cn = min(chunk, n - c0);
    const float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + chunk < n) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, hd, vc, kvd, kvh * hd, hd4, c0 + chunk, min(chunk, n - c0 - chunk), pos, sv, tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    if (md >= 0) o = value_mix(o, sc + c0, cur_buf + md, hd, cn);
    g.sync();
  }
  if (md >= 0) ll_store(P.attl + h * hd + md, o, tag_out);
}

// How `S` CTAs share one head when its cached rows do not fit one CTA's staging area.
// Scores: positions are cut into S contiguous ranges, one per CTA; every score is published
// as a tagged word. Value mix: the head's dimensions are cut into slices of `dw` (a multiple
// of 16, so staged slices stay 16-byte aligned and at least half a cache line); the first
// `n2` CTAs wait for all of the head's scores, run the softmax (each the same arithmetic on
// the same values, so the same bits) and mix their slice, positions in order.
struct AttnSplit {
  int S, dw, n2;
};
__device__ __forceinline__ AttnSplit attn_split_plan(int grid, int n_head, int hd) {
  AttnSplit a;
  a.S = n_head > 0 ? grid / n_head : 0;
  const int h16 = hd >> 4;
  a.dw = a.S > 0 ? 16 * ((h16 + a.S - 1) / a.S) : hd;
  a.n2 = (hd + a.dw - 1) / a.dw;
  return a;
}

// Requests the cached rows split-CTA `s` of head `h` will read into L2, long before use.
__device__ __noinline__ void attn_split_prefetch(const float* k_cache, const float* v_cache, int n_ctx, int hd, int n_head, int n_kv_head,
                                                 int li, int pos, int tid, int T) {
  const AttnSplit a = attn_split_plan(gridDim.x, n_head, hd);
  if ((int)blockIdx.x >= a.S * n_head) return;
  const int h = blockIdx.x % n_head, s = blockIdx.x / n_head;
  const int kvd = n_kv_head * hd, kvh = h / (n_head / n_kv_head), n = pos + 1;
  const int per = (n + a.S - 1) / a.S, t0 = min(pos, s * per), t1 = min(pos, t0 + per);
  const float* kc = k_cache + (size_t)li * n_ctx * kvd + kvh * hd;
  const float* vc = v_cache + (size_t)li * n_ctx * kvd + kvh * hd + s * a.dw;
  const int lines = (hd * 4 + 127) / 128;
  for (int j = tid; j < (t1 - t0) * lines; j += T) {
    const int t = t0 + j / lines, ln = j % lines;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + (size_t)t * kvd + 32 * ln));
  }
  if (s < a.n2) {
    const int vlines = (a.dw * 4 + 127) / 128;
    for (int j = tid; j < pos * vlines; j += T) {
      const int t = j / vlines, ln = j % vlines;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + (size_t)t * kvd + 32 * ln));
    }
  }
}

// Scores and value mix of split-CTA `s` of head h. q, k, v of the token being decoded are in
// sq, sk, sv (every CTA of the head prepared the same values). Only the long-context
// variant of the kernel contains this code; its inputs are gathered by value.
struct AttnSplitArgs {
  int li, h, s, pos, tid, T;
  int head_dim, n_head, n_kv_head, n_ctx, small_floats, v_chunk, fast;
  uint32_t tag_out;
  float *k_cache, *v_cache;
  LLWord *scl, *attl;
  float *scr, *red;
  SeqSumScratch* ss;
  volatile int* abort;
  int* err;
  unsigned long long* prof;
};
__device__ __forceinline__ void attention_split(const AttnSplitArgs A) {
  const int tid = A.tid, T = A.T, pos = A.pos, s = A.s;
  const CtaGroup g{tid, T, 1};
  const MegaSmem M{nullptr, A.scr, A.ss, A.red, A.abort, A.err};
  const AttnSplit a = attn_split_plan(gridDim.x, A.n_head, A.head_dim);
  const uint32_t tag_sc = A.tag_out | 1024u;
  SubProf pf{A.prof, clock64()};
  const int hd = A.head_dim, kvd = A.n_kv_head * hd, kvh = A.h / (A.n_head / A.n_kv_head), n = pos + 1, hd4 = hd >> 2;
  float* sq = A.scr;
  float* sk = sq + hd;
  float* sv = sk + hd;
  float* sc = sv + 3 * hd;
  float* vbuf = A.scr + A.small_floats;
  const float* kc = A.k_cache + (size_t)A.li * A.n_ctx * kvd;
  const float* vc = A.v_cache + (size_t)A.li * A.n_ctx * kvd;
  const float scale = 1.0f / sqrtf((float)hd);
  const float4* qt = reinterpret_cast<const float4*>(sq);
  const int kstride = hd + 4, chunk = A.v_chunk, buf_floats = chunk * kstride;
  LLWord* scl = A.scl + (size_t)A.h * A.n_ctx;
  const int per = (n + a.S - 1) / a.S, t0 = min(n, s * per), t1 = min(n, t0 + per);
  if (t0 < t1) stage_kv_rows(vbuf, kstride, kc, kvd, kvh * hd, hd4, t0, min(chunk, t1 - t0), pos, sk, tid, T);
#pragma unroll 1
  for (int c0 = t0, ci = 0; c0 < t1; c0 += chunk, ci++) {
    const int cn = min(chunk, t1 - c0);
    float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + chunk < t1) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, kstride, kc, kvd, kvh * hd, hd4, c0 + chunk, min(chunk, t1 - c0 - chunk), pos, sk, tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    for (int t = tid; t < cn; t += T) {
      const float4* kt = reinterpret_cast<const float4*>(cur_buf + t * kstride);
      const float dot = qk_dot(qt, [&](int j) { return kt[j]; }, hd4);
      ll_store(scl + c0 + t, fmul(dot, scale), tag_sc);
    }
    g.sync();  // this buffer is refilled two chunks later
  }
  pf.mark(21);
  if (s >= a.n2) return;
  const int d0 = s * a.dw, dn = min(a.dw, hd - d0), dn4 = dn >> 2;
  const int vchunk = (buf_floats / dn) & ~7;  // positions per buffer when rows are dn floats (a multiple of 8: aligned reads)
  stage_kv_rows(vbuf, dn, vc, kvd, kvh * hd + d0, dn4, 0, min(vchunk, n), pos, sv + d0, tid, T);
  float lmax = -INFINITY;
  for (int t = tid; t < n; t += T) {
    const float v = ll_wait(scl + t, tag_sc, A.abort, A.err);
    sc[t] = v;
    lmax = fmaxf(lmax, v);
  }
  pf.mark(22);
  softmax_rows(sc, n, lmax, A.fast, M, g);
  pf.mark(23);
  float o = 0.0f;
  const int md = mix_dim(tid, T, dn);
#pragma unroll 1
  for (int c0 = 0, ci = 0; c0 < n; c0 += vchunk, ci++) {
    const int cn = min(vchunk, n - c0);
    const float* cur_buf = vbuf + (ci & 1) * buf_floats;
    if (c0 + vchunk < n) {
      stage_kv_rows(vbuf + ((ci + 1) & 1) * buf_floats, dn, vc, kvd, kvh * hd + d0, dn4, c0 + vchunk, min(vchunk, n - c0 - vchunk), pos, sv + d0, tid, T);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    g.sync();
    pf.mark(25);
    if (md >= 0) o = value_mix(o, sc + c0, cur_buf + md, dn, cn);
    pf.mark(27);
    g.sync();
  }
  if (md >= 0) ll_store(A.attl + A.h * hd + d0 + md, o, A.tag_out);
  pf.mark(24);
}

// Per-head q/k norm, RoPE, KV store and attention for head `h` (ops.rs:74-87, 40-70,
// 152-157, 185-218), by the consumer warps of one CTA. `staged`: attn_stage_early has put
// the cached rows of this head into the staging area.
template <bool SPLIT>
__device__ __forceinline__ void phase_attention(const StepParams& P, int li, int h, int pos, uint32_t tag_in, uint32_t tag_out, bool staged,
                                             const MegaSmem& M, int tid, int T, unsigned long long* prof, int split_s) {
  const CtaGroup g{tid, T, 1};
  SubProf pf{prof, clock64()};
  const int hd = P.head_dim, kvd = P.n_kv_head * hd, gqa = P.n_head / P.n_kv_head, kvh = h / gqa;
  const int n = pos + 1;
  float* sq = M.scr;            // hd
  float* sk = sq + hd;          // hd
  float* sv = sk + hd;          // hd
  float* sp = sv + hd;          // 2 x hd (squares of q and of k)
  float* sc = sp + 2 * hd;      // n_ctx scores
  float* stg = M.scr + P.small_floats;  // staging area, 16-byte aligned
  float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd;
  float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd;
  // RoPE factors of this thread's pair, requested before the wait below
  const int rope_half = P.rot_dim / 2;
  float rope_c = 0.0f, rope_s = 0.0f;
  if (tid < 2 * rope_half) {
    const float* cs = P.rope_table + (size_t)pos * P.rot_dim;
    const int i = tid < rope_half ? tid : tid - rope_half;
    rope_c = cs[2 * i];
    rope_s = cs[2 * i + 1];
  }
  // this head's q and its group's k, v rows as the q/k/v products publish them
  for (int j = tid; j < 3 * hd; j += T) {
    const int which = j / hd, i = j - which * hd;
    const LLWord* src = which == 0 ? P.ql + h * hd + i : (which == 1 ? P.kl : P.vl) + kvh * hd + i;
    sq[j] = ll_wait(src, tag_in, M.abort, M.err);  // sq, sk, sv are consecutive
  }
  g.sync();
  if (P.qk_norm) {
    // per-head RMS norm of q and of k (ops.rs:74-87): the two sums of squares are
    // sequential add chains; one thread each, side by side
    for (int i = tid; i < 2 * hd; i += T) sp[i] = fmul(sq[i], sq[i]);  // sq, sk consecutive; sp holds 2 x hd
    float ss[2];
    if (!(P.fast & FAST_NORM_SUM) && hd <= SEQ_CHAIN_MAX) {
      g.sync();
      if ((tid & 31) == 0 && tid < 64) {
        const float* p = sp + (tid >> 5) * hd;
        float a = 0.0f;
        for (int i = 0; i < hd; i += 8) {
          const float4 u = *reinterpret_cast<const float4*>(p + i), w = *reinterpret_cast<const float4*>(p + i + 4);
          a = fadd(a, u.x); a = fadd(a, u.y); a = fadd(a, u.z); a = fadd(a, u.w);
          a = fadd(a, w.x); a = fadd(a, w.y); a = fadd(a, w.z); a = fadd(a, w.w);
        }
        M.red[40 + (tid >> 5)] = a;
      }
      g.sync();
      ss[0] = M.red[40];
      ss[1] = M.red[41];
    } else {
      ss[0] = cta_sum(sp, hd, (P.fast & FAST_NORM_SUM) != 0, M, g);
      g.sync();
      ss[1] = cta_sum(sp + hd, hd, (P.fast & FAST_NORM_SUM) != 0, M, g);
    }
    g.sync();
    for (int i = tid; i < 2 * hd; i += T) {
      const int which = i >= hd;
      const float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss[which], (float)hd), P.eps)));
      const float* nw = which ? P.layers[li].k_norm : P.layers[li].q_norm;
      sq[i] = fmul(fmul(sq[i], r), nw[i - which * hd]);
    }
    g.sync();
  }
  if (tid < 2 * rope_half) {  // rot_dim <= head_dim <= the group's thread count
    float* v = tid < rope_half ? sq : sk;
    const int i = tid < rope_half ? tid : tid - rope_half;
    const int i0 = P.neox ? i : 2 * i, i1 = P.neox ? i + rope_half : 2 * i + 1;
    const float x0 = v[i0], x1 = v[i1];
    v[i0] = fsub(fmul(x0, rope_c), fmul(x1, rope_s));
    v[i1] = fadd(fmul(x0, rope_s), fmul(x1, rope_c));
  }
  g.sync();
  if (h % gqa == 0 && split_s == 0) {
    for (int i = tid; i < hd; i += T) {
      kc[(size_t)pos * kvd + kvh * hd + i] = sk[i];
      vc[(size_t)pos * kvd + kvh * hd + i] = sv[i];
    }
  }
  pf.mark(20);
  if (SPLIT) {
    attention_split(AttnSplitArgs{li, h, split_s, pos, tid, T, P.head_dim, P.n_head, P.n_kv_head, P.n_ctx, P.small_floats, P.v_chunk,
                                  P.fast, tag_out, P.k_cache, P.v_cache, P.scl, P.attl, M.scr, M.red, M.ss, M.abort, M.err, prof});
    return;
  }
  if (!staged) {
    attention_chunked(P, li, h, pos, tag_out, M, tid, T);
    pf.mark(24);
    return;
  }
  // the row of the token being decoded joins the staged rows
  const int hd4 = hd >> 2, mask = (hd & 31) == 0 ? 7 : 0;
  float* kbuf = stg;
  float* vbuf = stg + (size_t)n * hd;
  for (int i4 = tid; i4 < 2 * hd4; i4 += T) {
    if (i4 < hd4) reinterpret_cast<float4*>(kbuf + pos * hd)[i4 ^ (pos & mask)] = reinterpret_cast<const float4*>(sk)[i4];
    else reinterpret_cast<float4*>(vbuf + pos * hd)[i4 - hd4] = reinterpret_cast<const float4*>(sv)[i4 - hd4];
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  g.sync();
  const float scale = 1.0f / sqrtf((float)hd);
  const float4* qt = reinterpret_cast<const float4*>(sq);
  float lmax = -INFINITY;
  for (int t = tid; t < n; t += T) {
    const float4* kt = reinterpret_cast<const float4*>(kbuf + t * hd);
    const int sw = t & mask;
    float s = qk_dot(qt, [&](int j) { return kt[j ^ sw]; }, hd4);
    s = fmul(s, scale);
    sc[t] = s;
    lmax = fmaxf(lmax, s);
  }
  pf.mark(21);
  softmax_rows(sc, n, lmax, P.fast, M, g);
  pf.mark(23);
  g.sync();
  // value mix, positions in order (ops.rs:208-214)
  {
    const int md = mix_dim(tid, T, hd);
    if (md >= 0) ll_store(P.attl + h * hd + md, value_mix(0.0f, sc, vbuf + md, hd, n), tag_out);
  }
  pf.mark(24);
}

// Greedy argmax of the logits (sampler.rs:99-109) and the cursor update, CTA 0 only. With a
// vocabulary-sharded head (TP) every rank finds the best of its slice, stores {logit, id}
// into every rank's inbox and picks the best of the world: highest logit, lowest id on ties,
// which is the first maximum of the whole vector.
template <bool TP>
__device__ void phase_argmax(const StepParams& P, const MegaSmem& M, const CtaGroup& g) {
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = g.tid; i < P.vocab; i += g.nthreads) {
    float v = __ldcg(P.logits + i);
    if (v > best) {
      best = v;
      idx = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float v2 = __shfl_xor_sync(0xffffffffu, best, o);
    int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
    if (v2 > best || (v2 == best && i2 < idx)) {
      best = v2;
      idx = i2;
    }
  }
  int* redi = reinterpret_cast<int*>(M.red + 32);
  if ((g.tid & 31) == 0) {
    M.red[g.tid >> 5] = best;
    redi[g.tid >> 5] = idx;
  }
  g.sync();
  if (g.tid < 32) {
    // warp 0: every lane folds the warps' candidates (the same result in each)
    for (int w = 1; w < (g.nthreads >> 5); w++) {
      if (M.red[w] > best || (M.red[w] == best && redi[w] < idx)) {
        best = M.red[w];
        idx = redi[w];
      }
    }
    if (idx == 0x7fffffff) idx = 0;
    if (TP && P.tp.head_sharded) {
      // lane r hands this rank's best {logit, id} to rank r; lane l waits for word l of the
      // ranks' slots here (one round trip for all of them), and the shuffles walk them in rank order
      const uint32_t tag = (*P.epoch << 11) + 5u * (uint32_t)P.n_layer + 8u;
      idx += P.tp.head_row0;
      if (g.tid < P.tp.world) {
        LLWord* slot = P.tp.inbox[g.tid] + P.tp.arg_off + 2 * P.tp.rank;
        ll_store_sys(slot, best, tag);
        ll_store_sys(slot + 1, __int_as_float(idx), tag);
      }
      float word = 0.0f;
      if (g.tid < 2 * P.tp.world) word = ll_wait_sys(P.tp.inbox[P.tp.rank] + P.tp.arg_off + g.tid, tag, M.abort, M.err);
      best = -INFINITY;
      idx = 0x7fffffff;
#pragma unroll
      for (int r = 0; r < TP_MAX_WORLD; r++) {
        const float v = __shfl_sync(0xffffffffu, word, 2 * r);
        const int i = __float_as_int(__shfl_sync(0xffffffffu, word, 2 * r + 1));
        if (r < P.tp.world && (v > best || (v == best && i < idx))) {
          best = v;
          idx = i;
        }
      }
      if (idx == 0x7fffffff) idx = 0;
    }
    if (g.tid == 0) {
      if (P.out_token) *P.out_token = idx;
      int gcount = P.step[2];
      if (P.history && gcount < P.history_cap) P.history[gcount] = idx;
      P.step[0] = idx;
      P.step[1] = P.step[1] + 1;
      P.step[2] = gcount + 1;
    }
  }
}

// ---- the kernel ---------------------------------------------------------------------------------

constexpr int MEGA_THREADS = MEGA_THREADS_N;
constexpr int MEGA_CONSUMER_WARPS = MEGA_THREADS / 32 - 1;
constexpr int MEGA_BAR_BYTES = 128 + 8 * 608;  // up to 8 stages x (full, empty), then their tile descriptors
// Bytes of shared memory besides the ring stages, the activation images and the scratch.
// Block-term strips of the consumer warps. Between products the same bytes hold the
// records of the exact sequential sums (norm and softmax phases never overlap a product).
constexpr int MEGA_TERMS_BYTES = MEGA_CONSUMER_WARPS * WARP_TERMS_FLOATS * 4;
static_assert(sizeof(SeqSumScratch) <= MEGA_TERMS_BYTES, "SeqSumScratch must fit the term strips");
constexpr int MEGA_TAIL_BYTES = MEGA_BAR_BYTES + 64 * 4 + 16 + MEGA_TERMS_BYTES;

// TP: this GPU holds one shard of a row-sharded model and exchanges partial rows with its peers.
// SPLIT: the long-context variant, in which several CTAs share each head's attention (the
// host picks the variant from the position; see attention_split).
template <bool TP, bool SPLIT>
__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_step_kernel(const StepParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][sx images][scratch][barriers 128 B][red 64 floats][abort][term strips | SeqSumScratch][table]
  const int nb_max = (max(max(P.dim, P.hidden), P.n_head * P.head_dim)) / 256;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  uint8_t* cur = sx + (size_t)nb_max * XK_STRIDE;  // 16-byte aligned: 304 = 19 * 16
  float* scr = reinterpret_cast<float*>(cur);
  cur += P.scratch_bytes;                          // a multiple of 128
  uint64_t* bars = reinterpret_cast<uint64_t*>(cur);
  cur += MEGA_BAR_BYTES;
  float* red = reinterpret_cast<float*>(cur);
  cur += 64 * sizeof(float);
  volatile int* abort = reinterpret_cast<volatile int*>(cur);
  cur += 16;
  float* const wterms_all = reinterpret_cast<float*>(cur);
  SeqSumScratch* ssc = reinterpret_cast<SeqSumScratch*>(cur);
  cur += MEGA_TERMS_BYTES;
  // The step's tensor table (one StepLayer per layer + the output head), copied from
  // global memory once so that no phase waits on a descriptor load.
  StepLayer* const table = reinterpret_cast<StepLayer*>(cur);
  {
    const uint4* src = reinterpret_cast<const uint4*>(P.layers);
    uint4* dst = reinterpret_cast<uint4*>(table);
    for (int i = threadIdx.x; i < P.table_bytes / 16; i += blockDim.x) dst[i] = src[i];
  }

  Ring R;
  R.stages = stages;
  R.full = bars;
  R.empty = bars + P.n_stages;
  R.desc = reinterpret_cast<TileDesc*>(bars + 16);
  R.n_stages = P.n_stages;
  R.stage_bytes = P.stage_bytes;
  R.abort = abort;
  R.err = P.err;
  if (threadIdx.x == 0) {
    for (int s = 0; s < P.n_stages; s++) {
      mbar_init(&R.full[s], 1);
      mbar_init(&R.empty[s], MEGA_CONSUMER_WARPS);
    }
    // A launch that finds the device error word set (an earlier step's wait gave up: a
    // peer is gone, say) does no work: steps already queued behind a failed one drain in
    // microseconds instead of each waiting out its own limits.
    abort[0] = *reinterpret_cast<volatile int*>(P.err) != 0 ? 1 : 0;
    abort[1] = P.spin_limit;
    mbar_fence_init();
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5;
  const int qd = P.n_head * P.head_dim;
  if (*abort) {
    // keep the launch count in step with the other ranks, whose tags follow it
    if (blockIdx.x == 0 && threadIdx.x == 0) *P.epoch = *P.epoch + 1u;
    return;
  }

  if (warp == MEGA_CONSUMER_WARPS) {
    // ---- producer warp: walks every matrix product of the step ----
    RingPos pp{0, 0u};
    uint32_t tiles_issued = 0;
    for (int li = 0; li < P.n_layer && !*abort; li++) {
      const StepLayer& L = table[li];
#pragma unroll 1
      for (int ph = 0; ph < 4; ph++) produce_op((&L.qkv)[ph], R, pp, MEGA_CONSUMER_WARPS, tiles_issued);  // qkv, wo, gu, down are consecutive members
    }
    if (P.want_logits && !*abort) produce_op(table[P.n_layer].qkv, R, pp, MEGA_CONSUMER_WARPS, tiles_issued);
    if ((threadIdx.x & 31) == 0) produce_drain(R, pp, tiles_issued);
    return;
  }

  // ---- consumer warps ----
  CtaGroup g{(int)threadIdx.x, MEGA_CONSUMER_WARPS * 32, 1};
  MegaSmem M{sx, scr, ssc, red, abort, P.err};
  float* const wterms = wterms_all + warp * WARP_TERMS_FLOATS;
  RingPos cp{0, 0u};
  unsigned bar_target = 0;
  bool staged = false;
  const int token = P.step[0], pos = P.step[1];
  // Long contexts: the cached rows of a head no longer fit one CTA's staging area, and the
  // CTAs beyond the head count would idle through the attention phase; share each head.
  // (The plan is a few integer operations: it is recomputed where it is used rather than
  // kept in registers across the whole step.)
  // Tags of this launch: phase k (1..5) of layer li is tag_base + 5 * li + k.
  const uint32_t tag_base = *P.epoch << 11;
  const bool prof_on = P.prof && (int)blockIdx.x == P.prof_cta && g.tid == 0;
  long long prof_last = clock64();
  int prof_li = -1;  // layer the phase marks belong to
#define MEGA_PROF(slot)                                 \
  do {                                                  \
    if (P.timeline && g.tid == 0 && prof_li == P.timeline_layer) {      \
      unsigned long long t_;                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
      P.timeline[blockIdx.x * 16 + (slot)] = t_;        \
    }                                                   \
    if (prof_on) {                                      \
      long long now_ = clock64();                       \
      atomicAdd(&P.prof[slot], (unsigned long long)(now_ - prof_last)); \
      prof_last = now_;                                 \
    }                                                   \
  } while (0)

  // embedding row (quant.rs:300-443 via emit.rs:469): every CTA keeps a copy and publishes
  // the residual rows it owns (the rows of wo / down it computes)
  {
    const uint8_t* row = P.token_embd + (size_t)token * P.embd_row_bytes;
    int r0, r1;
    cta_rows(P.dim, r0, r1);
    for (int e = g.tid; e < P.dim; e += g.nthreads) {
      float v = dequant_elem_call(P.embd_kind, row, (size_t)e);
      scr[e] = v;
      if (e >= r0 && e < r1) ll_store(P.xl + e, v, 0u);
    }
    g.sync();
  }
  MEGA_PROF(0);

  // One loop over the step's matrix products (four per layer, then the output head), so
  // that each phase's code exists once. Phases hand their vectors on as tagged words;
  // the only grid-wide barrier left is the one in front of the argmax.
  const int n_stage = 4 * P.n_layer + (P.want_logits ? 1 : 0);
#pragma unroll 1
  for (int st = 0; st < n_stage; st++) {
    const int li = st >> 2, ph = st & 3;
    const bool head = li == P.n_layer;
    prof_li = li;
    const StepLayer& L = table[li];
    const MegaOp& op = (&L.qkv)[ph];  // qkv, wo, gu, down are consecutive members
    const int slot = ph == 0 ? 1 : 3 * ph + 3;
    const uint32_t tl = tag_base + 5u * (uint32_t)li;  // + k: phase k of this layer
    if (SPLIT) {
      if (ph == 0 && !head) attn_split_prefetch(P.k_cache, P.v_cache, P.n_ctx, P.head_dim, P.n_head, P.n_kv_head, li, pos, g.tid, g.nthreads);
    } else if (ph == 0 && !head && (int)blockIdx.x < P.n_head) {
      // The cached K and V rows this CTA's head will read do not depend on the token being
      // decoded: request them into shared memory now, two phases ahead of their use. When
      // they do not fit, at least ask for them into L2 (the weight stream evicts the cache
      // between tokens).
      staged = attn_stage_early(P, li, blockIdx.x, pos, scr + P.small_floats, g.tid, g.nthreads);
      for (int h = blockIdx.x + (staged ? gridDim.x : 0); h < P.n_head; h += gridDim.x) {
        const int kvd = P.n_kv_head * P.head_dim, kvh = h / (P.n_head / P.n_kv_head);
        const int lines = (P.head_dim * 4 + 127) / 128;  // 128-byte lines per cached row of one head
        const float* kc = P.k_cache + (size_t)li * P.n_ctx * kvd + kvh * P.head_dim;
        const float* vc = P.v_cache + (size_t)li * P.n_ctx * kvd + kvh * P.head_dim;
        for (int j = g.tid; j < pos * lines; j += g.nthreads) {
          const int t = j / lines, ln = j - t * lines;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + (size_t)t * kvd + 32 * ln));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + (size_t)t * kvd + 32 * ln));
        }
      }
    }
    if ((ph & 1) == 0) {
      // attention norm -> q/k/v, ffn norm -> gate/up + SiLU, output norm -> logits
      const float* w = head ? P.output_norm : (ph == 0 ? L.attn_norm : L.ffn_norm);
      const uint32_t tin = ph == 0 ? tl : tl + 3u;  // residual after the previous layer's down / this layer's wo
      phase_norm_quant(P.xl, tin, st == 0, head && blockIdx.x == 0 ? P.x : nullptr, w, P.dim, P.eps, P.fast, M, g,
                       SubProf{prof_on && ph == 0 && !head ? P.prof : nullptr, 0},
                       P.prof && (int)blockIdx.x == P.prof_cta && ph == 0 && !head && g.tid == (MEGA_CONSUMER_WARPS - 1) * 32 ? P.prof : nullptr);
    } else {
      // attention output -> wo, activated hidden -> down; both join the residual stream
      if (ph == 1) phase_quant(P.attl, tl + 2u, qd, M, g);
      else phase_quant(P.hbl, tl + 4u, P.hidden, M, g);
    }
    if (!head) MEGA_PROF(slot);
    // q/k/v: tl+1, wo: tl+3, gate/up: tl+4, down: tl+5 (the head writes plain floats)
    const uint32_t tag_out = tl + (ph == 0 ? 1u : (uint32_t)ph + 2u);
    const bool exchange = TP && (ph & 1) && !head;
    int xr0 = 0, xr1 = 0;  // rows of the residual stream this CTA owns (the rows of wo / down it computes)
    if (TP && exchange) cta_rows(P.dim, xr0, xr1);
    consume_op<TP>(op, R, cp, sx, wterms, warp, MEGA_CONSUMER_WARPS, tag_out, exchange ? &P.tp : nullptr, ph >> 1,
                   SubProf{nullptr, 0}, M.red, xr0);
    if (head) break;
    // The next phase rewrites the activation images and the scratch rows; warps that are
    // done must also not start polling while others still compute.
    g.sync();
    if (TP && exchange) {
      // Hand this CTA's partial rows to every rank (this one included): warp d sends to rank
      // d, its lanes consecutive rows, so a rank receives each CTA's rows as whole sectors.
      const int r0 = xr0, r1 = xr1;
      for (int dst = warp; dst < P.tp.world; dst += MEGA_CONSUMER_WARPS) {
        LLWord* const to = P.tp.inbox[dst] + ((size_t)(ph >> 1) * P.tp.world + P.tp.rank) * P.dim + r0;
        for (int i = g.tid & 31; i < r1 - r0; i += 32) ll_store_sys(to + i, M.red[i], tag_out);
      }
      g.sync();  // the next phase reuses the parking strip
      // The rows this CTA owns: wait for every rank's partial, add them in rank order, join
      // the residual stream and publish the row for this GPU's CTAs. Eight lanes per row,
      // lane s waiting for rank s's word (one after the other, eight ranks would cost one
      // thread eight round trips to memory that peers write); lane 0 adds them through shuffles.
      {
        const int sub = g.tid & (TP_MAX_WORLD - 1), slot_row = g.tid / TP_MAX_WORLD;
        const LLWord* const in = P.tp.inbox[P.tp.rank] + (size_t)(ph >> 1) * P.tp.world * P.dim + (size_t)sub * P.dim;
        for (int i0 = r0; i0 < r1; i0 += g.nthreads / TP_MAX_WORLD) {  // the same trip count in every lane of a warp
          const int i = i0 + slot_row;
          float v = 0.0f;
          if (i < r1 && sub < P.tp.world) v = ll_wait_sys(in + i, tag_out, abort, P.err);
          const int base = (g.tid & 31) & ~(TP_MAX_WORLD - 1);
          float sum = __shfl_sync(0xffffffffu, v, base);
#pragma unroll
          for (int src = 1; src < TP_MAX_WORLD; src++) {
            const float t = __shfl_sync(0xffffffffu, v, base + src);
            if (src < P.tp.world) sum = fadd(sum, t);
          }
          if (i < r1 && sub == 0) ll_store(P.xl + i, fadd(ll_value(P.xl + i), sum), tag_out);
        }
      }
    }
    MEGA_PROF(slot + 1);
    if (ph == 0) {
      // attention: one head per CTA, or several CTAs per head once the context is long
      if (SPLIT) {
        if ((int)blockIdx.x < ((int)gridDim.x / P.n_head) * P.n_head) {
          phase_attention<true>(P, li, blockIdx.x % P.n_head, pos, tl + 1u, tl + 2u, false, M, g.tid, g.nthreads, prof_on ? P.prof : nullptr,
                                blockIdx.x / P.n_head);
          g.sync();
        }
      } else {
        for (int h = blockIdx.x; h < P.n_head; h += gridDim.x) {
          phase_attention<false>(P, li, h, pos, tl + 1u, tl + 2u, staged && h == (int)blockIdx.x, M, g.tid, g.nthreads,
                                 prof_on ? P.prof : nullptr, 0);
          g.sync();
        }
      }
      MEGA_PROF(4);
    }
  }
  if (!P.want_logits && blockIdx.x == 0) {
    // no output head: still leave a plain copy of the final residual stream
    const uint32_t tin = tag_base + 5u * (uint32_t)P.n_layer;
    for (int i = g.tid; i < P.dim; i += g.nthreads) P.x[i] = ll_wait(P.xl + i, tin, abort, P.err);
  }
  if (P.want_logits && P.with_argmax) {
    const bool ok = grid_sync(P, g, bar_target, abort);  // uniform across the CTA
    if (blockIdx.x == 0 && ok) phase_argmax<TP>(P, M, g);
  }
  // Next launch, next tags. Every CTA read the count before it published anything, and
  // CTA 0 gets here only after consuming words from every CTA.
  if (blockIdx.x == 0 && g.tid == 0) *P.epoch = *P.epoch + 1u;
  MEGA_PROF(15);
#undef MEGA_PROF
}

// ---- Q4_0 / Q5_0 / Q8_0 rows from the ring --------------------------------------------------
// The reference's AVX2 kernels keep eight f32 lane accumulators per row; lane k adds
// fma(d_w*d_x, float(p_k), acc_k) per 32-weight block, in block order, and the row ends
// with a fixed 8-lane tree (simd_avx2.rs:29-34, 61-72). Here eight threads own the eight
// lane chains of a row (four rows per warp pass).
__device__ __forceinline__ uint32_t lds32_a2s(uint32_t a) {  // 32-bit word at a 2-byte aligned shared address
  uint32_t lo, hi;
  asm("ld.shared.u16 %0, [%1];" : "=r"(lo) : "r"(a));
  asm("ld.shared.u16 %0, [%1];" : "=r"(hi) : "r"(a + 2));
  return lo | (hi << 16);
}

template <int KIND>
__device__ __forceinline__ float row_chain_q80(uint32_t row, uint32_t sx, int nb, int k) {
  constexpr int BS = KIND == Q4_0 ? 18 : (KIND == Q5_0 ? 22 : 34);
  float acc = 0.0f;
#pragma unroll 4
  for (int b = 0; b < nb; b++) {
    const uint32_t wb = row + (uint32_t)b * BS, xb = sx + (uint32_t)b * X0_STRIDE;
    uint32_t hd;
    asm("ld.shared.u16 %0, [%1];" : "=r"(hd) : "r"(wb));
    const float d = fmul(half_bits_hw(hd), __uint_as_float(rd_lds32(xb + X0_D)));
    const uint32_t y = rd_lds32(xb + 4 * k);
    int p;
    if (KIND == Q8_0) p = q8_0_lane(lds32_a2s(wb + 2 + 4 * k), y);
    else if (KIND == Q4_0) p = q4_0_lane(lds32_a2s(wb + 2 + 4 * (k & 3)), k, y);
    else p = q5_0_lane(lds32_a2s(wb + 6 + 4 * (k & 3)), lds32_a2s(wb + 2), k, y);
    acc = ffma(d, i2f(p), acc);
  }
  return acc;
}

// Consumer side for matrices of the Q8_0 family; `sx` holds the 48-byte Q8_0 images.
// `m` activation rows (their images back to back in `sx`) are applied to every resident row;
// output element (token, row) goes to out[token * rows + row].
__device__ __forceinline__ void consume_op_q80(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, int warp,
                                               int n_warps, int m) {
  const int tile_rows = op.tile_rows, pair = op.pair, epilogue = op.epilogue, nb = op.cols >> 5;
  int c0, c1;
  op_cta_rows(op, c0, c1);
  const int lane = threadIdx.x & 31, k = lane & 7, gi = lane >> 3;
  const uint32_t sxa = smem_addr(sx);
  int rot = 0;
  const int n_tiles = (c1 - c0 + tile_rows - 1) / tile_rows;
  for (int tile = 0; tile < n_tiles; tile++) {
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    const TileDesc& D = R.desc[cp.st];
    const int R_rows = D.n_units;
    const int n_pass = (R_rows + 3) / 4;  // four rows per warp pass
    int ps = warp - rot;
    if (ps < 0) ps += n_warps;
    for (; ps < n_pass; ps += n_warps) {
      const int u = ps * 4 + gi;
      float v[2] = {0.0f, 0.0f};
      int pi = 0, lr = u;
      if (!pair && u < R_rows) {
        while (pi < 2 && lr >= D.rows[pi]) {
          lr -= D.rows[pi];
          pi++;
        }
      }
      const int n_mat = pair ? 2 : 1;
      for (int tok = 0; tok < m; tok++) {
        const uint32_t sxt = sxa + (uint32_t)tok * (uint32_t)nb * X0_STRIDE;
        for (int mt = 0; mt < n_mat; mt++) {
          const int part = pair ? mt : pi, sg = D.seg[part];
          const int kind = op.seg[sg].kind;
          const uint32_t row = D.base[part] + (uint32_t)(pair ? u : lr) * op.row_bytes[sg];
          float a = 0.0f;
          if (u < R_rows) {
            if (kind == Q4_0) a = row_chain_q80<Q4_0>(row, sxt, nb, k);
            else if (kind == Q5_0) a = row_chain_q80<Q5_0>(row, sxt, nb, k);
            else a = row_chain_q80<Q8_0>(row, sxt, nb, k);
          }
          // ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)) over the row's eight lanes
          a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 4));
          a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 2));
          a = fadd(a, __shfl_xor_sync(0xffffffffu, a, 1));
          v[mt] = a;
        }
        if (u < R_rows && k == 0) {
          if (pair) {
            const size_t r = (size_t)tok * op.seg[0].rows + D.row0[0] + u;
            op.seg[0].out[r] = epilogue == EPI_SILU_MUL ? silu_mul_exact(v[0], v[1]) : v[0];
            op.seg[1].out[r] = v[1];
          } else {
            const int sg = D.seg[pi];
            float* o = op.seg[sg].out + (size_t)tok * op.seg[sg].rows + D.row0[pi] + lr;
            *o = epilogue == EPI_ACCUM ? fadd(__ldcg(o), v[0]) : v[0];
          }
        }
      }
    }
    rot = (rot + n_pass) % n_warps;
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
}

// ---- one matrix product with the same machinery ------------------------------------------
// A single K-quant product (up to three matrices, or a gate/up pair) against one Q8_K
// activation vector: the producer warp streams this CTA's rows through the ring while the
// consumer warps take whole rows, with no CTA-wide barrier per tile. Used for single-row
// products outside the one-kernel step (the operator API, models the step does not cover).
struct StreamGemvParams {
  MegaOp op;
  const void* x;  // activation images (x_image) or reference-layout blocks
  int x_image;
  int q80;        // matrices of the Q8_0 family (Q8_0 activations) instead of K-quants
  int m;          // activation rows (more than one only for the Q8_0 family)
  int wide;       // many rows per CTA: one lane per super-block (rowwide.cuh) instead of four
  int tg;         // MODE 3: activation rows per CTA group (group blockIdx.y takes rows tg * y ..)
  int n_stages, stage_bytes;
  int* err;
};

// Consumer side for launches with many rows per CTA (rowwide.cuh): passes of 32 / L rows are
// dealt to the warps round robin across tiles, so that with several tiles in the ring every
// warp has rows; a warp that has no pass in a tile still takes part in the tile's barriers.
// Plain stores or residual adds only (no tagged words, no pairs): the single-row entry points.
__device__ __forceinline__ void consume_op_wide(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, int warp, int n_warps) {
  const int nb = op.nb, lane = threadIdx.x & 31;
  int L = 1;
  while (L < nb && L < 32) L <<= 1;
  const int rpp = 32 / L, gi = lane / L, bl = lane & (L - 1);
  const uint32_t sxa = smem_addr(sx);
  const int n_tiles = (int)blockIdx.x < op.cta_rem ? op.n_tiles_hi : op.n_tiles_lo;
  int pass_base = 0;  // passes of the tiles before this one
#pragma unroll 1
  for (int tile = 0; tile < n_tiles; tile++) {
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    const TileDesc& D = R.desc[cp.st];
    const int n_units = D.n_units, n_pass = (n_units + rpp - 1) / rpp;
    int p = (warp - pass_base % n_warps + n_warps) % n_warps;  // this warp's first pass inside the tile
#pragma unroll 1
    for (; p < n_pass; p += n_warps) {
      const int i = p * rpp + gi;
      uint32_t row = 0;
      int kind = Q4_K;
      float* out = nullptr;
      if (i < n_units) {
        const TileUnit U = D.unit[i];
        row = U.row[0] & 0xFFFFFFu;
        kind = (int)(U.row[0] >> 24);
        out = U.out;
      }
      const float sum = wide_row_dot(row, kind, sxa, nb, L);
      if (row != 0 && bl == 0) *out = op.epilogue == EPI_ACCUM ? fadd(__ldcg(out), sum) : sum;
    }
    pass_base += n_pass;
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
}

// One lane per super-block against several activation rows (short batches: 2..7 rows, a few
// dozen on small matrices): a warp pass takes 32 / L rows
// as consume_op_wide does, and every lane forms its block's term for each of the CTA's `mt`
// activation rows in turn, the terms of a row added in block order through the same shuffles
// as for one activation row, so a batch gives the bits of its single products by
// construction. `sx` holds the images of the CTA's `mt` rows (tok0 ..) back to back; output
// element (t, row) goes to out + t * (rows of its matrix). The grid is (row ranges) x (groups of activation
// rows): every CTA streams its rows' weights once, the groups of a range share them in L2.
__device__ __forceinline__ void consume_op_wide_multi(const MegaOp& op, const Ring& R, RingPos& cp, const uint8_t* sx, int warp, int n_warps,
                                                      int tok0, int mt) {
  const int nb = op.nb, lane = threadIdx.x & 31;
  int L = 1;
  while (L < nb && L < 32) L <<= 1;
  const int rpp = 32 / L, gi = lane / L, bl = lane & (L - 1);
  const uint32_t sxa = smem_addr(sx), xrow = (uint32_t)nb * XK_STRIDE;
  const int n_tiles = (int)blockIdx.x < op.cta_rem ? op.n_tiles_hi : op.n_tiles_lo;
  int pass_base = 0;  // passes of the tiles before this one
#pragma unroll 1
  for (int tile = 0; tile < n_tiles; tile++) {
    if (!ring_wait(R, &R.full[cp.st], cp.parity)) return;
    const TileDesc& D = R.desc[cp.st];
    const int n_units = D.n_units, n_pass = (n_units + rpp - 1) / rpp;
    int p = (warp - pass_base % n_warps + n_warps) % n_warps;  // this warp's first pass inside the tile
#pragma unroll 1
    for (; p < n_pass; p += n_warps) {
      const int i = p * rpp + gi;
      uint32_t row = 0;
      int kind = Q4_K;
      float* out = nullptr;
      size_t tstride = 0;  // rows of the unit's matrix: distance between the outputs of two activation rows
      if (i < n_units) {
        const TileUnit U = D.unit[i];
        row = U.row[0] & 0xFFFFFFu;
        kind = (int)(U.row[0] >> 24);
        out = U.out;
        for (int sg = 0; sg < op.nseg; sg++)
          if (out >= op.seg[sg].out && out < op.seg[sg].out + op.seg[sg].rows) tstride = (size_t)op.seg[sg].rows;
      }
#pragma unroll 1
      for (int t = 0; t < mt; t++) {
        const float sum = wide_row_dot(row, kind, sxa + (uint32_t)t * xrow, nb, L);
        if (row != 0 && bl == 0) {
          float* o = out + (size_t)(tok0 + t) * tstride;
          *o = op.epilogue == EPI_ACCUM ? fadd(__ldcg(o), sum) : sum;
        }
      }
    }
    pass_base += n_pass;
    __syncwarp();
    if (lane == 0) mbar_arrive(&R.empty[cp.st]);
    cp.advance(R.n_stages);
  }
}

// MODE picks the consumer that is compiled in (0: Q8_0 family, 1: one lane per super-block,
// 2: four lanes per super-block, 3: one lane per super-block against blockIdx.y's group of
// activation rows): a launch starts with a cold instruction cache, so each
// variant carries only the code it runs.
template <int MODE>
__global__ void __launch_bounds__(MEGA_THREADS, 1) gemv_stream_kernel(const StreamGemvParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // [stages][sx images][barriers 128 B][abort][term strips]
  const int nb = P.q80 ? P.op.cols >> 5 : P.op.cols >> 8;
  const int xstride = P.q80 ? X0_STRIDE : XK_STRIDE;
  uint8_t* stages = smem;
  uint8_t* sx = stages + (size_t)P.n_stages * P.stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sx + (size_t)(MODE == 3 ? P.tg : P.m) * nb * xstride);
  volatile int* abort = reinterpret_cast<volatile int*>(bars + MEGA_BAR_BYTES / 8);
  float* const wterms_all = reinterpret_cast<float*>(const_cast<int*>(abort) + 4);
  Ring R;
  R.stages = stages;
  R.full = bars;
  R.empty = bars + P.n_stages;
  R.desc = reinterpret_cast<TileDesc*>(bars + 16);
  R.n_stages = P.n_stages;
  R.stage_bytes = P.stage_bytes;
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
  const int warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  if (warp == MEGA_CONSUMER_WARPS) {
    // weights do not depend on the previous kernel: stream them right away
    RingPos pp{0, 0u};
    uint32_t tiles_issued = 0;
    produce_op(P.op, R, pp, MEGA_CONSUMER_WARPS, tiles_issued);
    if ((threadIdx.x & 31) == 0) produce_drain(R, pp, tiles_issued);
    return;
  }
  pdl_wait();
  CtaGroup g{(int)threadIdx.x, MEGA_CONSUMER_WARPS * 32, 1};
  // activation rows of this CTA: all of the launch's, or group blockIdx.y's
  const int tok0 = MODE == 3 ? (int)blockIdx.y * P.tg : 0, mt = MODE == 3 ? min(P.tg, P.m - tok0) : P.m;
  const int nbm = nb * mt;  // their blocks, back to back
  const uint8_t* const xsrc = reinterpret_cast<const uint8_t*>(P.x) + (size_t)tok0 * nb * (P.x_image ? xstride : (P.q80 ? 36 : 292));
  if (P.x_image) {
    const uint4* src4 = reinterpret_cast<const uint4*>(xsrc);
    for (int i = g.tid; i < nbm * (xstride / 16); i += g.nthreads) reinterpret_cast<uint4*>(sx)[i] = src4[i];
  } else if (P.q80) {
    // BlockQ8_0 {f32 d; i8 qs[32]} (quant.rs:16-20) -> image {qs; d}
    const uint32_t* src = reinterpret_cast<const uint32_t*>(xsrc);
    for (int i = g.tid; i < nbm * 9; i += g.nthreads) {
      const int b = i / 9, w = i - b * 9;
      *reinterpret_cast<uint32_t*>(sx + b * X0_STRIDE + (w == 0 ? X0_D : (w - 1) * 4)) = src[i];
    }
  } else {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(xsrc);
    for (int i = g.tid; i < nbm * 73; i += g.nthreads) {
      const int b = i / 73, w = i - b * 73;
      const int off = w == 0 ? XK_D : (w <= 64 ? (w - 1) * 4 : XK_BSUMS + (w - 65) * 4);
      *reinterpret_cast<uint32_t*>(sx + b * XK_STRIDE + off) = src[i];
    }
  }
  g.sync();
  RingPos cp{0, 0u};
  if (MODE == 0) consume_op_q80(P.op, R, cp, sx, warp, MEGA_CONSUMER_WARPS, P.m);
  else if (MODE == 1) consume_op_wide(P.op, R, cp, sx, warp, MEGA_CONSUMER_WARPS);
  else if (MODE == 3) consume_op_wide_multi(P.op, R, cp, sx, warp, MEGA_CONSUMER_WARPS, tok0, mt);
  else consume_op(P.op, R, cp, sx, wterms_all + warp * WARP_TERMS_FLOATS, warp, MEGA_CONSUMER_WARPS, 0u);
}


}  // namespace aot
