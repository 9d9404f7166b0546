// Exact sequential-order f32 sums evaluated by a group of warps (device side of seqsum.cuh).
#pragma once
#include "blockmath.cuh"
#include "seqsum.cuh"

namespace aot {

// ---- a group of warps inside a CTA that synchronise on a named barrier ---------------
struct CtaGroup {
  int tid;       // thread index inside the group
  int nthreads;  // multiple of 32
  int bar_id;    // hardware barrier id (0 = the whole CTA, like __syncthreads)
  __device__ __forceinline__ void sync() const {
    if (nthreads == 32) {  // a single warp needs no hardware barrier (there are only 16 of them)
      __syncwarp();
      return;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
  }
};

// Optional sub-phase cycle counters (slots 16..31 of the profile array).
struct SubProf {
  unsigned long long* prof;
  long long last;
  __device__ __forceinline__ void mark(int slot) {
    if (prof) {
      long long now = clock64();
      atomicAdd(&prof[slot], (unsigned long long)(now - last));  // fire and forget: no wait for the old value
      last = now;
    }
  }
};

// ---- exact sequential-order sum of non-negative floats in shared memory --------------
// (((0 + p[0]) + p[1]) + ...) with the rounding of a scalar f32 loop, evaluated by the
// chunked scheme of seqsum.cuh: lanes own chunks of SEQ_E terms, warps own groups of 32
// chunks. Pass 1 gives every chunk an inexact prefix sum (warp scan, then the group totals);
// pass 2 turns chunks into integer increments for their predicted exponents, joins runs of
// fast chunks with a segmented warp scan and writes the group's item list; one thread
// (of the last warp, which adds the opening chain while the others work) walks the items.
// Every thread of the group calls it and receives the result.
__device__ float group_seq_sum(const float* p, int n, SeqSumScratch* sc, const CtaGroup& g, unsigned long long* prof = nullptr) {
  SubProf sp{prof, clock64()};
  const int tid = g.tid, lane = tid & 31, warp = tid >> 5, nwarps = g.nthreads >> 5;
  const bool walker = tid == (nwarps - 1) * 32;
  g.sync();
  if (n <= SEQ_HEAD) {
    // short sums: one thread's add chain
    if (walker) {
      float s = 0.0f;
      for (int i = 0; i < n; i++) s = fadd(s, p[i]);
      sc->s = s;
    }
    g.sync();
    return sc->s;
  }
  if (walker) {
    // the opening chain, beside passes 1 and 2 of the warps that own groups
    float s = 0.0f;
    // all loads first, then the chain
    float hv[SEQ_HEAD];
#pragma unroll
    for (int k = 0; k < SEQ_HEAD; k++) hv[k] = p[k];
#pragma unroll
    for (int k = 0; k < SEQ_HEAD; k++) s = fadd(s, hv[k]);
    sc->s = s;
  }
  float approx = 0.0f;  // inexact sum of the passes before this one
  for (int base = 0; base < n; base += SEQ_CHUNKS * SEQ_E) {
    const int len = min(n - base, SEQ_CHUNKS * SEQ_E), nch = (len + SEQ_E - 1) / SEQ_E, ngr = (nch + 31) >> 5;
    // 1. inexact sums: per chunk, prefix inside the group, group totals
    for (int gr = warp; gr < ngr; gr += nwarps) {
      const int c = gr * 32 + lane, i0 = c * SEQ_E;
      float t = 0.0f;
#pragma unroll
      for (int j = 0; j < SEQ_E; j++) t += i0 + j < len ? p[base + i0 + j] : 0.0f;
      float incl = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      sc->excl[c] = incl - t;
      if (lane == 31) sc->gtot[gr] = incl;
    }
    g.sync();
    if (prof && tid == 0) sp.mark(26);
    // 2. predicted exponents, increments, runs, items
    float total = approx;
#pragma unroll
    for (int k = 0; k < SEQ_CHUNKS / 32; k++) total += k < ngr ? sc->gtot[k] : 0.0f;
    for (int gr = warp; gr < ngr; gr += nwarps) {
      const int c = gr * 32 + lane, i0 = c * SEQ_E;
      float before = approx;
#pragma unroll
      for (int k = 0; k < SEQ_CHUNKS / 32; k++) before += k < gr ? sc->gtot[k] : 0.0f;  // all loads issue together
      before += sc->excl[c];
      float t = 0.0f;
      uint32_t vb[SEQ_E];
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < SEQ_E; j++) {
        const float v = i0 + j < len ? p[base + i0 + j] : 0.0f;
        vb[j] = f2u(v) & 0x7FFFFFFFu;
        cnt += i0 + j < len ? 1 : 0;
        t += v;
      }
      const int eb = seq_exp_field(before), ea = seq_exp_field(before + t);
      const int head_lanes = base == 0 && gr == 0 ? SEQ_HEAD / SEQ_E : 0;  // chunks of the opening chain
      const bool live = lane >= head_lanes;
      bool bad = ea != eb || eb >= 255;
      int inc = 0;
#pragma unroll
      for (int j = 0; j < SEQ_E; j++) inc += seq_increment(vb[j], eb, bad);
      const bool slow = live && cnt > 0 && bad;
      inc = slow || !live ? 0 : min(inc, SUMFN_SAT);
      const int eb_prev = __shfl_up_sync(0xffffffffu, eb, 1);
      const int slow_prev = __shfl_up_sync(0xffffffffu, (int)slow, 1);
      const bool starts = live && (lane == head_lanes || slow_prev || eb != eb_prev);
      const uint32_t slow_mask = __ballot_sync(0xffffffffu, slow);
      const uint32_t begin = __ballot_sync(0xffffffffu, starts) | slow_mask;  // lanes at which an item begins
      // first chunk of this lane's item: the highest item begin at or below the lane
      const uint32_t below = begin & (0xFFFFFFFFu >> (31 - lane));
      const int rs = below ? 31 - __clz((int)below) : lane;
      // segmented inclusive scan of the increments inside runs
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane - d >= rs) inc = min(inc + o, SUMFN_SAT);
      }
      // the last chunk of an item writes it
      const bool next_begins = lane == 31 || ((begin >> (lane + 1)) & 1u);
      if (live && next_begins) {
        const int first = (gr * 32 + rs) * SEQ_E;
        SeqItem it;
        it.csum = inc;
        it.ep = slow ? -1 : eb;
        it.first = first;
        it.count = max(0, min(len, (c + 1) * SEQ_E) - first);
        sc->item[32 * gr + __popc(below) - 1] = it;
      }
      if (lane == 0) sc->n_items[gr] = __popc(begin);
    }
    g.sync();
    if (prof && tid == 0) sp.mark(28);
    // 3. the walk
    if (walker) {
      const long long tw = clock64();
      sc->s = seqsum_walk(p + base, sc, ngr, sc->s);
      if (prof) {
        atomicAdd(&prof[31], (unsigned long long)(clock64() - tw));
      }
    }
    if (prof && tid == 0) sp.mark(29);
    g.sync();
    approx = total;
  }
  return sc->s;
}

}  // namespace aot
