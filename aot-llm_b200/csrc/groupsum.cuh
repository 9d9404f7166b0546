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
// pass 2 builds the chunk composites for the predicted exponents and joins runs of fast
// chunks with a segmented warp scan; one thread walks the records. Every thread of the
// group calls it and receives the result. About 1.5 K cycles for 2048 terms, against 8 K
// for the dependent chain of adds.
__device__ __forceinline__ SumFn shfl_up_fn(const SumFn& f, int d) {
  SumFn r;
  r.a0 = __shfl_up_sync(0xffffffffu, f.a0, d);
  r.a1 = __shfl_up_sync(0xffffffffu, f.a1, d);
  return r;
}

__device__ float group_seq_sum(const float* p, int n, SeqSumScratch* sc, const CtaGroup& g, SubProf* sp = nullptr) {
  const int tid = g.tid, lane = tid & 31, warp = tid >> 5, nwarps = g.nthreads >> 5;
  g.sync();
  if (n <= 64) {
    // short sums: one thread's add chain
    if (tid == 0) {
      float s = 0.0f;
      for (int i = 0; i < n; i++) s = fadd(s, p[i]);
      sc->s = s;
    }
    g.sync();
    return sc->s;
  }
  if (tid == 0) sc->s = 0.0f;
  for (int base = 0; base < n; base += SEQ_CHUNKS * SEQ_E) {
    const int len = min(n - base, SEQ_CHUNKS * SEQ_E), nch = (len + SEQ_E - 1) / SEQ_E, ngr = (nch + 31) >> 5;
    // 1. inexact sums: per chunk, prefix inside the group (parked in ep[]), group totals
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
      sc->ep[c] = (int)f2u(incl - t);
      if (lane == 31) sc->gtot[gr] = incl;
    }
    g.sync();
    if (sp) sp->mark(26);
    // 2. predicted exponents, chunk composites, runs
    const float run0 = sc->s;
    for (int gr = warp; gr < ngr; gr += nwarps) {
      const int c = gr * 32 + lane, i0 = c * SEQ_E;
      float before = run0;
      for (int k = 0; k < gr; k++) before += sc->gtot[k];
      before += u2f((uint32_t)sc->ep[c]);
      float v[SEQ_E], t = 0.0f;
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < SEQ_E; j++) {
        v[j] = i0 + j < len ? p[base + i0 + j] : 0.0f;
        cnt += i0 + j < len ? 1 : 0;
        t += v[j];
      }
      const int eb = seq_exp_field(before), ea = seq_exp_field(before + t);
      const bool slow = cnt > 0 && (ea != eb || eb >= 255);
      const int eb_prev = __shfl_up_sync(0xffffffffu, eb, 1);
      const int slow_prev = __shfl_up_sync(0xffffffffu, (int)slow, 1);
      const bool starts = lane == 0 || slow_prev || eb != eb_prev;
      const uint32_t slow_mask = __ballot_sync(0xffffffffu, slow), start_mask = __ballot_sync(0xffffffffu, starts);
      SumFn f = sumfn_identity();
      if (!slow) {
#pragma unroll
        for (int j = 0; j < SEQ_E; j++) f = sumfn_compose(f, sumfn_elem(f2u(v[j]) & 0x7FFFFFFFu, eb));
      }
      // first chunk of this lane's run: the highest run start at or below the lane
      const int rs = 31 - __clz((int)(start_mask & (0xFFFFFFFFu >> (31 - lane))));
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const SumFn o = shfl_up_fn(f, d);
        if (!slow && lane - d >= rs) f = sumfn_compose(o, f);
      }
      sc->a0[c] = f.a0;
      sc->a1[c] = f.a1;
      sc->ep[c] = eb;
      if (lane == 0) {
        sc->slow[gr] = slow_mask;
        sc->start[gr] = start_mask;
      }
    }
    g.sync();
    if (sp) sp->mark(28);
    // 3. the walk
    if (tid == 0) sc->s = seqsum_walk(p + base, len, sc, nch, run0);
    if (sp) sp->mark(29);
    g.sync();
  }
  return sc->s;
}

}  // namespace aot
