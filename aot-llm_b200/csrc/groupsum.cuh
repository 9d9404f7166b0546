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
// (((0 + p[0]) + p[1]) + ...) with the rounding of a scalar f32 loop (see seqsum.cuh).
// Terms are cut into 32-element segments. The binade in which each segment starts is
// predicted from an inexact prefix sum; every warp builds the exact composite
// "mantissa -> mantissa" function of its segments for the predicted binade; one thread
// then walks the segments, applying a composite when the prediction holds and the
// result stays inside the binade, and otherwise adding that segment's 32 terms one by
// one. A wrong prediction costs time, never accuracy.
constexpr int SEQSUM_SEGS = 128;  // segments per pass (4096 terms)

struct SeqSumScratch {
  float est[SEQSUM_SEGS];     // per-segment inexact sums, then predicted start values
  int csum[SEQSUM_SEGS];      // integer mantissa increment of the segment in its predicted binade
  int epred[SEQSUM_SEGS];     // predicted exponent field, or -1 when the segment needs term-by-term adds
  float s;
  float head_s;               // sum of the first 128 terms when an idle warp computed it ahead of the walk
};

// Every thread of the group calls it and receives the result.
//
// Inside one binade and without exact ties, adding a whole segment is adding the integer
// C = sum_i round(p_i / ulp) to the mantissa, so the walk over segments is an integer
// prefix sum (one warp, one scan per 32 segments). A segment is handled term by term,
// with real f32 adds, when its predicted binade is wrong, when the mantissa would leave
// the binade inside it, or when one of its terms is an exact tie.
__device__ float group_seq_sum(const float* p, int n, SeqSumScratch* sc, const CtaGroup& g, SubProf* sp = nullptr) {
  const int tid = g.tid, lane = tid & 31, warp = tid >> 5, nwarps = g.nthreads >> 5;
  g.sync();
  if (n <= 128) {
    // short sums: one warp, terms handed to the add chain by shuffles
    if (warp == 0) {
      float s = 0.0f;
      for (int c = 0; c < n; c += 32) {
        const float v = c + lane < n ? p[c + lane] : 0.0f;
#pragma unroll
        for (int k = 0; k < 32; k++) s = fadd(s, __shfl_sync(0xffffffffu, v, k));
      }
      if (lane == 0) sc->s = s;
    }
    g.sync();
    return sc->s;
  }
  if (tid == 0) sc->s = 0.0f;
  // The plain add chain over the first 128 terms (see the walk) can run beside steps 1-3
  // when the group's last warp has no segments of its own there.
  const int S_first = (min(n, SEQSUM_SEGS * 32) + 31) >> 5;
  const bool head_ahead = nwarps >= 2 && (nwarps - 1) * 4 >= S_first;
  if (head_ahead && warp == nwarps - 1) {
    float s = 0.0f;
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll 4
    for (int k = 0; k < 32; k++) {
      const float4 a = q[k];
      s = fadd(s, a.x);
      s = fadd(s, a.y);
      s = fadd(s, a.z);
      s = fadd(s, a.w);
    }
    if (lane == 0) sc->head_s = s;
  }
  for (int base = 0; base < n; base += SEQSUM_SEGS * 32) {
    const int len = min(n - base, SEQSUM_SEGS * 32), S = (len + 31) >> 5;
    // 1. inexact per-segment sums; a warp takes four segments at a time so that their
    //    shuffle chains overlap
    for (int seg0 = warp * 4; seg0 < S; seg0 += nwarps * 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = (seg0 + u) * 32 + lane;
        v[u] = i < len ? p[base + i] : 0.0f;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] += __shfl_xor_sync(0xffffffffu, v[u], o);
      }
      if (lane < 4 && seg0 + lane < S) sc->est[seg0 + lane] = lane == 0 ? v[0] : lane == 1 ? v[1] : lane == 2 ? v[2] : v[3];
    }
    g.sync();
    if (sp) sp->mark(26);
    // 2. predicted value at the start of every segment (one warp, the four 32-segment
    //    chunks scanned side by side)
    if (warp == 0) {
      float x[4], inc[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        x[u] = u * 32 + lane < S ? sc->est[u * 32 + lane] : 0.0f;
        inc[u] = x[u];
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const float y = __shfl_up_sync(0xffffffffu, inc[u], o);
          if (lane >= o) inc[u] += y;
        }
      }
      float run = sc->s;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (u * 32 + lane < S) sc->est[u * 32 + lane] = run + (inc[u] - x[u]);
        run += __shfl_sync(0xffffffffu, inc[u], 31);
      }
    }
    g.sync();
    if (sp) sp->mark(27);
    // 3. integer increment of every segment for its predicted binade, four segments per
    //    warp at a time
    for (int seg0 = warp * 4; seg0 < S; seg0 += nwarps * 4) {
      int c[4], e[4];
      bool bad[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int seg = seg0 + u;
        uint32_t b = seg < S ? f2u(sc->est[seg]) : 0u;
        if ((b >> 23) >= 255u || (b >> 31)) b = 0;
        int m;
        sum_decompose(b, e[u], m);
        const int i = seg * 32 + lane;
        const SumFn f = i < len ? sumfn_elem(f2u(p[base + i]), e[u]) : sumfn_identity();
        bad[u] = f.a0 != f.a1 || f.a0 >= SUMFN_SAT;
        c[u] = f.a0 > (1 << 25) ? (1 << 25) : f.a0;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; u++) c[u] += __shfl_xor_sync(0xffffffffu, c[u], o);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const unsigned any_bad = __ballot_sync(0xffffffffu, bad[u]);
        if (lane == u && seg0 + u < S) {
          sc->csum[seg0 + u] = c[u];
          sc->epred[seg0 + u] = any_bad ? -1 : e[u];
        }
      }
    }
    g.sync();
    if (sp) sp->mark(28);
    // 4. the walk (one warp, uniform control flow)
    if (warp == 0) {
      int e, m;
      // The first terms of a sum are about as large as the sum itself: binade changes and
      // ties at every step. They go through one plain add chain (every lane the same).
      int head_segs = 0;
      if (base == 0 && len >= 128) {
        float s = sc->s;  // 0
        if (head_ahead) {
          s = sc->head_s;
        } else {
          const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll 4
          for (int k = 0; k < 32; k++) {
            const float4 a = q[k];
            s = fadd(s, a.x);
            s = fadd(s, a.y);
            s = fadd(s, a.z);
            s = fadd(s, a.w);
          }
        }
        sum_decompose(f2u(s), e, m);
        head_segs = 4;
      } else {
        sum_decompose(f2u(sc->s), e, m);
      }
      for (int c0 = 0; c0 < S; c0 += 32) {
        const int seg = c0 + lane;
        const int cs = seg < S && seg >= head_segs ? sc->csum[seg] : 0;
        const int ep = seg < S ? sc->epred[seg] : -2;
        int pre = cs;  // inclusive prefix of the increments
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, pre, o);
          if (lane >= o) pre += y;
        }
        int j0 = c0 == 0 ? head_segs : 0, pbase = 0;
        for (int guard = 0; guard < 33; guard++) {
          const bool stop = lane >= j0 && (ep != e || m + (pre - pbase) >= SUMFN_LIMIT);
          const unsigned mask = __ballot_sync(0xffffffffu, stop);
          const int js = mask ? __ffs(mask) - 1 : 32;
          if (js > j0) {
            const int pend = __shfl_sync(0xffffffffu, pre, js - 1);
            m += pend - pbase;
            pbase = pend;
          }
          if (js >= 32 || c0 + js >= S) break;
          // segment c0 + js term by term
          float s = u2f(sum_pack(e, m));
          const int first = (c0 + js) * 32;
          if (first + 32 <= len) {
            // a full segment: every lane reads the same 32 terms (broadcast loads)
            const float4* q = reinterpret_cast<const float4*>(p + base + first);
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
              const float4 a = q[k], b = q[k + 1];
              s = fadd(s, a.x);
              s = fadd(s, a.y);
              s = fadd(s, a.z);
              s = fadd(s, a.w);
              s = fadd(s, b.x);
              s = fadd(s, b.y);
              s = fadd(s, b.z);
              s = fadd(s, b.w);
            }
          } else {
            const int i = first + lane;
            const float v = i < len ? p[base + i] : 0.0f;
#pragma unroll
            for (int k = 0; k < 32; k++) s = fadd(s, __shfl_sync(0xffffffffu, v, k));
          }
          sum_decompose(f2u(s), e, m);
          pbase = __shfl_sync(0xffffffffu, pre, js);
          j0 = js + 1;
        }
      }
      if (lane == 0) sc->s = u2f(sum_pack(e, m));
    }
    if (sp) sp->mark(29);
    g.sync();
    if (sp) sp->mark(30);
  }
  return sc->s;
}

}  // namespace aot
