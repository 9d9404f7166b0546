// Activation quantizers and the non-matmul operators of a transformer block
// (crates/aot-kernels/src/quant.rs:231-283, crates/aot-kernels/src/ops.rs,
// crates/aot-kernels/src/sampler.rs:99-109) as CUDA kernels.
//
// The reference's f32 reductions are strictly sequential loops. Results here
// are bit-identical: every reduction whose order is observable (sum of
// squares, q.k dots, softmax denominator, the value mix) is evaluated in the
// reference's order with unfused round-to-nearest operations; order-free
// reductions (max, argmax, integer sums) run in parallel.
#pragma once
#include "blockmath.cuh"
#include "device_utils.cuh"
#include "expf_exact.cuh"
#include "groupsum.cuh"

namespace aot {

// ---- sequential-order sum of a shared-memory array --------------------------------
// (((0 + p[0]) + p[1]) + ...) exactly as a scalar loop would round it. Called by
// the whole block; the result is returned to every thread. `slot` is one float of
// shared memory.
__device__ __forceinline__ float block_seq_sum(const float* p, int n, float* slot) {
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
      float a0 = p[i], a1 = p[i + 1], a2 = p[i + 2], a3 = p[i + 3], a4 = p[i + 4], a5 = p[i + 5], a6 = p[i + 6],
            a7 = p[i + 7];
      s = fadd(s, a0);
      s = fadd(s, a1);
      s = fadd(s, a2);
      s = fadd(s, a3);
      s = fadd(s, a4);
      s = fadd(s, a5);
      s = fadd(s, a6);
      s = fadd(s, a7);
    }
    for (; i < n; i++) s = fadd(s, p[i]);
    *slot = s;
  }
  __syncthreads();
  return *slot;
}

// ---- Q8_K quantization of one 256-value block by one warp ----------------------------
// quant.rs:248-283. `src` may be shared or global. The block is written either in
// the reference's BlockQ8_K layout (image == 0) or as the 304-byte image the GEMV
// kernels read (image == 1).
// Core: lane holds elements 8*lane .. 8*lane+7 of the block in v[].
__device__ __forceinline__ void warp_quantize_q8k_vals(const float (&v)[8], uint8_t* dst, int image) {
  const int lane = threadIdx.x & 31;
  // signed extreme: the first element with strictly larger |v|. |v| orders like its bit
  // pattern; a NaN never compares larger in the reference and counts as zero here. Two
  // warp-wide integer reductions find the largest pattern and the first index holding it.
  uint32_t best = 0;
  float mx = 0.0f;
  int idx = 8 * lane;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    uint32_t a = __float_as_uint(v[i]) & 0x7FFFFFFFu;
    a = a > 0x7F800000u ? 0u : a;
    if (a > best) {
      best = a;
      mx = v[i];
      idx = 8 * lane + i;
    }
  }
  const uint32_t wmax = __reduce_max_sync(0xffffffffu, best);
  const uint32_t widx = __reduce_min_sync(0xffffffffu, best == wmax ? (uint32_t)idx : 256u);
  mx = __shfl_sync(0xffffffffu, mx, (int)(widx >> 3));
  const float amax = __uint_as_float(wmax);
  int8_t* qs = reinterpret_cast<int8_t*>(dst + (image ? 0 : 4));
  int16_t* bs = reinterpret_cast<int16_t*>(dst + (image ? 256 : 260));
  float* dptr = reinterpret_cast<float*>(dst + (image ? 288 : 0));
  uint32_t w0 = 0, w1 = 0;
  int s = 0;
  float d = 0.0f;
  if (amax != 0.0f) {
    float iscale = fdiv(-127.0f, mx);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int q = (int)roundf(fmul(iscale, v[i]));
      q = q > 127 ? 127 : q;
      s += q;
      uint32_t b = (uint32_t)(q & 0xFF);
      if (i < 4) w0 |= b << (8 * i); else w1 |= b << (8 * (i - 4));
    }
    d = fdiv(1.0f, iscale);
  }
  reinterpret_cast<uint32_t*>(qs)[2 * lane] = w0;
  reinterpret_cast<uint32_t*>(qs)[2 * lane + 1] = w1;
  int s2 = s + __shfl_xor_sync(0xffffffffu, s, 1);
  if ((lane & 1) == 0) bs[lane >> 1] = (int16_t)s2;
  if (lane == 0) *dptr = d;
}

template <bool CG = false>
__device__ __forceinline__ void warp_quantize_q8k(const float* src, uint8_t* dst, int image) {
  const int lane = threadIdx.x & 31;
  float v[8];
  if (CG) {
    // data written by other CTAs of the same launch: bypass L1
    float4 a = __ldcg(reinterpret_cast<const float4*>(src) + 2 * lane), b = __ldcg(reinterpret_cast<const float4*>(src) + 2 * lane + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = src[8 * lane + i];
  }
  warp_quantize_q8k_vals(v, dst, image);
}

// quant.rs:231-245 for one 32-value block handled by one warp (lane = element).
__device__ __forceinline__ void warp_quantize_q80(const float* src, uint8_t* dst, int image) {
  const int lane = threadIdx.x & 31;
  float v = src[lane];
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float d = fdiv(amax, 127.0f);
  float id = d != 0.0f ? fdiv(1.0f, d) : 0.0f;
  int q = (int)roundf(fmul(v, id));
  q = q < -127 ? -127 : (q > 127 ? 127 : q);
  reinterpret_cast<int8_t*>(dst + (image ? 0 : 4))[lane] = (int8_t)q;
  if (lane == 0) *reinterpret_cast<float*>(dst + (image ? 32 : 0)) = d;
}

constexpr int XIMG_K = 304;  // bytes per Q8_K block image
constexpr int XIMG_0 = 48;   // bytes per Q8_0 block image

// Quantize `n_total` floats (a multiple of the block size; rows back to back).
__global__ void quantize_q8k_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, int n_blocks, int image) {
  pdl_launch_dependents();
  pdl_wait();
  int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int nw = (gridDim.x * blockDim.x) >> 5;
  for (int b = wid; b < n_blocks; b += nw) warp_quantize_q8k(x + (size_t)b * 256, out + (size_t)b * (image ? XIMG_K : 292), image);
}
__global__ void quantize_q80_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, int n_blocks, int image) {
  pdl_launch_dependents();
  pdl_wait();
  int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int nw = (gridDim.x * blockDim.x) >> 5;
  for (int b = wid; b < n_blocks; b += nw) warp_quantize_q80(x + (size_t)b * 32, out + (size_t)b * (image ? XIMG_0 : 36), image);
}

// Reference-layout blocks -> images (for callers that hand in BlockQ8_K / BlockQ8_0 arrays).
__global__ void q8k_to_image_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int n_blocks) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks * 73; i += gridDim.x * blockDim.x) {
    int b = i / 73, w = i - b * 73;
    int off = w == 0 ? 288 : (w <= 64 ? (w - 1) * 4 : 256 + (w - 65) * 4);
    *reinterpret_cast<uint32_t*>(out + (size_t)b * XIMG_K + off) = reinterpret_cast<const uint32_t*>(in)[i];
  }
}
__global__ void q80_to_image_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int n_blocks) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks * 9; i += gridDim.x * blockDim.x) {
    int b = i / 9, w = i - b * 9;
    int off = w == 0 ? 32 : (w - 1) * 4;
    *reinterpret_cast<uint32_t*>(out + (size_t)b * XIMG_0 + off) = reinterpret_cast<const uint32_t*>(in)[i];
  }
}

// ---- rmsnorm (ops.rs:7-18), one CTA per row, optional fused quantization ------------------
// out may alias x. When q8k_out / q80_out are given, the normalised row is also
// quantized (as the generated code does right after every rmsnorm, emit.rs:131-139).
struct RmsnormParams {
  const float* x;
  const float* w;
  float* out;
  int n;
  int x_stride, out_stride;
  float eps;
  int accumulate;    // out[i] = out[i] + y[i] (Gemma post-norm residual join)
  uint8_t* q8k_out;  // images, n/256 per row
  uint8_t* q80_out;  // images, n/32 per row
};

__global__ void __launch_bounds__(512) rmsnorm_kernel(const RmsnormParams P) {
  extern __shared__ __align__(16) float sm_f[];
  float* row = sm_f;          // n
  float* sq = sm_f + P.n;     // n
  __shared__ SeqSumScratch ssc;
  pdl_launch_dependents();
  pdl_wait();
  const float* x = P.x + (size_t)blockIdx.x * P.x_stride;
  float* out = P.out + (size_t)blockIdx.x * P.out_stride;
  for (int i = threadIdx.x; i < P.n; i += blockDim.x) {
    float v = x[i];
    row[i] = v;
    sq[i] = fmul(v, v);
  }
  __syncthreads();
  float ss = group_seq_sum(sq, P.n, &ssc, CtaGroup{(int)threadIdx.x, (int)blockDim.x, 0});
  float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)P.n), P.eps)));
  for (int i = threadIdx.x; i < P.n; i += blockDim.x) {
    float y = fmul(fmul(row[i], r), P.w[i]);
    row[i] = y;
    if (P.out) out[i] = P.accumulate ? fadd(out[i], y) : y;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (P.q8k_out) {
    int nb = P.n / 256;
    for (int b = warp; b < nb; b += nwarps)
      warp_quantize_q8k(row + b * 256, P.q8k_out + ((size_t)blockIdx.x * nb + b) * XIMG_K, 1);
  }
  if (P.q80_out) {
    int nb = P.n / 32;
    for (int b = warp; b < nb; b += nwarps)
      warp_quantize_q80(row + b * 32, P.q80_out + ((size_t)blockIdx.x * nb + b) * XIMG_0, 1);
  }
}

// ---- per-head rmsnorm + RoPE + KV store ("qk post") -----------------------------------------
// After the q/k/v products of one or more tokens: optional per-head RMSNorm of q
// and k (ops.rs:74-87), RoPE in the adjacent-pair or NEOX layout (ops.rs:40-70)
// with the (cos, sin) row of each token's position, then k and v are copied into
// the cache (ops.rs:152-157, 505-510). One CTA per (head slot, token): head slots
// 0..n_head-1 are query heads, n_head..n_head+n_kv-1 key heads (which also move
// the matching value head).
struct QkPostParams {
  float* q;           // m x q_dim, in place
  const float* k;     // m x kv_dim
  const float* v;     // m x kv_dim
  float* k_cache;     // already offset to the layer: ctx x kv_dim
  float* v_cache;
  const float* q_norm;  // head_dim weights or null
  const float* k_norm;
  const float* rope_table;  // ctx x rot_dim, interleaved (cos, sin)
  const int* pos_ptr;       // device word holding pos0 (or null -> pos0 below)
  int pos0;
  int n_head, n_kv_head, head_dim, rot_dim;
  int neox;
  float eps;
};

__global__ void __launch_bounds__(128) qk_post_kernel(const QkPostParams P) {
  __shared__ float h[256];
  __shared__ float sq[256];
  __shared__ float slot;
  pdl_launch_dependents();
  pdl_wait();
  const int hs = blockIdx.x, tok = blockIdx.y;
  const int pos = (P.pos_ptr ? *P.pos_ptr : P.pos0) + tok;
  const int hd = P.head_dim;
  const bool is_q = hs < P.n_head;
  const int kvh = hs - P.n_head;
  const int q_dim = P.n_head * hd, kv_dim = P.n_kv_head * hd;
  const float* src = is_q ? P.q + (size_t)tok * q_dim + hs * hd : P.k + (size_t)tok * kv_dim + kvh * hd;
  const float* nw = is_q ? P.q_norm : P.k_norm;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float a = src[i];
    h[i] = a;
    sq[i] = fmul(a, a);
  }
  if (nw) {
    float ss = block_seq_sum(sq, hd, &slot);
    float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)hd), P.eps)));
    for (int i = threadIdx.x; i < hd; i += blockDim.x) h[i] = fmul(fmul(h[i], r), nw[i]);
  }
  __syncthreads();
  const float* cs = P.rope_table + (size_t)pos * P.rot_dim;
  const int half = P.rot_dim / 2;
  float* dst = is_q ? P.q + (size_t)tok * q_dim + hs * hd : P.k_cache + (size_t)pos * kv_dim + kvh * hd;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    int i0 = P.neox ? i : 2 * i, i1 = P.neox ? i + half : 2 * i + 1;
    float c = cs[2 * i], s = cs[2 * i + 1];
    float x0 = h[i0], x1 = h[i1];
    dst[i0] = fsub(fmul(x0, c), fmul(x1, s));
    dst[i1] = fadd(fmul(x0, s), fmul(x1, c));
  }
  for (int i = P.rot_dim + threadIdx.x; i < hd; i += blockDim.x) dst[i] = h[i];
  if (!is_q) {
    const float* vs = P.v + (size_t)tok * kv_dim + kvh * hd;
    float* vd = P.v_cache + (size_t)pos * kv_dim + kvh * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) vd[i] = vs[i];
  }
}

// Stand-alone pieces of the same, for the operator-level API.
__global__ void rope_kernel(float* x, int m, int n_heads, int head_dim, int rot_dim, const float* cs, int cs_stride,
                            int neox) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  const int half = rot_dim / 2;
  const size_t total = (size_t)m * n_heads * half;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    int i = (int)(t % half);
    size_t hh = t / half;
    int row = (int)(hh / n_heads);
    float* v = x + hh * head_dim;
    const float* c_s = cs + (size_t)row * cs_stride;
    int i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
    float c = c_s[2 * i], s = c_s[2 * i + 1];
    float x0 = v[i0], x1 = v[i1];
    v[i0] = fsub(fmul(x0, c), fmul(x1, s));
    v[i1] = fadd(fmul(x0, s), fmul(x1, c));
  }
}

__global__ void __launch_bounds__(128) rmsnorm_heads_kernel(float* x, const float* w, int head_dim, float eps) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  __shared__ float h[256];
  __shared__ float sq[256];
  __shared__ float slot;
  float* v = x + (size_t)blockIdx.x * head_dim;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    float a = v[i];
    h[i] = a;
    sq[i] = fmul(a, a);
  }
  float ss = block_seq_sum(sq, head_dim, &slot);
  float r = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)head_dim), eps)));
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) v[i] = fmul(fmul(h[i], r), w[i]);
}

// ---- attention (ops.rs:185-218, 517-556) ------------------------------------------------------
// One CTA per (group of up to 8 query heads that share a KV head, query row); one warp
// per query head. Cached K and V rows are staged through shared memory once per CTA and
// used by all its heads. Scores and the softmax live in shared memory (or in `scratch`
// for contexts that do not fit). Order-sensitive reductions keep the reference's order:
// each q.k dot is one sequential chain, the softmax denominator is the exact sequential
// sum, the value mix runs over positions in order.
struct AttnParams {
  float* out;         // m x q_dim
  const float* q;     // m x q_dim
  const float* k_cache;  // layer base: ctx x kv_dim
  const float* v_cache;
  float* scratch;     // (m x n_head) x ctx floats, used when smem_scores == 0
  const int* pos_ptr;
  int pos0;
  int n_head, n_kv_head, head_dim, ctx, window;
  int smem_scores;    // capacity (floats per head) of the shared score buffer, 0 = use scratch
  int heads_per_cta;  // query heads of one KV head handled by a CTA (<= 8)
  int rows_per_cta;   // consecutive query rows handled by a CTA (heads_per_cta x rows_per_cta warps, <= 16)
  int m;              // query rows
  int chunk;          // cached positions per staging buffer
  float scale;
};

constexpr int ATTN_MAX_WARPS = 16;
// Bytes of the warps' exact-sum scratch at the head of the kernel's shared memory, rounded so
// that what follows stays 16-byte aligned for any warp count.
__host__ __device__ inline size_t attn_ssc_bytes(size_t warps) { return (warps * sizeof(SeqSumScratch) + 15) & ~(size_t)15; }
constexpr int ATTN_CHUNK = 64;      // cached positions staged at a time ...
constexpr int ATTN_CHUNK_BIG = 128;  // ... or this many when shared memory allows: half the staging rounds

// o[j] += a[t] * v[t][lane + 32 j] for t in [ta, tb), positions in order (ops.rs:208-214), for
// the NJ dims a lane owns; only the last of them can lie beyond the head width.
template <int NJ>
__device__ __forceinline__ void attn_value_mix(float (&o)[8], const float* a, const float* cur, int ta, int tb, int hd, int lane) {
  const bool last = lane + 32 * (NJ - 1) < hd;
#pragma unroll 4
  for (int t = ta; t < tb; t++) {
    const float at = a[t];
    const float* v = cur + t * hd + lane;
#pragma unroll
    for (int j = 0; j < NJ - 1; j++) o[j] = fadd(o[j], fmul(at, v[32 * j]));
    if (last) o[NJ - 1] = fadd(o[NJ - 1], fmul(at, v[32 * (NJ - 1)]));
  }
}

// One CTA serves `rows_per_cta` consecutive query rows of one KV head: a warp per (row, query
// head). The cached rows the CTA stages cover the union of its rows' ranges (rows differ by
// one position each, and by their window start), so they are fetched once for all of them.
__global__ void __launch_bounds__(ATTN_MAX_WARPS * 32) attention_kernel(const AttnParams P) {
  extern __shared__ __align__(16) float sm_f[];
  pdl_launch_dependents();
  pdl_wait();
  const int hd = P.head_dim, hd4 = hd >> 2, kv_dim = P.n_kv_head * hd, q_dim = P.n_head * hd;
  const int gqa = P.n_head / P.n_kv_head, hpc = P.heads_per_cta, rpc = P.rows_per_cta;
  const int nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int splits = (gqa + hpc - 1) / hpc;
  const int kvh = blockIdx.x / splits, part = blockIdx.x - kvh * splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rs = warp / hpc, wh = warp - rs * hpc;            // row slot and head slot of this warp
  const int row = blockIdx.y * rpc + rs;
  const int h_local = part * hpc + wh;                        // head inside the KV group
  const bool has_head = rs < rpc && row < P.m && h_local < gqa;
  const int h = kvh * gqa + (h_local < gqa ? h_local : 0);
  const int base_pos = P.pos_ptr ? *P.pos_ptr : P.pos0;
  const int pos = base_pos + row;
  const int n = pos + 1;
  const int t0 = (P.window > 0 && pos + 1 > P.window) ? pos + 1 - P.window : 0;
  const int len = n - t0;
  // the CTA's rows: first and last valid one, and the union [T0, N) of their ranges
  const int row_a = blockIdx.y * rpc, row_b = min(row_a + rpc, P.m) - 1;
  const int pos_a = base_pos + row_a, pos_b = base_pos + row_b;
  const int T0 = (P.window > 0 && pos_a + 1 > P.window) ? pos_a + 1 - P.window : 0;
  const int LEN = pos_b + 1 - T0;
  const int kstride = hd + 4, CH = P.chunk;
  SeqSumScratch* ssc = reinterpret_cast<SeqSumScratch*>(sm_f);
  float* qs = sm_f + attn_ssc_bytes(nwarps) / sizeof(float);  // nwarps x hd, 16-byte aligned
  float* kv = qs + nwarps * hd;                       // two buffers of CH x (hd + 4)
  const int buf_floats = CH * kstride;
  float* sc_all = kv + 2 * buf_floats;                // nwarps x smem_scores
  float* sc = P.smem_scores ? sc_all + warp * P.smem_scores : P.scratch + ((size_t)(has_head ? row : 0) * P.n_head + h) * P.ctx;
  for (int i = threadIdx.x; i < nwarps * hd; i += nthreads) {
    const int w = i / hd, wr = w / hpc, hl = part * hpc + (w - wr * hpc), r = row_a + wr;
    qs[i] = (wr < rpc && r < P.m && hl < gqa) ? P.q[(size_t)r * q_dim + (kvh * gqa + hl) * hd + (i - w * hd)] : 0.0f;
  }
  // Cached rows [c0, c0 + cn) of the union, of this KV head, into a chunk buffer with cp.async:
  // the next chunk loads while the current one is consumed.
  auto stage = [&](float* buf, const float* cache, int stride, int c0, int cn) {
    for (int j = threadIdx.x; j < cn * hd4; j += nthreads) {
      const int t = j / hd4, i4 = j - t * hd4;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(buf + t * stride + 4 * i4)),
                   "l"(cache + (size_t)(T0 + c0 + t) * kv_dim + kvh * hd + 4 * i4)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // scores: dot(q, k_t) * scale, each dot a sequential f32 loop (ops.rs:160-166)
  float lmax = -INFINITY;
  const float* qh = qs + warp * hd;
  const int off = t0 - T0;                            // this row's first position inside the union
  stage(kv, P.k_cache, kstride, 0, min(CH, LEN));
  for (int c0 = 0, ci = 0; c0 < LEN; c0 += CH, ci++) {
    const int cn = min(CH, LEN - c0);
    const float* cur = kv + (ci & 1) * buf_floats;
    if (c0 + CH < LEN) {
      stage(kv + ((ci + 1) & 1) * buf_floats, P.k_cache, kstride, c0 + CH, min(CH, LEN - c0 - CH));
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (has_head) {
      for (int t = lane; t < cn; t += 32) {
        const int u = c0 + t - off;                   // position index inside this row's range
        if (u < 0 || u >= len) continue;
        const float4* kt = reinterpret_cast<const float4*>(cur + t * kstride);
        float s = 0.0f;
#pragma unroll 4
        for (int i = 0; i < hd4; i++) {
          const float4 kk = kt[i];
          const float4 qq = reinterpret_cast<const float4*>(qh)[i];
          s = fadd(s, fmul(qq.x, kk.x));
          s = fadd(s, fmul(qq.y, kk.y));
          s = fadd(s, fmul(qq.z, kk.z));
          s = fadd(s, fmul(qq.w, kk.w));
        }
        s = fmul(s, P.scale);
        sc[u] = s;
        lmax = fmaxf(lmax, s);
      }
    }
    __syncthreads();  // this buffer is refilled two chunks later
  }
  // the first chunk of V rows loads while the softmax runs
  stage(kv, P.v_cache, hd, 0, min(CH, LEN));
  if (has_head) {
    // this head's softmax, by its own warp: max (order-free), exp, the denominator in
    // position order (ops.rs:103-107)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    __syncwarp();
    for (int t = lane; t < len; t += 32) sc[t] = expf_exact(fsub(sc[t], lmax));
    __syncwarp();
    const float sum = group_seq_sum(sc, len, &ssc[warp], CtaGroup{lane, 32, 1 + warp});
    const float inv = fdiv(1.0f, sum);
    for (int t = lane; t < len; t += 32) sc[t] = fmul(sc[t], inv);
    __syncwarp();
  }
  // out[i] = sum_t a_t * v_t[i], t in order (ops.rs:208-214); lane owns dims lane, lane+32, ...
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) o[j] = 0.0f;
  for (int c0 = 0, ci = 0; c0 < LEN; c0 += CH, ci++) {
    const int cn = min(CH, LEN - c0);
    const float* cur = kv + (ci & 1) * buf_floats;
    if (c0 + CH < LEN) {
      stage(kv + ((ci + 1) & 1) * buf_floats, P.v_cache, hd, c0 + CH, min(CH, LEN - c0 - CH));
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (has_head) {
      // this row's positions inside the chunk; the loop over a lane's dims is instantiated for
      // the head width (predicated-off iterations of a fixed eight would still issue)
      const int ta = max(0, off - c0), tb = min(cn, off + len - c0);
      const float* a = sc + (c0 - off);
      switch ((hd + 31) >> 5) {
        case 1: attn_value_mix<1>(o, a, cur, ta, tb, hd, lane); break;
        case 2: attn_value_mix<2>(o, a, cur, ta, tb, hd, lane); break;
        case 3: attn_value_mix<3>(o, a, cur, ta, tb, hd, lane); break;
        case 4: attn_value_mix<4>(o, a, cur, ta, tb, hd, lane); break;
        case 5: attn_value_mix<5>(o, a, cur, ta, tb, hd, lane); break;
        case 6: attn_value_mix<6>(o, a, cur, ta, tb, hd, lane); break;
        case 7: attn_value_mix<7>(o, a, cur, ta, tb, hd, lane); break;
        default: attn_value_mix<8>(o, a, cur, ta, tb, hd, lane); break;  // head_dim <= 256
      }
    }
    __syncthreads();
  }
  if (has_head) {
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (lane + 32 * j < hd) P.out[(size_t)row * q_dim + h * hd + lane + 32 * j] = o[j];
  }
}

// ---- element-wise ----------------------------------------------------------------------------------
__global__ void silu_mul_kernel(float* h, const float* up, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = h[i];
    h[i] = fmul(fdiv(v, fadd(1.0f, expf_exact(-v))), up[i]);
  }
}
// GELU, tanh approximation (ops.rs:124-127): 0.5 v (1 + tanh(k (v + 0.044715 v^3))) with every
// product and sum rounded to f32 in the reference's order. The reference takes tanh from
// the platform's libm; here it is the correctly rounded f32 value (double tanh, then one
// rounding), which is what a correctly rounded libm returns.
__device__ __forceinline__ float gelu_exact(float v) {
  const float k = 1.1283791670955126f / 1.4142135623730951f;  // FRAC_2_SQRT_PI / SQRT_2 in f32
  const float cube = fmul(fmul(fmul(0.044715f, v), v), v);
  const float t = (float)tanh((double)fmul(k, fadd(v, cube)));
  return fmul(fmul(0.5f, v), fadd(1.0f, t));
}
// h = gelu(h) * up (ops.rs:130-134)
__global__ void gelu_mul_kernel(float* h, const float* up, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    h[i] = fmul(gelu_exact(h[i]), up[i]);
}
__global__ void add_inplace_kernel(float* x, const float* y, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = fadd(x[i], y[i]);
}
__global__ void add_bias_rows_kernel(float* x, const float* b, size_t n, size_t m) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * m; i += (size_t)gridDim.x * blockDim.x)
    x[i] = fadd(x[i], b[i % n]);
}
__global__ void scale_inplace_kernel(float* x, float s, size_t n) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = fmul(x[i], s);
}
__global__ void store_kv_kernel(float* k_cache, float* v_cache, const float* k, const float* v, size_t n,
                                const int* pos_ptr, int pos0, int kv_dim) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  size_t at = (size_t)(pos_ptr ? *pos_ptr : pos0) * kv_dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    k_cache[at + i] = k[i];
    v_cache[at + i] = v[i];
  }
}

// ---- token embedding rows (quant.rs:300-443 through emit.rs:469, 497) ---------------------------------
__global__ void embed_rows_kernel(float* out, const uint8_t* table, const int* tokens, int kind, int dim,
                                  size_t row_bytes, float scale, int do_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = tokens[blockIdx.y];
  const uint8_t* row = table + (size_t)tok * row_bytes;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < dim; e += gridDim.x * blockDim.x) {
    float v = dequant_elem(kind, row, (size_t)e);
    out[(size_t)blockIdx.y * dim + e] = do_scale ? fmul(v, scale) : v;
  }
}

// ---- greedy argmax (sampler.rs:99-109): the first maximum wins, NaN never does ----------------------------
// `step`, when given, is the device-side decode cursor {token, pos, n_generated}:
// the winner becomes the next step's token, is appended to `history`, and the
// position advances, so a generation loop needs no host round trip per token.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* x, int n, int* out_token, int* step, int* history,
                                                      int history_cap) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_launch_dependents();
  pdl_wait();
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = x[i];
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
  if ((threadIdx.x & 31) == 0) {
    bv[threadIdx.x >> 5] = best;
    bi[threadIdx.x >> 5] = idx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) {
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
        best = bv[w];
        idx = bi[w];
      }
    }
    if (idx == 0x7fffffff) idx = 0;  // nothing exceeded -inf
    if (out_token) *out_token = idx;
    if (step) {
      int g = step[2];
      if (history && g < history_cap) history[g] = idx;
      step[0] = idx;
      step[1] = step[1] + 1;
      step[2] = g + 1;
    }
  }
}

}  // namespace aot
