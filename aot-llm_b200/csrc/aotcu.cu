// Host side of libaot_cuda: context, kernel launchers, the device-resident State
// and the operator API that mirrors the reference's GPU backend slot
// (crates/aot-kernels/src/metal.rs `Gpu`), the interpreted forward pass
// (crates/aot-codegen/src/emit.rs:243-333, 466-516) and the extern "C" surface
// declared in include/aot_cuda.h.
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include <dlfcn.h>

#include "../../include/aot_cuda.h"
#include "gemv.cuh"
#include "gemm.cuh"
#include "gemm_tc.cuh"
#include "mega.cuh"
#include "q80stream.cuh"
#include "floatstream.cuh"
#include "ops.cuh"

using namespace aot;

// ---- errors ------------------------------------------------------------------------
static thread_local std::string g_last_error;

static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define CU_TRY(expr)                                                                                  \
  do {                                                                                                \
    cudaError_t e_ = (expr);                                                                          \
    if (e_ != cudaSuccess) return fail(AOTCU_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_));      \
  } while (0)

#define ARG_CHECK(cond, ...)                                  \
  do {                                                        \
    if (!(cond)) return fail(AOTCU_ERR_BAD_ARG, __VA_ARGS__); \
  } while (0)

static_assert(sizeof(aotcu_block_q8_0) == 36 && sizeof(aotcu_block_q8_k) == 292, "block layout");

// ---- context --------------------------------------------------------------------------
struct aotcu_ctx {
  int device = 0;
  int n_sm = 0;
  size_t max_smem = 0;
  cudaStream_t stream = nullptr;
  int* d_err = nullptr;
  bool pdl = true;  // programmatic dependent launch between the kernels of a stream
  uint64_t launches = 0;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  std::vector<struct aotcu_gpu*> gpus;  // live Gpus of this context (freed with it)
  uint8_t* ximg = nullptr;              // Q8_0 activation images made from reference-layout blocks (launch_q80_stream)
  size_t ximg_bytes = 0;
};

constexpr size_t WEIGHT_PAD = 256;

static int ctx_set_device(aotcu_ctx* c) {
  CU_TRY(cudaSetDevice(c->device));
  return 0;
}

template <class... KArgs, class... Args>
static int launch(aotcu_ctx* c, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  if (c->pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  c->launches++;
  return 0;
}

static int grid_for(aotcu_ctx* c, size_t work_items, int per_block) {
  size_t g = (work_items + per_block - 1) / per_block;
  size_t cap = (size_t)c->n_sm * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// ---- GEMV / matmul launcher ------------------------------------------------------------
struct GemvCall {
  GemvSeg seg[3];
  int nseg = 1;
  int pair = 0;
  size_t cols = 0;
  const void* x = nullptr;
  int x_mode = 0;  // 0 reference-layout blocks (or f32 for float kinds), 1 block images
  size_t m = 1;
  int epilogue = EPI_STORE;
  const uint8_t* prep[3] = {nullptr, nullptr, nullptr};  // prepared tensor-core operands of each matrix, if any
};

static int check_weight_alignment(int kind, const void* w) {
  uintptr_t a = (uintptr_t)w;
  uintptr_t need = (kind == Q4_K || kind == Q5_K) ? 16 : (kind == F32 ? 4 : 2);
  ARG_CHECK((a % need) == 0, "weights of kind %d must be %zu-byte aligned", kind, (size_t)need);
  return 0;
}

// m = 8..64 activation rows against K-quant matrices: int8 tensor-core tiles (gemm.cuh).
// Arguments were checked by launch_gemv.
template <bool PAIR>
static int launch_gemm_t(aotcu_ctx* c, const GemmParams& P, int grid, size_t smem) {
  static bool attr_set[64] = {};
  int dev = c->device;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    CU_TRY(cudaFuncSetAttribute(gemm_q8k_mma_kernel<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    attr_set[dev] = true;
  }
  return launch(c, gemm_q8k_mma_kernel<PAIR>, dim3(grid), dim3(GEMM_WARPS * 32), smem, P);
}

// Q4_K / Q5_K matrices: the tcgen05 kernel (gemm_tc.cuh). A gate/up pair runs as two
// matrices of one launch, the SiLU gate as a separate element-wise pass (the same two
// operations in the same order as the fused epilogue).
// Set only by aotcu_block_sums_of around its one launch: where the product kernels leave
// their integer block sums.
static int32_t* g_dbg_sumi = nullptr;
static int32_t* g_dbg_summ = nullptr;

static bool g_use_tc = []() {
  const char* e = getenv("AOTCU_TC_GEMM");  // "0": keep prompt chunks on the mma.sync tiles
  return !(e && e[0] == '0');
}();
static int launch_gemm_tc(aotcu_ctx* c, const GemvCall& call) {
  GemmTcParams P = {};
  int tiles = 0;
  for (int s = 0; s < call.nseg; s++) {
    P.seg[s] = call.seg[s];
    P.tiles_before[s] = tiles;
    tiles += (call.seg[s].rows + TC_ROWS - 1) / TC_ROWS;
  }
  for (int s = call.nseg; s < 4; s++) P.tiles_before[s] = tiles;
  P.nseg = call.nseg;
  P.cols = (int)call.cols;
  P.m = (int)call.m;
  P.epilogue = call.epilogue == EPI_ACCUM ? EPI_ACCUM : EPI_STORE;
  P.x = reinterpret_cast<const uint8_t*>(call.x);
  P.x_image = call.x_mode == 1;
  P.n_tiles = tiles;
  P.err = c->d_err;
  P.dbg_sumi = g_dbg_sumi;
  P.dbg_summ = g_dbg_summ;
  bool prep = true;
  for (int s = 0; s < call.nseg; s++) {
    P.prep[s] = call.prep[s];
    prep = prep && call.prep[s] != nullptr;
  }
  static bool attr_set[64] = {};
  if (c->device >= 0 && c->device < 64 && !attr_set[c->device]) {
    CU_TRY(cudaFuncSetAttribute(gemm_k4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
    CU_TRY(cudaFuncSetAttribute(gemm_k4_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM_BYTES));
    attr_set[c->device] = true;
  }
  const int grid = tiles < c->n_sm ? tiles : c->n_sm;
  if (prep) {
    if (int rc = launch(c, gemm_k4_prep_kernel, dim3(grid), dim3(TP_THREADS), (size_t)TP_SMEM_BYTES, P)) return rc;
  } else {
    if (int rc = launch(c, gemm_k4_tc_kernel, dim3(grid), dim3(TC_THREADS), (size_t)TC_SMEM_BYTES, P)) return rc;
  }
  if (call.pair && call.epilogue == EPI_SILU_MUL) {
    const size_t n = call.m * (size_t)call.seg[0].rows;
    return launch(c, silu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, call.seg[0].out, (const float*)call.seg[1].out, n);
  }
  return 0;
}

// 0: choose by size (the tcgen05 kernel works on tiles of 128 rows, one CTA each: it wins
// once a launch has enough tiles to occupy the GPU, measured 32 us against 45 us for the
// gate/up pair of the TinyLlama shape, and loses on 16..20 tiles); 1: always; -1: never.
static int g_tc_force = 0;
// Does a prompt chunk go to a tcgen05 kernel? Q4_K / Q5_K only, and (128-row tiles, one CTA
// each) only with enough tiles to occupy the GPU.
static bool takes_tc(const aotcu_ctx* c, const GemvCall& call) {
  bool k4 = g_use_tc && g_tc_force >= 0;
  int tc_tiles = 0;
  for (int s = 0; s < call.nseg; s++) {
    k4 = k4 && (call.seg[s].kind == Q4_K || call.seg[s].kind == Q5_K);
    tc_tiles += (call.seg[s].rows + TC_ROWS - 1) / TC_ROWS;
  }
  return k4 && (g_tc_force > 0 || tc_tiles >= c->n_sm / 2);
}
static int launch_gemm(aotcu_ctx* c, const GemvCall& call) {
  if (takes_tc(c, call)) return launch_gemm_tc(c, call);
  GemmParams P = {};
  int tiles = 0;
  for (int s = 0; s < call.nseg; s++) {
    P.seg[s] = call.seg[s];
    P.tiles_before[s] = tiles;
    if (!call.pair || s == 0) tiles += (call.seg[s].rows + 15) / 16;
  }
  if (call.pair) P.tiles_before[1] = 0;
  P.nseg = call.nseg;
  P.pair = call.pair;
  P.cols = (int)call.cols;
  P.m = (int)call.m;
  P.epilogue = call.epilogue;
  P.x = reinterpret_cast<const uint8_t*>(call.x);
  P.x_image = call.x_mode == 1;
  P.n_tiles = tiles;
  P.n_groups = (P.m + GEMM_TOK - 1) / GEMM_TOK;
  const int nb = (int)(call.cols / 256), n_mat = call.pair ? 2 : 1;
  // The warps of a tile split its super-blocks four ways when there are enough of them.
  P.ks = nb >= 4 ? 4 : (nb >= 2 ? 2 : 1);
  const int tpc = GEMM_WARPS / P.ks;
  // Super-blocks staged at a time: all of them if images + terms fit, else as many as fit
  // beside a second resident CTA.
  const size_t per_block = (size_t)GEMM_TOK * XK_STRIDE + (size_t)tpc * n_mat * 32 * GEMM_NT * 4 * sizeof(float);
  const size_t budget = c->max_smem / 2 - 2048;
  int kc = nb;
  if ((size_t)kc * per_block > budget) kc = (int)(budget / per_block);
  ARG_CHECK(kc >= 1, "one super-block column does not fit in shared memory");
  kc = (kc / P.ks) * P.ks > 0 ? (kc / P.ks) * P.ks : kc;  // whole strides of the k-split
  P.kc = kc;
  const size_t smem = (size_t)kc * per_block;
  int ctas_per_group = (tiles + tpc - 1) / tpc;
  const int cap = (c->n_sm * 2) / P.n_groups;
  if (ctas_per_group > cap) ctas_per_group = cap < 1 ? 1 : cap;
  const int grid = ctas_per_group * P.n_groups;
  return call.pair ? launch_gemm_t<true>(c, P, grid, smem) : launch_gemm_t<false>(c, P, grid, smem);
}

// Fields of a MegaOp the kernels would otherwise derive with integer divisions.
static void megaop_derive(MegaOp& op) {
  const int mats = op.pair ? 2 : 1;
  op.nb = op.cols >> 8;
  op.tstride = op.nb | 1;
  int cap = WARP_TERMS_FLOATS / (op.tstride * mats);
  const int cap_max = op.pair ? 16 : 32;
  op.cap = cap > cap_max ? cap_max : (cap < 1 ? 1 : cap);
  op.n_tiles_lo = (op.cta_base + op.tile_rows - 1) / op.tile_rows;
  op.n_tiles_hi = (op.cta_base + 1 + op.tile_rows - 1) / op.tile_rows;
}

// One product on the ring producer/consumer kernel: a single activation row for K-quants,
// one or more rows for the Q8_0 family (as many at a time as their images fit in shared
// memory; the matrix is streamed once per such group).
constexpr size_t STREAM_STAGE_BYTES = 32768;
#ifndef AOT_WIDE_ROWS
#define AOT_WIDE_ROWS 1
#endif
static int g_wide_rows = AOT_WIDE_ROWS;  // rows per CTA from which the single-row kernel goes one lane per super-block (option "wide_rows")
static int launch_gemv_stream(aotcu_ctx* c, const GemvCall& call, size_t span) {
  StreamGemvParams P = {};
  MegaOp& op = P.op;
  size_t max_rb = 1;
  for (int s = 0; s < call.nseg; s++) {
    op.seg[s] = call.seg[s];
    op.row_bytes[s] = (uint32_t)kind_row_bytes(call.seg[s].kind, call.cols);
    max_rb = std::max(max_rb, (size_t)op.row_bytes[s]);
  }
  op.nseg = call.nseg;
  op.pair = call.pair;
  op.cols = (int)call.cols;
  op.span_rows = (int)span;
  op.rows_per_cta = (int)((span + c->n_sm - 1) / c->n_sm);
  {
    const int grid_ctas = span < (size_t)c->n_sm ? (int)span : c->n_sm;
    op.cta_base = (int)(span / grid_ctas);
    op.cta_rem = (int)(span % grid_ctas);
  }
  const int tr = (int)((STREAM_STAGE_BYTES - 192) / (max_rb * (call.pair ? 2 : 1)));
  op.tile_rows = tr < 1 ? 1 : (tr > TILE_MAX_UNITS ? TILE_MAX_UNITS : tr);
  op.epilogue = call.epilogue;
  op.ll = 0;
  op.dbg_sumi = g_dbg_sumi;
  op.dbg_summ = g_dbg_summ;
  megaop_derive(op);
  P.x_image = call.x_mode == 1;
  P.q80 = kind_act(call.seg[0].kind) == ACT_Q8_0;
  // One lane per super-block for everything but gate/up pairs. (By measurement, back-to-back
  // launches: 128256 x 4096 Q4_K 54 us against 96 us with four lanes per block, 5632 x 2048
  // 3.7 against 5.0 us, 2048 x 5632 4.7 against 5.5 us, and no shape where it loses.)
  P.wide = !P.q80 && !call.pair && call.epilogue != EPI_SILU_MUL && !g_dbg_sumi && op.rows_per_cta >= g_wide_rows ? 1 : 0;
  P.err = c->d_err;
  P.stage_bytes = (int)STREAM_STAGE_BYTES;
  const size_t x_image_bytes = P.q80 ? (call.cols / 32) * X0_STRIDE : (call.cols / 256) * XK_STRIDE;
  const size_t x_src_bytes = P.x_image ? x_image_bytes : (P.q80 ? (call.cols / 32) * 36 : (call.cols / 256) * 292);
  const size_t tail = MEGA_BAR_BYTES + 16 + MEGA_TERMS_BYTES;
  ARG_CHECK(x_image_bytes + tail + 2 * STREAM_STAGE_BYTES <= c->max_smem, "activation vector too long for shared memory");
  // activation rows per launch: leave room for at least three stages
  size_t group = (c->max_smem - tail - 3 * STREAM_STAGE_BYTES) / x_image_bytes;
  if (group < 1) group = 1;
  if (group > call.m) group = call.m;
  static bool attr_set[64] = {};
  if (c->device >= 0 && c->device < 64 && !attr_set[c->device]) {
    CU_TRY(cudaFuncSetAttribute(gemv_stream_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    CU_TRY(cudaFuncSetAttribute(gemv_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    CU_TRY(cudaFuncSetAttribute(gemv_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    attr_set[c->device] = true;
  }
  const int grid = span < (size_t)c->n_sm ? (int)span : c->n_sm;
  for (size_t t0 = 0; t0 < call.m; t0 += group) {
    const size_t mg = std::min(group, call.m - t0);
    P.m = (int)mg;
    P.x = reinterpret_cast<const uint8_t*>(call.x) + t0 * x_src_bytes;
    for (int s = 0; s < call.nseg; s++) op.seg[s].out = call.seg[s].out + t0 * (size_t)call.seg[s].rows;
    const size_t fixed = mg * x_image_bytes + tail;
    int n_stages = (int)((c->max_smem - fixed) / STREAM_STAGE_BYTES);
    if (n_stages > 6) n_stages = 6;
    P.n_stages = n_stages;
    const size_t smem = (size_t)n_stages * STREAM_STAGE_BYTES + fixed;
    auto kernel = P.q80 ? gemv_stream_kernel<0> : (P.wide ? gemv_stream_kernel<1> : gemv_stream_kernel<2>);
    if (int rc = launch(c, kernel, dim3(grid), dim3(MEGA_THREADS), smem, P)) return rc;
  }
  return 0;
}

// Q4_0 / Q5_0 / Q8_0 products on the chunk-streaming kernel (q80stream.cuh): matrices of one
// kind, up to Q80S_MAX_TOK activation rows per launch (fewer when their images leave no room
// for three ring stages). Returns 1 when the call does not fit this kernel.
static int g_q80_chunks = 1;         // 0: keep Q8_0-family products on the whole-row kernels (option "q80_chunks")
static int g_q80_rows_per_lane = 0;  // 0: by shape; 1 / 2: forced (option "q80_rows_per_lane")
template <int KIND, int NR, int NT>
static int launch_q80_stream_t(aotcu_ctx* c, const Q80StreamParams& P, int grid, size_t smem) {
  static bool attr_set[64] = {};
  if (c->device >= 0 && c->device < 64 && !attr_set[c->device]) {
    CU_TRY(cudaFuncSetAttribute(q80_stream_kernel<KIND, NR, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    attr_set[c->device] = true;
  }
  return launch(c, q80_stream_kernel<KIND, NR, NT>, dim3(grid), dim3(MEGA_THREADS), smem, P);
}
template <int KIND>
static int launch_q80_stream_k(aotcu_ctx* c, const Q80StreamParams& P, int nr, int nt, int grid, size_t smem) {
  if (nt == 16) return launch_q80_stream_t<KIND, 2, 16>(c, P, grid, smem);
  if (nt == 8) return nr == 2 ? launch_q80_stream_t<KIND, 2, 8>(c, P, grid, smem) : launch_q80_stream_t<KIND, 1, 8>(c, P, grid, smem);
  return nr == 2 ? launch_q80_stream_t<KIND, 2, 1>(c, P, grid, smem) : launch_q80_stream_t<KIND, 1, 1>(c, P, grid, smem);
}
// 2-D tensor map over 32-bit elements: [dim1][dim0] with rows `stride_bytes` apart, box
// [box1][box0]. cuTensorMapEncodeTiled comes from the driver through the runtime (no link
// against libcuda). Returns false when the driver refuses the map.
static bool tensor_map_2d(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, size_t dim0, size_t dim1, size_t stride_bytes,
                          int box0, int box1) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return false;
  const cuuint64_t gdim[2] = {dim0, dim1}, gstride[1] = {stride_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1}, estride[2] = {1, 1};
  return encode(out, dtype, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// A weight matrix as rows of u32 words, box of four rows by one chunk.
static bool weight_tensor_map(CUtensorMap* out, const uint8_t* w, size_t rows, size_t row_bytes, int chunk_bytes) {
  return tensor_map_2d(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, w, row_bytes / 4, rows, row_bytes, chunk_bytes / 4, 4);
}

// Shape of a stage of the chunk-streaming kernels. One activation row: every consumer warp
// owns a quad, or two where a CTA has more quads than warps (and for pairs). Several: up to
// 16 rows per launch, as 16 per lane, or as two token groups of 8 on half of the warps each
// where a CTA has few quads.
struct ChunkShape {
  int nr, nt, qw, ts;
};
static ChunkShape chunk_shape(int quads_per_cta, bool pair, size_t m, int force_nr) {
  ChunkShape s = {1, 1, MEGA_CONSUMER_WARPS, 1};
  if (m == 1) {
    s.nr = pair || quads_per_cta > MEGA_CONSUMER_WARPS ? 2 : 1;
    if (force_nr && !pair) s.nr = force_nr;
    return s;
  }
  const int half = MEGA_CONSUMER_WARPS / 2;
  s.nr = pair || quads_per_cta > half ? 2 : 1;
  const int lane_quads = pair ? quads_per_cta : (quads_per_cta + s.nr - 1) / s.nr;  // quads (pair quads) a warp column must cover
  if (lane_quads <= half) {
    s.qw = half;
    s.ts = 2;
    s.nt = 8;
  } else {
    s.nr = 2;
    s.nt = 16;
  }
  return s;
}

static int launch_q80_stream(aotcu_ctx* c, const GemvCall& call, size_t span) {
  const int kind = call.seg[0].kind;
  const size_t row_bytes = kind_row_bytes(kind, call.cols);
  // what the tensor copies need: one kind, rows in fours, 16-byte aligned rows
  if (row_bytes % 16 || span % 4) return 1;
  for (int s = 0; s < call.nseg; s++)
    if (call.seg[s].kind != kind || call.seg[s].rows % 4 || ((uintptr_t)call.seg[s].w & 15)) return 1;
  Q80StreamParams P = {};
  for (int s = 0; s < call.nseg; s++) {
    P.seg[s] = call.seg[s];
    if (!weight_tensor_map(&P.map[s], call.seg[s].w, (size_t)call.seg[s].rows, row_bytes, q80s_chunk_bytes(kind))) return 1;
  }
  P.nseg = call.nseg;
  P.pair = call.pair;
  P.cols = (int)call.cols;
  P.epilogue = call.epilogue;
  P.x_image = call.x_mode == 1;
  P.err = c->d_err;
  const size_t quads = span / 4;
  const int grid = quads < (size_t)c->n_sm ? (int)quads : c->n_sm;
  P.quad_base = (int)(quads / grid);
  P.quad_rem = (int)(quads % grid);
  const size_t nb = call.cols / 32, x_image_bytes = nb * X0_STRIDE;
  const size_t tail = 128 + 16 + 128;
  const ChunkShape shape = chunk_shape(P.quad_base + (P.quad_rem ? 1 : 0), call.pair != 0, call.m, g_q80_rows_per_lane);
  int nr = shape.nr, nt = shape.nt, qw = shape.qw, ts = shape.ts;
  if (nt == 16 && call.m <= 8) nt = 8;  // fewer accumulators for a short batch
  const size_t quad_bytes = (size_t)4 * q80s_chunk_bytes(kind);
  P.qw = qw;
  P.ts = ts;
  if (call.m == 1) {
    const size_t stage = (size_t)qw * nr * quad_bytes, fixed = ((x_image_bytes + 127) & ~(size_t)127) + tail;
    if (c->max_smem < fixed + 2 * stage) return 1;
    int n_stages = (int)((c->max_smem - fixed) / stage);
    P.n_stages = n_stages > 8 ? 8 : n_stages;
    P.m = 1;
    P.x = call.x;
    const size_t smem = (size_t)P.n_stages * stage + fixed;
    if (kind == Q4_0) return launch_q80_stream_k<Q4_0>(c, P, nr, nt, grid, smem);
    if (kind == Q5_0) return launch_q80_stream_k<Q5_0>(c, P, nr, nt, grid, smem);
    return launch_q80_stream_k<Q8_0>(c, P, nr, nt, grid, smem);
  }
  // Several activation rows: their images stream with the stages (16 rows x 16 blocks per
  // stage), so they have to be images in global memory; reference-layout blocks are
  // converted into a buffer of the context first (grown here: not during a stream capture).
  const uint8_t* ximg = reinterpret_cast<const uint8_t*>(call.x);
  if (!P.x_image) {
    const size_t need = call.m * x_image_bytes;
    if (need > c->ximg_bytes) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      CU_TRY(cudaStreamIsCapturing(c->stream, &cs));
      if (cs != cudaStreamCaptureStatusNone) return 1;
      CU_TRY(cudaStreamSynchronize(c->stream));
      if (c->ximg) cudaFree(c->ximg);
      c->ximg = nullptr;
      c->ximg_bytes = 0;
      CU_TRY(cudaMalloc(&c->ximg, need));
      c->ximg_bytes = need;
    }
    const int n_blocks = (int)(call.m * nb);
    if (int rc = launch(c, q80_to_image_kernel, dim3(grid_for(c, (size_t)n_blocks * 9, 256)), dim3(256), 0,
                        reinterpret_cast<const uint8_t*>(call.x), c->ximg, n_blocks))
      return rc;
    ximg = c->ximg;
  }
  if ((uintptr_t)ximg & 15) return 1;
  const size_t stage = (size_t)qw * nr * quad_bytes + (size_t)Q80S_MAX_TOK * Q80S_CBLK * X0_STRIDE;
  if (c->max_smem < tail + 2 * stage) return 1;
  int n_stages = (int)((c->max_smem - tail) / stage);
  P.n_stages = n_stages > 8 ? 8 : n_stages;
  const size_t smem = (size_t)P.n_stages * stage + tail;
  const size_t group = (size_t)ts * nt;  // 16
  for (size_t t0 = 0; t0 < call.m; t0 += group) {
    const size_t mg = std::min(group, call.m - t0);
    P.m = (int)mg;
    if (!tensor_map_2d(&P.xmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, ximg + t0 * x_image_bytes, nb * (X0_STRIDE / 4), mg, x_image_bytes,
                       Q80S_CBLK * (X0_STRIDE / 4), Q80S_MAX_TOK))
      return t0 == 0 ? 1 : fail(AOTCU_ERR_CUDA, "tensor map of the activation images refused");
    for (int s = 0; s < call.nseg; s++) P.seg[s].out = call.seg[s].out + t0 * (size_t)call.seg[s].rows;
    int rc;
    if (kind == Q4_0) rc = launch_q80_stream_k<Q4_0>(c, P, nr, nt, grid, smem);
    else if (kind == Q5_0) rc = launch_q80_stream_k<Q5_0>(c, P, nr, nt, grid, smem);
    else rc = launch_q80_stream_k<Q8_0>(c, P, nr, nt, grid, smem);
    if (rc) return rc;
  }
  return 0;
}

// F16 / BF16 / F32 products on the chunk-streaming kernel (floatstream.cuh): matrices of one
// kind, columns in eights, rows in fours, 16-byte aligned rows and activations. Returns 1
// when the call does not fit.
template <int KIND, int NR, int NT>
static int launch_float_stream_t(aotcu_ctx* c, const FloatStreamParams& P, int grid, size_t smem) {
  static bool attr_set[64] = {};
  if (c->device >= 0 && c->device < 64 && !attr_set[c->device]) {
    CU_TRY(cudaFuncSetAttribute(float_stream_kernel<KIND, NR, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    attr_set[c->device] = true;
  }
  return launch(c, float_stream_kernel<KIND, NR, NT>, dim3(grid), dim3(MEGA_THREADS), smem, P);
}
template <int KIND>
static int launch_float_stream_k(aotcu_ctx* c, const FloatStreamParams& P, int nr, int nt, int grid, size_t smem) {
  if (nr == 4) return launch_float_stream_t<KIND, 4, 8>(c, P, grid, smem);
  if (nt == 16) return launch_float_stream_t<KIND, 2, 16>(c, P, grid, smem);
  if (nt == 8) return nr == 2 ? launch_float_stream_t<KIND, 2, 8>(c, P, grid, smem) : launch_float_stream_t<KIND, 1, 8>(c, P, grid, smem);
  return nr == 2 ? launch_float_stream_t<KIND, 2, 1>(c, P, grid, smem) : launch_float_stream_t<KIND, 1, 1>(c, P, grid, smem);
}
static int g_float_chunks = 1;  // 0: keep float-kind products on gemv_float_kernel (option "float_chunks")
static int g_float_rows4 = 1;   // several activation rows, many weight rows per CTA: four weight rows per lane (option "float_rows4")
static int launch_float_stream(aotcu_ctx* c, const GemvCall& call, size_t span) {
  const int kind = call.seg[0].kind;
  const size_t row_bytes = kind_row_bytes(kind, call.cols);
  if (call.cols % 8 || row_bytes % 16 || span % 4 || ((uintptr_t)call.x & 15)) return 1;
  for (int s = 0; s < call.nseg; s++)
    if (call.seg[s].kind != kind || call.seg[s].rows % 4 || ((uintptr_t)call.seg[s].w & 15)) return 1;
  const int cb = fs_chunk_bytes(call.m);
  FloatStreamParams P = {};
  for (int s = 0; s < call.nseg; s++) {
    P.seg[s] = call.seg[s];
    if (!weight_tensor_map(&P.map[s], call.seg[s].w, (size_t)call.seg[s].rows, row_bytes, cb)) return 1;
  }
  P.nseg = call.nseg;
  P.pair = call.pair;
  P.cols = (int)call.cols;
  P.epilogue = call.epilogue;
  P.err = c->d_err;
  const size_t quads = span / 4;
  const int grid = quads < (size_t)c->n_sm ? (int)quads : c->n_sm;
  P.quad_base = (int)(quads / grid);
  P.quad_rem = (int)(quads % grid);
  ChunkShape shape = chunk_shape(P.quad_base + (P.quad_rem ? 1 : 0), call.pair != 0, call.m, 0);
  if (shape.nt == 16 && !call.pair && g_float_rows4) {
    // 16 rows as two token groups of 8 with four weight rows per lane: 12 shared-memory loads
    // per 32 fused multiply-adds instead of 18 (the load/store pipe is what bounds this kernel)
    shape = ChunkShape{4, 8, MEGA_CONSUMER_WARPS / 2, 2};
  }
  if (shape.nt == 16 && call.m <= 8) shape = ChunkShape{2, 8, MEGA_CONSUMER_WARPS, 1};  // a short batch: one token group
  if (shape.nr == 4 && call.m <= 8) shape = ChunkShape{2, 8, MEGA_CONSUMER_WARPS, 1};
  P.qw = shape.qw;
  P.ts = shape.ts;
  const int chunk_cols = cb / (kind == F32 ? 4 : 2), xrows = call.m == 1 ? 1 : FS_MAX_TOK;
  const int x_copies = chunk_cols > 256 ? 2 : 1, xbox = chunk_cols / x_copies;  // a box row holds at most 256 elements
  const size_t stage = (size_t)shape.qw * shape.nr * 4 * cb + x_copies * (((size_t)xrows * xbox * 4 + 127) & ~(size_t)127);
  const size_t tail = 128 + 16 + 128;
  int n_stages = (int)((c->max_smem - tail) / stage);
  n_stages = n_stages > 8 ? 8 : n_stages;
  if (n_stages < 2) return 1;
  P.n_stages = n_stages;
  const size_t smem = (size_t)n_stages * stage + tail;
  const size_t group = (size_t)shape.ts * shape.nt;
  const float* x = reinterpret_cast<const float*>(call.x);
  for (size_t t0 = 0; t0 < call.m; t0 += group) {
    const size_t mg = std::min(group, call.m - t0);
    P.m = (int)mg;
    if (!tensor_map_2d(&P.xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, x + t0 * call.cols, call.cols, mg, call.cols * 4, xbox, xrows))
      return t0 == 0 ? 1 : fail(AOTCU_ERR_CUDA, "tensor map of the activation rows refused");
    for (int s = 0; s < call.nseg; s++) P.seg[s].out = call.seg[s].out + t0 * (size_t)call.seg[s].rows;
    int rc;
    if (kind == F16) rc = launch_float_stream_k<F16>(c, P, shape.nr, shape.nt, grid, smem);
    else if (kind == BF16) rc = launch_float_stream_k<BF16>(c, P, shape.nr, shape.nt, grid, smem);
    else rc = launch_float_stream_k<F32>(c, P, shape.nr, shape.nt, grid, smem);
    if (rc) return rc;
  }
  return 0;
}

// K-quant products of a short batch of activation rows (2..7, and up to a few dozen on small
// matrices: see launch_gemv): gemv_stream_kernel<3>, one lane per super-block, grid = (row
// ranges) x (groups of activation rows). Returns 1 when the call does not fit.
static int g_wide_multi = 1;  // option "wide_multi": 0 keeps these launches on gemm_q8k_mma_kernel / the per-row loop
static int g_wide_multi_work = 57344;  // option "wide_multi_work": weight rows x activation rows up to which 8..64 rows take it
static int launch_gemv_stream_multi(aotcu_ctx* c, const GemvCall& call, size_t span) {
  if (call.pair || g_dbg_sumi || call.cols % 256) return 1;
  StreamGemvParams P = {};
  MegaOp& op = P.op;
  size_t max_rb = 1;
  for (int s = 0; s < call.nseg; s++) {
    op.seg[s] = call.seg[s];
    op.row_bytes[s] = (uint32_t)kind_row_bytes(call.seg[s].kind, call.cols);
    max_rb = std::max(max_rb, (size_t)op.row_bytes[s]);
  }
  if (2 * max_rb + 192 > STREAM_STAGE_BYTES) return 1;
  const size_t nb = call.cols / 256, x_image_bytes = nb * XK_STRIDE;
  const size_t tail = MEGA_BAR_BYTES + 16 + MEGA_TERMS_BYTES;
  if (c->max_smem < tail + 3 * STREAM_STAGE_BYTES + x_image_bytes) return 1;
  // activation rows per CTA: up to 16, fewer when their images leave no room for three stages;
  // then as many row ranges as give every SM a CTA
  size_t tg = std::min<size_t>(16, (c->max_smem - tail - 3 * STREAM_STAGE_BYTES) / x_image_bytes);
  tg = std::min(tg, call.m);
  const int n_tg = (int)((call.m + tg - 1) / tg);
  tg = (call.m + n_tg - 1) / n_tg;  // even groups
  int n_ranges = std::max(1, c->n_sm / n_tg);
  if ((size_t)n_ranges > span) n_ranges = (int)span;
  op.nseg = call.nseg;
  op.pair = 0;
  op.cols = (int)call.cols;
  op.span_rows = (int)span;
  op.rows_per_cta = (int)((span + n_ranges - 1) / n_ranges);
  op.cta_base = (int)(span / n_ranges);
  op.cta_rem = (int)(span % n_ranges);
  const int tr = (int)((STREAM_STAGE_BYTES - 192) / max_rb);
  op.tile_rows = tr < 1 ? 1 : (tr > TILE_MAX_UNITS ? TILE_MAX_UNITS : tr);
  op.epilogue = call.epilogue;
  op.ll = 0;
  megaop_derive(op);
  P.x = call.x;
  P.x_image = call.x_mode == 1;
  P.q80 = 0;
  P.wide = 1;
  P.m = (int)call.m;
  P.tg = (int)tg;
  P.err = c->d_err;
  P.stage_bytes = (int)STREAM_STAGE_BYTES;
  const size_t fixed = tg * x_image_bytes + tail;
  int n_stages = (int)((c->max_smem - fixed) / STREAM_STAGE_BYTES);
  P.n_stages = n_stages > 6 ? 6 : n_stages;
  const size_t smem = (size_t)P.n_stages * STREAM_STAGE_BYTES + fixed;
  static bool attr_set[64] = {};
  if (c->device >= 0 && c->device < 64 && !attr_set[c->device]) {
    CU_TRY(cudaFuncSetAttribute(gemv_stream_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
    attr_set[c->device] = true;
  }
  return launch(c, gemv_stream_kernel<3>, dim3(n_ranges, n_tg), dim3(MEGA_THREADS), smem, P);
}

static int launch_gemv(aotcu_ctx* c, const GemvCall& call) {
  ARG_CHECK(call.nseg >= 1 && call.nseg <= 3, "1..3 matrices per launch");
  const int act = kind_act(call.seg[0].kind);
  size_t span = 0, max_rb = 0;
  for (int s = 0; s < call.nseg; s++) {
    const GemvSeg& sg = call.seg[s];
    ARG_CHECK(sg.kind >= 0 && sg.kind < N_KINDS, "unknown weight kind %d", sg.kind);
    ARG_CHECK(kind_act(sg.kind) == act, "matrices of one launch must share the activation format");
    ARG_CHECK(sg.w && sg.out, "null weight or output pointer");
    ARG_CHECK(sg.rows > 0, "rows must be positive");
    if (int rc = check_weight_alignment(sg.kind, sg.w)) return rc;
    size_t rb = kind_row_bytes(sg.kind, call.cols);
    max_rb = rb > max_rb ? rb : max_rb;
    span += (size_t)sg.rows;
  }
  ARG_CHECK(call.cols > 0 && call.cols % (size_t)kind_block(call.seg[0].kind) == 0,
            "cols (%zu) must be a positive multiple of the block size", call.cols);
  ARG_CHECK(call.x, "null activation pointer");
  ARG_CHECK(call.m >= 1, "m must be at least 1");
  if (call.pair) {
    ARG_CHECK(call.nseg == 2 && call.seg[0].rows == call.seg[1].rows, "pair mode needs two matrices of equal rows");
    span = (size_t)call.seg[0].rows;
  }
  ARG_CHECK(span < (1u << 30) && call.cols < (1u << 24), "matrix too large");

  GemvParams P = {};
  for (int s = 0; s < call.nseg; s++) P.seg[s] = call.seg[s];
  P.nseg = call.nseg;
  P.pair = call.pair;
  P.cols = (int)call.cols;
  P.span_rows = (int)span;
  P.x = call.x;
  P.x_image = call.x_mode == 1;
  P.m = (int)call.m;
  P.epilogue = call.epilogue;
  P.err = c->d_err;

  if (act == ACT_F32) {
    ARG_CHECK(((uintptr_t)call.x % 4) == 0, "activations must be 4-byte aligned");
    if (g_float_chunks) {
      const int rc = launch_float_stream(c, call, span);
      if (rc <= 0) return rc;  // 1: a shape the tensor copies do not take, the plain kernel does
    }
    int rows_per_block = 32;
    int grid = (int)((span + rows_per_block - 1) / rows_per_block);
    int cap = c->n_sm * 8;
    grid = grid > cap ? cap : grid;
    return launch(c, gemv_float_kernel, dim3(grid), dim3(256), 0, P);
  }
  ARG_CHECK(((uintptr_t)call.x % (P.x_image ? 16 : 4)) == 0, "activation blocks are misaligned");

  // Prompt chunks of K-quant matrices go to the tensor-core kernel, single rows to the
  // streaming kernel (whole rows per warp, no barrier per tile).
  // Short batches of K-quant products: one lane per super-block against every activation row
  // (time grows with rows x batch: 2048 x 2048 8.5 us at 8 rows, 17 us at 32), where the
  // tile kernels' time hardly depends on the batch (14-17 us). Measured break-even: about
  // 57 K (weight rows x activation rows); below 8 rows the alternative is a loop over rows.
  if (act == ACT_Q8_K && call.m >= 2 && call.m <= (size_t)GEMM_MAX_M && g_wide_multi &&
      (call.m < 8 || (!takes_tc(c, call) && call.m * span <= (size_t)g_wide_multi_work))) {
    const int rc = launch_gemv_stream_multi(c, call, span);
    if (rc <= 0) return rc;  // 1: a pair or a very long row, the tile kernels take it
  }
  if (act == ACT_Q8_K && call.m >= 8 && call.m <= (size_t)GEMM_MAX_M) return launch_gemm(c, call);
  if (act == ACT_Q8_0 && g_q80_chunks) {
    const int rc = launch_q80_stream(c, call, span);
    if (rc <= 0) return rc;  // 1: mixed kinds or a very long activation row, the whole-row kernels take it
  }
  if ((call.m == 1 || act == ACT_Q8_0) && 2 * max_rb + 192 <= STREAM_STAGE_BYTES) return launch_gemv_stream(c, call, span);

  const int mult = call.pair ? 2 : 1;
  int grid = c->n_sm;
  if (span < (size_t)grid * 4) grid = (int)((span + 3) / 4);
  int rows_per_cta = (int)((span + grid - 1) / grid);
  grid = (int)((span + rows_per_cta - 1) / rows_per_cta);
  const size_t STAGE_MAX = 48 * 1024;
  int tile_rows = (int)(STAGE_MAX / (max_rb * mult));
  if (tile_rows > GEMV_TRP / mult) tile_rows = GEMV_TRP / mult;
  if (tile_rows > rows_per_cta) tile_rows = rows_per_cta;
  if (tile_rows < 1) tile_rows = 1;
  size_t stage_bytes = (((size_t)tile_rows * mult * max_rb + 15) & ~(size_t)15) + 256;
  size_t fixed;
  if (act == ACT_Q8_K) {
    size_t nb = call.cols / 256;
    fixed = nb * XK_STRIDE + 2 * nb * GEMV_TRP * sizeof(float) + 8 * sizeof(uint64_t);
  } else {
    size_t nb = call.cols / 32;
    fixed = ((nb * X0_STRIDE + 15) & ~(size_t)15) + 2 * GEMV_TRP * sizeof(float) + 8 * sizeof(uint64_t);
  }
  ARG_CHECK(fixed + stage_bytes <= c->max_smem, "a single row tile (%zu bytes) does not fit in shared memory",
            fixed + stage_bytes);
  int n_tiles = (rows_per_cta + tile_rows - 1) / tile_rows;
  int n_stages = (int)((c->max_smem - fixed) / stage_bytes);
  if (n_stages > n_tiles) n_stages = n_tiles;
  if (n_stages > 8) n_stages = 8;
  P.rows_per_cta = rows_per_cta;
  P.tile_rows = tile_rows;
  P.stage_bytes = (int)stage_bytes;
  P.n_stages = n_stages;
  size_t smem = (size_t)n_stages * stage_bytes + fixed;
  if (act == ACT_Q8_K) return launch(c, gemv_q8k_kernel, dim3(grid), dim3(GEMV_THREADS), smem, P);
  return launch(c, gemv_q80_kernel, dim3(grid), dim3(GEMV_THREADS), smem, P);
}

// ---- parity export: integer block sums -------------------------------------------------------
__global__ void block_sums_kernel(int kind, const uint8_t* w, const uint8_t* x, int rows, int nb, int32_t* sumi,
                                  int32_t* summ) {
  pdl_launch_dependents();
  pdl_wait();  // a launch with programmatic stream serialization must not run ahead of its predecessor
  // One thread per (row, block), straight from global memory with byte reads; this
  // is a checker for the integer arithmetic, not a fast path.
  for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < (size_t)rows * nb;
       it += (size_t)gridDim.x * blockDim.x) {
    const int b = (int)(it % nb);
    const uint8_t* wb = w + it * kind_size(kind);
    auto w32 = [&](const uint8_t* p, int i) -> uint32_t {
      return (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) |
             ((uint32_t)p[4 * i + 3] << 24);
    };
    if (kind_act(kind) == ACT_Q8_K) {
      const BlockQ8_K* y = reinterpret_cast<const BlockQ8_K*>(x) + b;
      auto yw = [&](int i) -> uint32_t { return w32(reinterpret_cast<const uint8_t*>(y->qs), i); };
      if (kind == Q6_K) {
        sumi[it] = q6k_block_sum([&](int i) { return w32(wb, i); }, yw, y->bsums);
      } else {
        const bool q5 = kind == Q5_K;
        K4Scales s = k4_unpack(w32(wb + 4, 0), w32(wb + 4, 1), w32(wb + 4, 2));
        const uint8_t* qs = wb + (q5 ? 48 : 16);
        const uint8_t* qh = wb + 16;
        int si, sm;
        if (q5)
          k4_block_sums<true>(s, [&](int i) { return w32(qs, i); }, [&](int i) { return w32(qh, i); }, yw, y->bsums, si, sm);
        else
          k4_block_sums<false>(s, [&](int i) { return w32(qs, i); }, [&](int i) { return w32(qh, i); }, yw, y->bsums, si, sm);
        sumi[it] = si;
        if (summ) summ[it] = sm;
      }
    } else {
      const BlockQ8_0* y = reinterpret_cast<const BlockQ8_0*>(x) + b;
      int s = 0;
      for (int k = 0; k < 8; k++) {
        uint32_t y4 = w32(reinterpret_cast<const uint8_t*>(y->qs), k);
        if (kind == Q8_0) s += q8_0_lane(w32(wb + 2, k), y4);
        else if (kind == Q4_0) s += q4_0_lane(w32(wb + 2, k & 3), k, y4);
        else s += q5_0_lane(w32(wb + 6, k & 3), w32(wb + 2, 0), k, y4);
      }
      sumi[it] = s;
    }
  }
}

// ---- device State + model (the `Gpu` of metal.rs) ------------------------------------------------
// ---- tensor parallel exchange (NCCL, loaded at run time) ----------------------------------
// Row-sharded models sum the partial outputs of attn_output and ffn_down over the ranks.
// NCCL is not linked: the host names the shared library (the one its process already
// uses), and the five entry points needed are looked up with dlsym.
struct TpState {
  void* lib = nullptr;
  void* comm = nullptr;   // ncclComm_t
  int rank = 0, world = 1;
  // ncclResult_t (0 = success) f(...)
  int (*get_unique_id)(void*) = nullptr;
  int (*comm_init_rank)(void**, int, /* ncclUniqueId by value: 128 bytes */ struct NcclId, int) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*all_gather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*comm_destroy)(void*) = nullptr;
  const char* (*get_error_string)(int) = nullptr;
};
struct NcclId {
  char bytes[128];
};
constexpr int NCCL_FLOAT32 = 7, NCCL_SUM = 0;  // ncclFloat32, ncclSum of nccl.h

static int tp_load(TpState* t, const char* path) {
  t->lib = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!t->lib) return fail(AOTCU_ERR_UNSUPPORTED, "cannot load NCCL (%s): %s", path ? path : "libnccl.so.2", dlerror());
  t->get_unique_id = reinterpret_cast<decltype(t->get_unique_id)>(dlsym(t->lib, "ncclGetUniqueId"));
  t->comm_init_rank = reinterpret_cast<decltype(t->comm_init_rank)>(dlsym(t->lib, "ncclCommInitRank"));
  t->all_reduce = reinterpret_cast<decltype(t->all_reduce)>(dlsym(t->lib, "ncclAllReduce"));
  t->all_gather = reinterpret_cast<decltype(t->all_gather)>(dlsym(t->lib, "ncclAllGather"));
  t->comm_destroy = reinterpret_cast<decltype(t->comm_destroy)>(dlsym(t->lib, "ncclCommDestroy"));
  t->get_error_string = reinterpret_cast<decltype(t->get_error_string)>(dlsym(t->lib, "ncclGetErrorString"));
  if (!t->get_unique_id || !t->comm_init_rank || !t->all_reduce || !t->all_gather || !t->comm_destroy || !t->get_error_string)
    return fail(AOTCU_ERR_UNSUPPORTED, "the NCCL library lacks a required entry point");
  return 0;
}

struct aotcu_gpu {
  aotcu_ctx* c = nullptr;
  aotcu_model_head head;
  std::vector<aotcu_layer> layers;
  size_t n_ctx = 0, max_batch = 1;
  uint8_t* d_weights = nullptr;
  size_t weights_len = 0;
  float* bufs[AOTCU_N_BUFS] = {};
  size_t buf_len[AOTCU_N_BUFS] = {};
  float* rope_table = nullptr;        // n_ctx x rot_dim
  float* rope_table_local = nullptr;  // swa layers
  uint8_t* aqk = nullptr;             // Q8_K block images, max_batch rows of max(dim, q_dim, hidden)
  uint8_t* aq0 = nullptr;             // Q8_0 block images
  float* attn_scratch = nullptr;      // scores for contexts that do not fit shared memory
  int* d_step = nullptr;              // {token, pos, n_generated}
  int* d_tokens = nullptr;            // prompt batch ids
  int* d_history = nullptr;           // generated ids
  int* d_out_token = nullptr;
  int* h_pinned = nullptr;            // staging for step / tokens; [4]: the device error word read back with a step
  float* h_logits = nullptr;          // pinned copy of the logits of the last aotcu_forward(.., want_logits), fetched with the step's one sync
  bool h_logits_fresh = false;
  size_t history_cap = 0;
  bool need_q8k = false, need_q80 = false;
  // What the quantized-activation buffers currently hold.
  struct QSrc {
    const float* ptr = nullptr;
    size_t n = 0, m = 0;
    bool q8k = false, q80 = false;
  } qsrc;
  bool use_graph = true;
  // Persistent one-kernel decode step (mega.cuh), when the model qualifies.
  bool mega_ok = false, use_mega = true;
  TpState* tp = nullptr;              // set by aotcu_tp_attach: this Gpu holds one shard of the model
  LLWord* tp_inbox = nullptr;         // partial rows from every rank (aotcu_tp_inbox_handle)
  void* tp_peer_map[8] = {};          // peers' inboxes mapped into this process
  // Vocabulary-sharded output head: this rank's `output` holds rows [head_row0, head_row0 +
  // rows) of the vocabulary; its logits sit at the front of the logits buffer and the whole
  // vector is gathered (NCCL) only when the host asks for it.
  bool head_sharded = false;
  size_t head_row0 = 0;
  float* tp_logits_full = nullptr;
  StepLayer* d_step_layers = nullptr;
  unsigned* d_grid_bar = nullptr;     // [0] barrier arrivals of one launch, [1] launch count
  void* d_ll = nullptr;               // tagged activation vectors of the one-kernel step
  StepParams step_params = {};
  size_t mega_smem = 0;
  // Captured decode steps: [want_logits + 2 * long-context variant of the one-kernel step]
  cudaGraphExec_t decode_graph[4] = {};
  cudaGraphExec_t gen_graph[2] = {};            // [long-context variant]
  uint64_t decode_graph_kernels[4] = {};        // kernel nodes per replay
  uint64_t gen_graph_kernels[2] = {};
  int split_now = 0;                            // the step being enqueued shares heads between CTAs (mega_split)
  // Prepared tensor-core operands of the Q4_K / Q5_K layer matrices (gemm_tc.cuh), keyed by
  // the tensor's offset; built before the first prompt chunk of 8 tokens or more.
  std::unordered_map<uint64_t, uint8_t*> prep;
  int prep_state = 0;                           // 0 not built yet, 1 built, -1 off (option, memory, or nothing to prepare)
  int smem_scores = 0;
};

static size_t xb_width(const aotcu_dims& d) {
  size_t qd = (size_t)d.n_head * d.head_dim;
  return (size_t)d.dim > qd ? (size_t)d.dim : qd;
}

static int tensor_check(const aotcu_gpu* g, const aotcu_tensor& t, const char* name) {
  ARG_CHECK(t.kind >= 0 && t.kind < N_KINDS, "tensor %s: unknown kind %d", name, t.kind);
  ARG_CHECK(t.cols % (uint64_t)kind_block(t.kind) == 0, "tensor %s: cols not a multiple of the block size", name);
  uint64_t need = t.rows * kind_row_bytes(t.kind, t.cols);
  ARG_CHECK(t.off + need <= g->weights_len, "tensor %s lies outside the weights (%llu + %llu > %zu)", name,
            (unsigned long long)t.off, (unsigned long long)need, g->weights_len);
  ARG_CHECK(t.off % 32 == 0, "tensor %s: offset %llu is not 32-byte aligned", name, (unsigned long long)t.off);
  return 0;
}

static const uint8_t* wptr(const aotcu_gpu* g, const aotcu_tensor& t) { return g->d_weights + t.off; }
static const float* wf32(const aotcu_gpu* g, const aotcu_tensor& t) { return reinterpret_cast<const float*>(g->d_weights + t.off); }

static void note_write(aotcu_gpu* g, const float* p) {
  // A write to the buffer whose quantized image is cached invalidates the image.
  if (g->qsrc.ptr && p == g->qsrc.ptr) g->qsrc = aotcu_gpu::QSrc();
  if (p == g->bufs[AOTCU_BUF_LOGITS]) g->h_logits_fresh = false;  // the host copy made by aotcu_forward is stale
}

// Make sure the block images of `src` (m rows of n floats) exist for `act`.
static int ensure_quantized(aotcu_gpu* g, const float* src, size_t n, size_t m, int act) {
  if (act == ACT_F32) return 0;
  aotcu_ctx* c = g->c;
  bool same = g->qsrc.ptr == src && g->qsrc.n == n && g->qsrc.m == m;
  if (!same) {
    g->qsrc = aotcu_gpu::QSrc();
    g->qsrc.ptr = src;
    g->qsrc.n = n;
    g->qsrc.m = m;
  }
  if (act == ACT_Q8_K && !g->qsrc.q8k) {
    ARG_CHECK(n % 256 == 0, "row length %zu is not a multiple of 256", n);
    int nblk = (int)(n * m / 256);
    if (int rc = launch(c, quantize_q8k_kernel, dim3(grid_for(c, nblk, 8)), dim3(256), 0, src, g->aqk, nblk, 1)) return rc;
    g->qsrc.q8k = true;
  }
  if (act == ACT_Q8_0 && !g->qsrc.q80) {
    ARG_CHECK(n % 32 == 0, "row length %zu is not a multiple of 32", n);
    int nblk = (int)(n * m / 32);
    if (int rc = launch(c, quantize_q80_kernel, dim3(grid_for(c, nblk, 8)), dim3(256), 0, src, g->aq0, nblk, 1)) return rc;
    g->qsrc.q80 = true;
  }
  return 0;
}

static const void* act_images(const aotcu_gpu* g, int act, const float* src) {
  return act == ACT_Q8_K ? (const void*)g->aqk : act == ACT_Q8_0 ? (const void*)g->aq0 : (const void*)src;
}

static int gpu_rmsnorm(aotcu_gpu* g, float* dst, size_t dst_stride, const float* src, size_t src_stride, const float* w,
                       size_t n, size_t m, float eps, int accumulate, bool quantize) {
  aotcu_ctx* c = g->c;
  RmsnormParams P = {};
  P.x = src;
  P.w = w;
  P.out = dst;
  P.n = (int)n;
  P.x_stride = (int)src_stride;
  P.out_stride = (int)dst_stride;
  P.eps = eps;
  P.accumulate = accumulate;
  bool q = quantize && !accumulate && dst_stride == n;
  P.q8k_out = (q && g->need_q8k && n % 256 == 0) ? g->aqk : nullptr;
  P.q80_out = (q && g->need_q80 && n % 32 == 0) ? g->aq0 : nullptr;
  size_t smem = (2 * n + 4) * sizeof(float);
  ARG_CHECK(smem <= c->max_smem, "rmsnorm row of %zu floats does not fit shared memory", n);
  note_write(g, dst);
  if (int rc = launch(c, rmsnorm_kernel, dim3((unsigned)m), dim3(512), smem, P)) return rc;
  if (q) {
    g->qsrc = aotcu_gpu::QSrc();
    g->qsrc.ptr = dst;
    g->qsrc.n = n;
    g->qsrc.m = m;
    g->qsrc.q8k = P.q8k_out != nullptr;
    g->qsrc.q80 = P.q80_out != nullptr;
  }
  return 0;
}

// dst (+)= W . src for m rows (Gpu::mv / Gpu::matmul).
// Prepared operands of tensor t for a batch of m rows, or null.
static const uint8_t* prep_of(const aotcu_gpu* g, const aotcu_tensor& t, size_t m) {
  if (g->prep_state != 1 || m < 8 || m > (size_t)TC_TOK) return nullptr;
  auto it = g->prep.find(t.off);
  return it == g->prep.end() ? nullptr : it->second;
}

// Builds the prepared operands of every Q4_K / Q5_K layer matrix once (3.7 x their bytes):
// only when they take at most half of the memory that is free, so that a model sized for
// the device keeps fitting; otherwise prompt chunks keep unpacking weights per launch.
static int ensure_prepared(aotcu_gpu* g) {
  if (g->prep_state != 0) return 0;
  g->prep_state = -1;
  if (!g_use_tc || g_tc_force < 0) return 0;
  std::vector<const aotcu_tensor*> ts;
  size_t total = 0;
  // only matrices whose launches reach the tensor-core kernel (launch_gemm: at least n_sm / 2
  // tiles of 128 rows per launch): q/k/v go out as one launch, gate/up as one, wo and down alone
  auto k4 = [](const aotcu_tensor* t) { return (t->kind == Q4_K || t->kind == Q5_K) && t->cols % 256 == 0; };
  auto tiles = [](const aotcu_tensor* t) { return (int)((t->rows + TC_ROWS - 1) / TC_ROWS); };
  const int need = g_tc_force > 0 ? 1 : g->c->n_sm / 2;
  auto want = [&](std::initializer_list<const aotcu_tensor*> group) {
    int n = 0;
    for (auto t : group) {
      if (!k4(t) || t->cols != (*group.begin())->cols) return;
      n += tiles(t);
    }
    if (n < need) return;
    for (auto t : group)
      if (!g->prep.count(t->off) && std::find(ts.begin(), ts.end(), t) == ts.end()) {
        ts.push_back(t);
        total += tc_prep_bytes(t->rows, t->cols);
      }
  };
  for (const auto& l : g->layers) {
    want({&l.wq, &l.wk, &l.wv});
    want({&l.gate, &l.up});
    want({&l.wo});
    want({&l.down});
  }
  if (ts.empty()) return 0;
  size_t free_b = 0, total_b = 0;
  CU_TRY(cudaMemGetInfo(&free_b, &total_b));
  if (total > free_b / 2) return 0;
  for (auto t : ts) {
    if (g->prep.count(t->off)) continue;  // a tensor shared by two layers
    uint8_t* p = nullptr;
    CU_TRY(cudaMalloc(&p, tc_prep_bytes(t->rows, t->cols)));
    g->prep[t->off] = p;
    const unsigned blocks = (unsigned)(((t->rows + TC_ROWS - 1) / TC_ROWS) * (t->cols / 256));
    if (int rc = launch(g->c, k4_prepare_kernel, dim3(blocks), dim3(256), 0, wptr(g, *t), (int)t->kind, (int)t->rows, (int)t->cols, p))
      return rc;
  }
  g->prep_state = 1;
  return 0;
}

static int gpu_matmul(aotcu_gpu* g, float* dst, const aotcu_tensor& t, const float* src, size_t m, int accumulate) {
  int act = kind_act(t.kind);
  if (int rc = ensure_quantized(g, src, t.cols, m, act)) return rc;
  GemvCall call;
  call.seg[0] = GemvSeg{wptr(g, t), dst, (int)t.rows, t.kind};
  call.nseg = 1;
  call.cols = t.cols;
  call.x = act_images(g, act, src);
  call.x_mode = 1;
  call.m = m;
  call.epilogue = accumulate ? EPI_ACCUM : EPI_STORE;
  call.prep[0] = prep_of(g, t, m);
  note_write(g, dst);
  return launch_gemv(g->c, call);
}

static int gpu_mv3(aotcu_gpu* g, float* const dst[3], const aotcu_tensor* const t[3], const float* src, size_t m) {
  // One launch per activation format (the reference fuses only when all three kinds
  // are equal, emit.rs:256-272; mixed K-quants still share Q8_K activations here).
  bool done[3] = {false, false, false};
  for (int a = 0; a < 3; a++) {
    if (done[a]) continue;
    int act = kind_act(t[a]->kind);
    GemvCall call;
    call.nseg = 0;
    const bool prepared = prep_of(g, *t[a], m) != nullptr;
    for (int b = a; b < 3; b++) {
      // matrices with prepared tensor-core operands go together, the others together
      if (!done[b] && kind_act(t[b]->kind) == act && t[b]->cols == t[a]->cols && (prep_of(g, *t[b], m) != nullptr) == prepared) {
        call.prep[call.nseg] = prep_of(g, *t[b], m);
        call.seg[call.nseg++] = GemvSeg{wptr(g, *t[b]), dst[b], (int)t[b]->rows, t[b]->kind};
        done[b] = true;
        note_write(g, dst[b]);
      }
    }
    if (int rc = ensure_quantized(g, src, t[a]->cols, m, act)) return rc;
    call.cols = t[a]->cols;
    call.x = act_images(g, act, src);
    call.x_mode = 1;
    call.m = m;
    if (int rc = launch_gemv(g->c, call)) return rc;
  }
  return 0;
}

static int gpu_gate_up(aotcu_gpu* g, float* hb, float* hb2, const aotcu_tensor& gate, const aotcu_tensor& up,
                       const float* src, size_t m) {
  aotcu_ctx* c = g->c;
  const bool gelu = g->head.dims.gelu != 0;  // GeGLU (Gemma): h = gelu(gate) * up, emit.rs picks gelu_mul
  if (gate.kind == up.kind && gate.rows == up.rows && gate.cols == up.cols) {
    int act = kind_act(gate.kind);
    if (int rc = ensure_quantized(g, src, gate.cols, m, act)) return rc;
    GemvCall call;
    call.seg[0] = GemvSeg{wptr(g, gate), hb, (int)gate.rows, gate.kind};
    call.seg[1] = GemvSeg{wptr(g, up), hb2, (int)up.rows, up.kind};
    call.nseg = 2;
    call.pair = 1;
    call.cols = gate.cols;
    call.x = act_images(g, act, src);
    call.x_mode = 1;
    call.m = m;
    call.epilogue = gelu ? EPI_STORE : EPI_SILU_MUL;
    call.prep[0] = prep_of(g, gate, m);
    call.prep[1] = prep_of(g, up, m);
    note_write(g, hb);
    note_write(g, hb2);
    if (int rc = launch_gemv(c, call)) return rc;
    if (!gelu) return 0;
    const size_t n = m * gate.rows;
    return launch(c, gelu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, hb, (const float*)hb2, n);
  }
  if (int rc = gpu_matmul(g, hb, gate, src, m, 0)) return rc;
  if (int rc = gpu_matmul(g, hb2, up, src, m, 0)) return rc;
  size_t n = m * gate.rows;
  if (gelu) return launch(c, gelu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, hb, (const float*)hb2, n);
  return launch(c, silu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, hb, (const float*)hb2, n);
}

static int gpu_qk_post(aotcu_gpu* g, size_t li, const int* pos_ptr, size_t pos0, size_t m, bool batch) {
  const aotcu_dims& d = g->head.dims;
  const aotcu_layer& l = g->layers[li];
  size_t kvd = (size_t)d.n_kv_head * d.head_dim;
  QkPostParams P = {};
  P.q = g->bufs[batch ? AOTCU_BUF_BQ : AOTCU_BUF_Q];
  P.k = g->bufs[batch ? AOTCU_BUF_BK : AOTCU_BUF_K];
  P.v = g->bufs[batch ? AOTCU_BUF_BV : AOTCU_BUF_V];
  P.k_cache = g->bufs[AOTCU_BUF_KCACHE] + li * g->n_ctx * kvd;
  P.v_cache = g->bufs[AOTCU_BUF_VCACHE] + li * g->n_ctx * kvd;
  P.q_norm = d.qk_norm ? wf32(g, l.q_norm) : nullptr;
  P.k_norm = d.qk_norm ? wf32(g, l.k_norm) : nullptr;
  P.rope_table = l.local_attn ? g->rope_table_local : g->rope_table;
  P.pos_ptr = pos_ptr;
  P.pos0 = (int)pos0;
  P.n_head = d.n_head;
  P.n_kv_head = d.n_kv_head;
  P.head_dim = d.head_dim;
  P.rot_dim = d.rot_dim;
  P.neox = d.rope_neox;
  P.eps = d.eps;
  note_write(g, P.q);
  return launch(g->c, qk_post_kernel, dim3(d.n_head + d.n_kv_head, (unsigned)m), dim3(128), 0, P);
}

// Shared memory of the attention kernel with the scores of rows up to `max_len` positions
// kept on chip, and what a CTA may use.
// Shared memory of the attention kernel with the scores of rows up to `max_len` positions
// kept on chip, and what a CTA may use. A CTA has heads_per_cta x rows_per_cta warps, each
// with its exact-sum scratch, its query row and (when they fit) its scores.
static size_t attn_smem_budget(const aotcu_ctx* c) { return c->max_smem - 1024; }
struct AttnShape {
  int hpc, rpc, chunk;
  bool scores_in_smem;
  size_t smem;
};
static size_t attn_smem_of(int warps, int head_dim, int chunk, size_t score_floats) {
  return attn_ssc_bytes(warps) + ((size_t)warps * head_dim + (size_t)2 * chunk * (head_dim + 4) + (size_t)warps * score_floats) * sizeof(float);
}
// Warps per CTA and staging chunk for rows of up to `max_len` positions: scores stay in shared
// memory if any shape allows it (fewer rows per CTA rather than scores in global memory),
// and the larger chunk is taken when it still fits.
static AttnShape attn_shape(const aotcu_ctx* c, int n_head, int n_kv_head, int head_dim, size_t m, size_t max_len, bool want_smem_scores) {
  const int gqa = n_head / n_kv_head;
  AttnShape a;
  a.hpc = gqa < 8 ? gqa : 8;
  int rmax = ATTN_MAX_WARPS / a.hpc;
  if ((size_t)rmax > m) rmax = (int)m;
  if (rmax < 1) rmax = 1;
  max_len = (max_len + 3) & ~(size_t)3;
  const size_t budget = attn_smem_budget(c);
  if (want_smem_scores)
    for (int r = rmax; r >= 1; r--)
      for (int chunk : {ATTN_CHUNK_BIG, ATTN_CHUNK}) {
        const size_t need = attn_smem_of(a.hpc * r, head_dim, chunk, max_len);
        if (need <= budget) {
          a.rpc = r;
          a.chunk = chunk;
          a.scores_in_smem = true;
          a.smem = need;
          return a;
        }
      }
  a.rpc = rmax;
  a.chunk = ATTN_CHUNK;
  a.scores_in_smem = false;
  a.smem = attn_smem_of(a.hpc * rmax, head_dim, ATTN_CHUNK, 0);
  return a;
}
static size_t attn_smem_bytes(const aotcu_ctx* c, int n_head, int n_kv_head, int head_dim, size_t max_len, size_t m = 1) {
  const AttnShape a = attn_shape(c, n_head, n_kv_head, head_dim, m, max_len, true);
  return a.scores_in_smem ? a.smem : (size_t)-1;
}

static int launch_attention(aotcu_ctx* c, float* out, const float* q, const float* kc, const float* vc, float* scratch,
                            const int* pos_ptr, size_t pos0, size_t m, int n_head, int n_kv_head, int head_dim,
                            size_t n_ctx, size_t window, int smem_scores) {
  AttnParams P = {};
  P.out = out;
  P.q = q;
  P.k_cache = kc;
  P.v_cache = vc;
  P.scratch = scratch;
  P.pos_ptr = pos_ptr;
  P.pos0 = (int)pos0;
  P.n_head = n_head;
  P.n_kv_head = n_kv_head;
  P.head_dim = head_dim;
  P.ctx = (int)((n_ctx + 3) & ~(size_t)3);  // row stride of the score scratch, 16-byte aligned rows
  P.window = (int)window;
  P.scale = 1.0f / sqrtf((float)head_dim);
  ARG_CHECK(head_dim % 4 == 0 && head_dim <= 256, "head_dim must be a multiple of 4, at most 256");
  const int gqa = n_head / n_kv_head;
  // Scores in shared memory when the longest row of this call fits, else in `scratch`.
  size_t max_len = pos_ptr ? n_ctx : std::min(n_ctx, pos0 + m);
  max_len = (max_len + 3) & ~(size_t)3;
  const AttnShape a = attn_shape(c, n_head, n_kv_head, head_dim, m, max_len, smem_scores != 0);
  P.heads_per_cta = a.hpc;
  P.rows_per_cta = a.rpc;
  P.chunk = a.chunk;
  P.m = (int)m;
  const int splits = (gqa + P.heads_per_cta - 1) / P.heads_per_cta;
  const size_t warps = (size_t)P.heads_per_cta * P.rows_per_cta;
  const size_t smem = a.smem;
  if (a.scores_in_smem) {
    P.smem_scores = (int)max_len;
  } else {
    ARG_CHECK(scratch, "attention needs a score scratch buffer for this context length");
    P.smem_scores = 0;
  }
  const unsigned row_groups = (unsigned)((m + P.rows_per_cta - 1) / P.rows_per_cta);
  return launch(c, attention_kernel, dim3((unsigned)(n_kv_head * splits), row_groups), dim3((unsigned)warps * 32), smem, P);
}

static int gpu_attention(aotcu_gpu* g, float* out, const float* q, size_t li, const int* pos_ptr, size_t pos0, size_t m,
                         size_t window) {
  const aotcu_dims& d = g->head.dims;
  size_t kvd = (size_t)d.n_kv_head * d.head_dim;
  note_write(g, out);
  return launch_attention(g->c, out, q, g->bufs[AOTCU_BUF_KCACHE] + li * g->n_ctx * kvd,
                          g->bufs[AOTCU_BUF_VCACHE] + li * g->n_ctx * kvd, g->attn_scratch, pos_ptr, pos0, m, d.n_head,
                          d.n_kv_head, d.head_dim, g->n_ctx, window, g->smem_scores);
}

// ---- the generated forward pass, interpreted (emit.rs) -----------------------------------------------
// One transformer block for m tokens. `pos_ptr` (device) is used by decode steps so a
// captured graph can be replayed for any position; batches pass pos0 by value.
static int tp_all_reduce(aotcu_gpu* g, float* buf, size_t n) {
  TpState* t = g->tp;
  const int r = t->all_reduce(buf, buf, n, NCCL_FLOAT32, NCCL_SUM, t->comm, g->c->stream);
  if (r != 0) return fail(AOTCU_ERR_CUDA, "ncclAllReduce: %s", t->get_error_string(r));
  note_write(g, buf);
  return 0;
}

// Every rank's slice of the logits, in rank order, into tp_logits_full (collective).
static int tp_gather_logits(aotcu_gpu* g) {
  TpState* t = g->tp;
  const aotcu_tensor& out_t = g->head.output.present ? g->head.output : g->head.token_embd;
  const int r = t->all_gather(g->bufs[AOTCU_BUF_LOGITS], g->tp_logits_full, (size_t)out_t.rows, NCCL_FLOAT32, t->comm, g->c->stream);
  if (r != 0) return fail(AOTCU_ERR_CUDA, "ncclAllGather: %s", t->get_error_string(r));
  return 0;
}

static int gpu_add(aotcu_gpu* g, float* x, const float* y, size_t n) {
  note_write(g, x);
  return launch(g->c, add_inplace_kernel, dim3(grid_for(g->c, n, 256)), dim3(256), 0, x, y, n);
}

static int layer_forward(aotcu_gpu* g, size_t li, const int* pos_ptr, size_t pos0, size_t m, bool batch) {
  const aotcu_dims& d = g->head.dims;
  const aotcu_layer& l = g->layers[li];
  aotcu_ctx* c = g->c;
  const size_t dim = d.dim, qd = (size_t)d.n_head * d.head_dim, kvd = (size_t)d.n_kv_head * d.head_dim;
  float* x = g->bufs[batch ? AOTCU_BUF_BX : AOTCU_BUF_X];
  float* xb = g->bufs[batch ? AOTCU_BUF_BXB : AOTCU_BUF_XB];
  float* xb2 = g->bufs[batch ? AOTCU_BUF_BXB2 : AOTCU_BUF_XB2];
  float* q = g->bufs[batch ? AOTCU_BUF_BQ : AOTCU_BUF_Q];
  float* k = g->bufs[batch ? AOTCU_BUF_BK : AOTCU_BUF_K];
  float* v = g->bufs[batch ? AOTCU_BUF_BV : AOTCU_BUF_V];
  float* hb = g->bufs[batch ? AOTCU_BUF_BHB : AOTCU_BUF_HB];
  float* hb2 = g->bufs[batch ? AOTCU_BUF_BHB2 : AOTCU_BUF_HB2];
  const size_t window = l.local_attn ? (size_t)d.swa_window : 0;

  // emit.rs:250-272
  if (int rc = gpu_rmsnorm(g, xb, dim, x, dim, wf32(g, l.attn_norm), dim, m, d.eps, 0, true)) return rc;
  float* const qkv[3] = {q, k, v};
  const aotcu_tensor* const wqkv[3] = {&l.wq, &l.wk, &l.wv};
  if (int rc = gpu_mv3(g, qkv, wqkv, xb, m)) return rc;
  if (d.qkv_bias) {  // emit.rs:273-277
    if (int rc = launch(c, add_bias_rows_kernel, dim3(grid_for(c, qd * m, 256)), dim3(256), 0, q, wf32(g, l.bq), qd, m)) return rc;
    if (int rc = launch(c, add_bias_rows_kernel, dim3(grid_for(c, kvd * m, 256)), dim3(256), 0, k, wf32(g, l.bk), kvd, m)) return rc;
    if (int rc = launch(c, add_bias_rows_kernel, dim3(grid_for(c, kvd * m, 256)), dim3(256), 0, v, wf32(g, l.bv), kvd, m)) return rc;
  }
  // emit.rs:278-286: q/k norm, rope, store_kv
  if (int rc = gpu_qk_post(g, li, pos_ptr, pos0, m, batch)) return rc;
  // emit.rs:287
  if (int rc = gpu_attention(g, xb, q, li, pos_ptr, pos0, m, window)) return rc;
  // emit.rs:288-295
  const bool tp = g->tp && g->tp->world > 1;
  if (d.post_norms) {
    if (int rc = gpu_matmul(g, xb2, l.wo, xb, m, 0)) return rc;
    if (tp)
      if (int rc = tp_all_reduce(g, xb2, m * dim)) return rc;
    if (int rc = gpu_rmsnorm(g, x, dim, xb2, dim, wf32(g, l.attn_post_norm), dim, m, d.eps, 1, false)) return rc;
  } else if (tp) {
    // this rank's heads give a partial attn_output; the ranks' partials are summed, then joined
    if (int rc = gpu_matmul(g, xb2, l.wo, xb, m, 0)) return rc;
    if (int rc = tp_all_reduce(g, xb2, m * dim)) return rc;
    if (int rc = gpu_add(g, x, xb2, m * dim)) return rc;
  } else {
    if (int rc = gpu_matmul(g, x, l.wo, xb, m, 1)) return rc;
  }
  // emit.rs:297-331
  if (int rc = gpu_rmsnorm(g, xb, dim, x, dim, wf32(g, l.ffn_norm), dim, m, d.eps, 0, true)) return rc;
  if (int rc = gpu_gate_up(g, hb, hb2, l.gate, l.up, xb, m)) return rc;
  if (d.post_norms) {
    if (int rc = gpu_matmul(g, xb2, l.down, hb, m, 0)) return rc;
    if (tp)
      if (int rc = tp_all_reduce(g, xb2, m * dim)) return rc;
    if (int rc = gpu_rmsnorm(g, x, dim, xb2, dim, wf32(g, l.ffn_post_norm), dim, m, d.eps, 1, false)) return rc;
  } else if (tp) {
    if (int rc = gpu_matmul(g, xb2, l.down, hb, m, 0)) return rc;
    if (int rc = tp_all_reduce(g, xb2, m * dim)) return rc;
    if (int rc = gpu_add(g, x, xb2, m * dim)) return rc;
  } else {
    if (int rc = gpu_matmul(g, x, l.down, hb, m, 1)) return rc;
  }
  return 0;
}

static int embed(aotcu_gpu* g, float* dst, const int* d_tokens, size_t m) {
  const aotcu_dims& d = g->head.dims;
  const aotcu_tensor& e = g->head.token_embd;
  note_write(g, dst);
  return launch(g->c, embed_rows_kernel, dim3((d.dim + 255) / 256, (unsigned)m), dim3(256), 0, dst, wptr(g, e), d_tokens,
                (int)e.kind, (int)d.dim, kind_row_bytes(e.kind, e.cols), sqrtf((float)d.dim), (int)d.embd_scale);
}

static int logits_from(aotcu_gpu* g, const float* xrow) {
  const aotcu_dims& d = g->head.dims;
  const aotcu_tensor& out_t = g->head.output.present ? g->head.output : g->head.token_embd;
  float* xb = g->bufs[AOTCU_BUF_XB];
  if (int rc = gpu_rmsnorm(g, xb, d.dim, xrow, d.dim, wf32(g, g->head.output_norm), d.dim, 1, d.eps, 0, true)) return rc;
  return gpu_matmul(g, g->bufs[AOTCU_BUF_LOGITS], out_t, xb, 1, 0);
}


// Decide whether the one-kernel decode step can run this model and build its
// description. It handles the plain Llama / Qwen3 block (K-quant matrices, optional
// per-head q/k norm, either RoPE layout); everything else keeps the per-operator path.
static int mega_setup(aotcu_gpu* g) {
  aotcu_ctx* c = g->c;
  const aotcu_dims& d = g->head.dims;
  const aotcu_tensor& out_t = g->head.output.present ? g->head.output : g->head.token_embd;
  const size_t qd = (size_t)d.n_head * d.head_dim;
  bool ok = !d.qkv_bias && !d.post_norms && !d.gelu && !d.embd_scale && d.swa_window == 0 && d.dim % 256 == 0 &&
            d.hidden % 256 == 0 && qd % 256 == 0 && d.head_dim % 16 == 0 && kind_act(out_t.kind) == ACT_Q8_K;
  for (const auto& l : g->layers) {
    const aotcu_tensor* ts[7] = {&l.wq, &l.wk, &l.wv, &l.wo, &l.gate, &l.up, &l.down};
    for (auto t : ts) ok = ok && kind_act(t->kind) == ACT_Q8_K;
    ok = ok && l.gate.kind == l.up.kind && l.gate.rows == l.up.rows && !l.local_attn;
  }
  // Every CTA must own a row of every product (the tagged hand-over between phases relies
  // on it), and phase ids must fit the tag's low 10 bits.
  const size_t kvd = (size_t)d.n_kv_head * d.head_dim;
  ok = ok && d.n_layer <= 200 && (size_t)d.dim >= (size_t)c->n_sm && (size_t)d.hidden >= (size_t)c->n_sm &&
       (d.dim + c->n_sm - 1) / c->n_sm <= 64;  // a CTA's rows of the residual stream fit the 64-float parking strip
  if (!ok) return 0;
  size_t nb_max = std::max(std::max((size_t)d.dim, (size_t)d.hidden), qd) / 256;
  // Block-term strips hold two rows of a gate/up pair, norm rows stay in registers (two
  // super-blocks per warp).
  if (((nb_max | 1) * 2 > (size_t)WARP_TERMS_FLOATS) || (size_t)d.dim > (size_t)512 * MEGA_CONSUMER_WARPS) return 0;
  // The largest row of any matrix must fit a ring stage twice (a gate/up pair).
  size_t max_rb = 0;
  for (const auto& l : g->layers) {
    const aotcu_tensor* ts[7] = {&l.wq, &l.wk, &l.wv, &l.wo, &l.gate, &l.up, &l.down};
    for (auto t : ts) max_rb = std::max(max_rb, (size_t)kind_row_bytes(t->kind, t->cols));
  }
  max_rb = std::max(max_rb, (size_t)kind_row_bytes(out_t.kind, out_t.cols));
  // Scratch: a head of norm rows (2 x dim) or attention vectors (q, k, v, squares, scores),
  // then the area that stages cached K and V rows. 72 KB of staging hold every cached row of
  // one head up to 140 positions at head_dim 64; longer contexts go through two chunk buffers.
  const size_t small_floats = (std::max((size_t)2 * d.dim, (size_t)5 * d.head_dim + ((g->n_ctx + 3) & ~(size_t)3)) + 31) & ~(size_t)31;
  size_t stage_floats = 18432;
  const size_t table_bytes = (((size_t)d.n_layer + 1) * sizeof(StepLayer) + 15) & ~(size_t)15;
  size_t scratch = 0, fixed = 0;
  int stage_bytes = 0, n_stages = 0;
  for (;;) {
    scratch = ((small_floats + stage_floats) * sizeof(float) + 127) & ~(size_t)127;
    fixed = nb_max * XK_STRIDE + scratch + MEGA_TAIL_BYTES + table_bytes;
    // ring: the stage size that leaves the least shared memory unused
    size_t best = 0;
    for (int sb : {16384, 24576, 32768, 12288}) {
      if (2 * max_rb + 192 > (size_t)sb || fixed + 2 * (size_t)sb > c->max_smem) continue;
      int ns = (int)std::min<size_t>(8, (c->max_smem - fixed) / sb);
      if ((size_t)ns * sb > best) {
        best = (size_t)ns * sb;
        stage_bytes = sb;
        n_stages = ns;
      }
    }
    if (best >= 96 * 1024 || stage_floats <= 6144) break;
    stage_floats -= 2048;  // a small ring starves the products: give staging space back
  }
  if (n_stages < 2) return 0;
  const int v_chunk = (int)(stage_floats / 2 / (d.head_dim + 4)) & ~7;  // positions per chunk buffer (a multiple of 8)
  if (v_chunk < 8) return 0;
  // One CTA per SM must be resident for the grid barriers.
  CU_TRY(cudaFuncSetAttribute(decode_step_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  CU_TRY(cudaFuncSetAttribute(decode_step_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  CU_TRY(cudaFuncSetAttribute(decode_step_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  CU_TRY(cudaFuncSetAttribute(decode_step_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  g->mega_smem = (size_t)n_stages * stage_bytes + fixed;
  int per_sm = 0;
  CU_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<true, true>, MEGA_THREADS, g->mega_smem));
  if (per_sm < 1) return 0;

  auto seg = [&](const aotcu_tensor& t, float* out) { return GemvSeg{wptr(g, t), out, (int)t.rows, t.kind}; };
  auto make_op = [&](std::initializer_list<GemvSeg> segs, int pair, int cols, int epilogue, int ll) {
    MegaOp op = {};
    op.ll = ll;
    size_t max_rb = 1;
    int span = 0, i = 0;
    for (const GemvSeg& sg : segs) {
      op.seg[i] = sg;
      op.row_bytes[i] = (uint32_t)kind_row_bytes(sg.kind, cols);
      max_rb = std::max(max_rb, (size_t)op.row_bytes[i]);
      span += sg.rows;
      i++;
    }
    op.nseg = i;
    op.pair = pair;
    op.cols = cols;
    op.span_rows = pair ? op.seg[0].rows : span;
    op.rows_per_cta = (op.span_rows + c->n_sm - 1) / c->n_sm;
    op.cta_base = op.span_rows / c->n_sm;
    op.cta_rem = op.span_rows % c->n_sm;
    int tr = (int)((size_t)(stage_bytes - 192) / (max_rb * (pair ? 2 : 1)));
    op.tile_rows = tr < 1 ? 1 : (tr > TILE_MAX_UNITS ? TILE_MAX_UNITS : tr);
    op.epilogue = epilogue;
    megaop_derive(op);
    return op;
  };
  // Tagged vectors: residual, q, k, v, attention output, activated hidden. Zeroed once:
  // tag 0 is never waited for.
  const size_t ll_words = (size_t)d.dim + qd + 2 * kvd + qd + (size_t)d.hidden + (size_t)d.n_head * g->n_ctx;
  CU_TRY(cudaMalloc(&g->d_ll, ll_words * sizeof(LLWord)));
  CU_TRY(cudaMemset(g->d_ll, 0, ll_words * sizeof(LLWord)));
  LLWord* const xl = reinterpret_cast<LLWord*>(g->d_ll);
  LLWord* const ql = xl + d.dim;
  LLWord* const kl = ql + qd;
  LLWord* const vl = kl + kvd;
  LLWord* const attl = vl + kvd;
  LLWord* const hbl = attl + qd;
  LLWord* const scl = hbl + d.hidden;
  auto as_out = [](LLWord* p) { return reinterpret_cast<float*>(p); };
  std::vector<StepLayer> hl(d.n_layer + 1);
  for (int i = 0; i < d.n_layer; i++) {
    const aotcu_layer& l = g->layers[i];
    hl[i].attn_norm = wf32(g, l.attn_norm);
    hl[i].ffn_norm = wf32(g, l.ffn_norm);
    hl[i].q_norm = d.qk_norm ? wf32(g, l.q_norm) : nullptr;
    hl[i].k_norm = d.qk_norm ? wf32(g, l.k_norm) : nullptr;
    hl[i].qkv = make_op({seg(l.wq, as_out(ql)), seg(l.wk, as_out(kl)), seg(l.wv, as_out(vl))}, 0, d.dim, EPI_STORE, 1);
    hl[i].wo = make_op({seg(l.wo, as_out(xl))}, 0, (int)qd, EPI_ACCUM, 1);
    hl[i].gu = make_op({seg(l.gate, as_out(hbl)), seg(l.up, nullptr)}, 1, d.dim, EPI_SILU_MUL, 1);
    hl[i].down = make_op({seg(l.down, as_out(xl))}, 0, d.hidden, EPI_ACCUM, 1);
  }
  // The output head rides in the slot after the last layer (only its qkv field is used).
  hl[d.n_layer] = StepLayer{};
  hl[d.n_layer].qkv = make_op({seg(out_t, g->bufs[AOTCU_BUF_LOGITS])}, 0, d.dim, EPI_STORE, 0);
  CU_TRY(cudaMalloc(&g->d_step_layers, hl.size() * sizeof(StepLayer) + 16));
  CU_TRY(cudaMemcpy(g->d_step_layers, hl.data(), hl.size() * sizeof(StepLayer), cudaMemcpyHostToDevice));
  CU_TRY(cudaMalloc(&g->d_grid_bar, 2 * sizeof(unsigned)));
  CU_TRY(cudaMemset(g->d_grid_bar, 0, 2 * sizeof(unsigned)));
  StepParams& P = g->step_params;
  P.dim = d.dim; P.hidden = d.hidden; P.n_layer = d.n_layer; P.n_head = d.n_head; P.n_kv_head = d.n_kv_head;
  P.head_dim = d.head_dim; P.rot_dim = d.rot_dim; P.vocab = (int)out_t.rows; P.n_ctx = (int)g->n_ctx;
  P.eps = d.eps; P.qk_norm = d.qk_norm; P.neox = d.rope_neox;
  P.layers = g->d_step_layers;
  P.output_norm = wf32(g, g->head.output_norm);
  P.out_op = &g->d_step_layers[d.n_layer].qkv;
  P.token_embd = wptr(g, g->head.token_embd);
  P.embd_kind = g->head.token_embd.kind;
  P.embd_row_bytes = kind_row_bytes(g->head.token_embd.kind, g->head.token_embd.cols);
  P.xl = xl; P.ql = ql; P.kl = kl; P.vl = vl; P.attl = attl; P.hbl = hbl; P.scl = scl;
  P.x = g->bufs[AOTCU_BUF_X];
  P.logits = g->bufs[AOTCU_BUF_LOGITS]; P.k_cache = g->bufs[AOTCU_BUF_KCACHE]; P.v_cache = g->bufs[AOTCU_BUF_VCACHE];
  P.epoch = g->d_grid_bar + 1;
  P.rope_table = g->rope_table;
  P.step = g->d_step; P.history = g->d_history; P.history_cap = (int)g->history_cap; P.out_token = g->d_out_token;
  P.grid_bar = g->d_grid_bar; P.err = c->d_err;
  P.n_stages = n_stages; P.stage_bytes = stage_bytes; P.scratch_bytes = (int)scratch; P.v_chunk = v_chunk; P.table_bytes = (int)table_bytes;
  P.small_floats = (int)small_floats; P.stage_floats = (int)stage_floats;
  P.fast = 0;
  P.spin_limit = 1 << 21;  // about two seconds of polling
  g->mega_ok = true;
  return 0;
}

static void drop_graphs(aotcu_gpu* g) {
  for (auto& e : g->decode_graph)
    if (e) {
      cudaGraphExecDestroy(e);
      e = nullptr;
    }
  for (auto& e : g->gen_graph)
    if (e) {
      cudaGraphExecDestroy(e);
      e = nullptr;
    }
}

// Whether the one-kernel step at position `pos` shares each head between several CTAs: the
// head's cached K and V rows no longer fit one CTA's staging area, and there are at least
// two CTAs per head. The choice is the host's (it selects the kernel variant), so that the
// short-context variant carries none of the long-context code.
static int mega_split(const aotcu_gpu* g, size_t pos) {
  const StepParams& P = g->step_params;
  return g->mega_ok && g->use_mega && g->c->n_sm >= 2 * P.n_head && 2 * (pos + 1) * (size_t)P.head_dim > (size_t)P.stage_floats;
}

static int enqueue_mega(aotcu_gpu* g, int want_logits, bool with_argmax, unsigned long long* prof = nullptr,
                        int prof_cta = 0, unsigned long long* timeline = nullptr, int timeline_layer = 0) {
  aotcu_ctx* c = g->c;
  StepParams P = g->step_params;
  P.prof = prof;
  P.prof_cta = prof_cta;
  P.timeline = timeline;
  P.timeline_layer = timeline_layer;
  P.want_logits = want_logits;
  P.with_argmax = with_argmax ? 1 : 0;
  CU_TRY(cudaMemsetAsync(g->d_grid_bar, 0, sizeof(unsigned), c->stream));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c->n_sm);
  cfg.blockDim = dim3(MEGA_THREADS);
  cfg.dynamicSmemBytes = g->mega_smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (g->split_now)
    e = P.tp.world > 1 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<true, true>, P) : cudaLaunchKernelEx(&cfg, decode_step_kernel<false, true>, P);
  else
    e = P.tp.world > 1 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<true, false>, P) : cudaLaunchKernelEx(&cfg, decode_step_kernel<false, false>, P);
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "decode_step_kernel launch: %s", cudaGetErrorString(e));
  c->launches++;
  g->qsrc = aotcu_gpu::QSrc();
  return 0;
}

// Enqueue one decode step reading {token, pos} from g->d_step.
static int enqueue_decode(aotcu_gpu* g, int want_logits, bool with_argmax) {
  if (g->mega_ok && g->use_mega) return enqueue_mega(g, want_logits, with_argmax);
  const aotcu_dims& d = g->head.dims;
  g->qsrc = aotcu_gpu::QSrc();
  if (int rc = embed(g, g->bufs[AOTCU_BUF_X], g->d_step, 1)) return rc;
  for (int i = 0; i < d.n_layer; i++)
    if (int rc = layer_forward(g, (size_t)i, g->d_step + 1, 0, 1, false)) return rc;
  if (want_logits) {
    if (int rc = logits_from(g, g->bufs[AOTCU_BUF_X])) return rc;
    if (with_argmax) {
      if (g->head_sharded)
        if (int rc = tp_gather_logits(g)) return rc;
      if (int rc = launch(g->c, argmax_kernel, dim3(1), dim3(1024), 0,
                          (const float*)(g->head_sharded ? g->tp_logits_full : g->bufs[AOTCU_BUF_LOGITS]), (int)d.vocab,
                          g->d_out_token, g->d_step, g->d_history, (int)g->history_cap))
        return rc;
    }
  }
  g->qsrc = aotcu_gpu::QSrc();
  return 0;
}

static int capture_graph(aotcu_gpu* g, cudaGraphExec_t* exec, uint64_t* n_kernels, int want_logits, bool with_argmax) {
  aotcu_ctx* c = g->c;
  cudaGraph_t graph = nullptr;
  CU_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  uint64_t before = c->launches;
  int rc = enqueue_decode(g, want_logits, with_argmax);
  cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
  *n_kernels = c->launches - before;
  c->launches = before;  // captured, not launched
  if (rc) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  return 0;
}

static int check_device_errors(aotcu_ctx* c) {
  int h = 0;
  CU_TRY(cudaMemcpyAsync(&h, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  if (h) {
    CU_TRY(cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream));
    if (h & (DEVERR_MBAR_TIMEOUT | DEVERR_GRID_TIMEOUT))
      return fail(AOTCU_ERR_TIMEOUT, "a bounded device-side wait expired (error word %d)", h);
    return fail(AOTCU_ERR_CUDA, "device error word %d", h);
  }
  return 0;
}

// =====================================================================================
// extern "C"
// =====================================================================================
extern "C" {

const char* aotcu_last_error(void) { return g_last_error.c_str(); }
const char* aotcu_version(void) { return "aot-cuda 0.1 (sm_100a)"; }
size_t aotcu_row_bytes(int kind, size_t cols) { return kind_row_bytes(kind, cols); }

int aotcu_init(int device, aotcu_ctx** out) {
  ARG_CHECK(out, "out is NULL");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(AOTCU_ERR_CUDA, "no CUDA device (%s); this library has no CPU path", e == cudaSuccess ? "count 0" : cudaGetErrorString(e));
  ARG_CHECK(device >= 0 && device < n, "device %d out of range (have %d)", device, n);
  CU_TRY(cudaSetDevice(device));
  cudaDeviceProp prop;
  CU_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major < 10) return fail(AOTCU_ERR_UNSUPPORTED, "device %s is sm_%d%d; this library is built for sm_100a only", prop.name, prop.major, prop.minor);
  aotcu_ctx* c = new aotcu_ctx();
  c->device = device;
  c->n_sm = prop.multiProcessorCount;
  // Keep 1 KiB back for the kernels' small static shared arrays.
  c->max_smem = prop.sharedMemPerBlockOptin - 1024;
  CU_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  CU_TRY(cudaMalloc(&c->d_err, sizeof(int)));
  CU_TRY(cudaMemset(c->d_err, 0, sizeof(int)));
  CU_TRY(cudaFuncSetAttribute(gemv_q8k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  CU_TRY(cudaFuncSetAttribute(gemv_q80_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c->max_smem));
  // These two also hold the exact-sum scratch in static shared memory.
  CU_TRY(cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)(c->max_smem - sizeof(SeqSumScratch) - 1024)));
  CU_TRY(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem_budget(c)));
  *out = c;
  return 0;
}

void aotcu_free(aotcu_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  // A Gpu must not outlive its context: whatever the caller left alive goes first.
  while (!c->gpus.empty()) aotcu_gpu_free(c->gpus.back());
  if (c->stream) {
    cudaStreamSynchronize(c->stream);
    cudaStreamDestroy(c->stream);
  }
  cudaFree(c->d_err);
  if (c->ximg) cudaFree(c->ximg);
  if (c->t0) cudaEventDestroy(c->t0);
  if (c->t1) cudaEventDestroy(c->t1);
  delete c;
}

int aotcu_sync(aotcu_ctx* c) {
  ARG_CHECK(c, "ctx is NULL");
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

int aotcu_malloc(aotcu_ctx* c, size_t bytes, void** p) {
  ARG_CHECK(c && p, "NULL argument");
  if (int rc = ctx_set_device(c)) return rc;
  CU_TRY(cudaMalloc(p, bytes + WEIGHT_PAD));
  CU_TRY(cudaMemsetAsync((uint8_t*)*p + bytes, 0, WEIGHT_PAD, c->stream));
  return 0;
}

int aotcu_dev_free(aotcu_ctx* c, void* p) {
  ARG_CHECK(c, "ctx is NULL");
  CU_TRY(cudaStreamSynchronize(c->stream));
  CU_TRY(cudaFree(p));
  return 0;
}

int aotcu_h2d(aotcu_ctx* c, void* dst, const void* src, size_t bytes) {
  ARG_CHECK(c && (bytes == 0 || (dst && src)), "NULL argument");
  CU_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

int aotcu_d2h(aotcu_ctx* c, void* dst, const void* src, size_t bytes) {
  ARG_CHECK(c && (bytes == 0 || (dst && src)), "NULL argument");
  CU_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

int aotcu_timer_start(aotcu_ctx* c) {
  ARG_CHECK(c, "ctx is NULL");
  if (!c->t0) {
    CU_TRY(cudaEventCreate(&c->t0));
    CU_TRY(cudaEventCreate(&c->t1));
  }
  CU_TRY(cudaEventRecord(c->t0, c->stream));
  return 0;
}

int aotcu_timer_stop(aotcu_ctx* c, float* ms) {
  ARG_CHECK(c && ms && c->t0, "timer was not started");
  CU_TRY(cudaEventRecord(c->t1, c->stream));
  CU_TRY(cudaEventSynchronize(c->t1));
  CU_TRY(cudaEventElapsedTime(ms, c->t0, c->t1));
  return 0;
}

int aotcu_device_status(aotcu_ctx* c) {
  ARG_CHECK(c, "ctx is NULL");
  return check_device_errors(c);
}

// ---- kernel level ---------------------------------------------------------------------
int aotcu_quantize_q8_0(aotcu_ctx* c, const float* x, size_t n, aotcu_block_q8_0* out) {
  ARG_CHECK(c && x && out, "NULL argument");
  ARG_CHECK(n % 32 == 0, "n (%zu) is not a multiple of 32", n);
  if (n == 0) return 0;
  int nblk = (int)(n / 32);
  return launch(c, quantize_q80_kernel, dim3(grid_for(c, nblk, 8)), dim3(256), 0, x, (uint8_t*)out, nblk, 0);
}

int aotcu_quantize_q8_k(aotcu_ctx* c, const float* x, size_t n, aotcu_block_q8_k* out) {
  ARG_CHECK(c && x && out, "NULL argument");
  ARG_CHECK(n % 256 == 0, "n (%zu) is not a multiple of 256", n);
  if (n == 0) return 0;
  int nblk = (int)(n / 256);
  return launch(c, quantize_q8k_kernel, dim3(grid_for(c, nblk, 8)), dim3(256), 0, x, (uint8_t*)out, nblk, 0);
}

int aotcu_dequant_rows(aotcu_ctx* c, int kind, const uint8_t* table, const int32_t* row_ids, size_t n_rows, size_t cols,
                       float* out) {
  ARG_CHECK(c && table && row_ids && out, "NULL argument");
  ARG_CHECK(kind >= 0 && kind < N_KINDS, "unknown kind %d", kind);
  ARG_CHECK(cols % (size_t)kind_block(kind) == 0, "cols not a multiple of the block size");
  if (n_rows == 0 || cols == 0) return 0;
  return launch(c, embed_rows_kernel, dim3((unsigned)((cols + 255) / 256), (unsigned)n_rows), dim3(256), 0, out, table,
                (const int*)row_ids, kind, (int)cols, kind_row_bytes(kind, cols), 1.0f, 0);
}

int aotcu_matvec(aotcu_ctx* c, int kind, float* out, const uint8_t* w, const void* x, size_t rows, size_t cols) {
  return aotcu_matmul(c, kind, out, w, x, 1, rows, cols);
}

#define MATVEC_FN(name, KIND, XT)                                                                              \
  int aotcu_matvec_##name(aotcu_ctx* c, float* out, const uint8_t* w, const XT* x, size_t rows, size_t cols) { \
    return aotcu_matmul(c, KIND, out, w, x, 1, rows, cols);                                                    \
  }
MATVEC_FN(q4_0, AOTCU_Q4_0, aotcu_block_q8_0)
MATVEC_FN(q5_0, AOTCU_Q5_0, aotcu_block_q8_0)
MATVEC_FN(q8_0, AOTCU_Q8_0, aotcu_block_q8_0)
MATVEC_FN(q4_k, AOTCU_Q4_K, aotcu_block_q8_k)
MATVEC_FN(q5_k, AOTCU_Q5_K, aotcu_block_q8_k)
MATVEC_FN(q6_k, AOTCU_Q6_K, aotcu_block_q8_k)
MATVEC_FN(f16, AOTCU_F16, float)
MATVEC_FN(bf16, AOTCU_BF16, float)
MATVEC_FN(f32, AOTCU_F32, float)

int aotcu_matmul(aotcu_ctx* c, int kind, float* out, const uint8_t* w, const void* xs, size_t m, size_t rows,
                 size_t cols) {
  ARG_CHECK(c, "ctx is NULL");
  ARG_CHECK(kind >= 0 && kind < N_KINDS, "unknown kind %d", kind);
  if (rows == 0 || m == 0) return 0;
  GemvCall call;
  call.seg[0] = GemvSeg{w, out, (int)rows, kind};
  call.nseg = 1;
  call.cols = cols;
  call.x = xs;
  call.x_mode = 0;
  call.m = m;
  return launch_gemv(c, call);
}

int aotcu_matvec2(aotcu_ctx* c, int kind, float* out_a, float* out_b, const uint8_t* w_a, const uint8_t* w_b,
                  const void* x, size_t rows, size_t cols) {
  ARG_CHECK(c, "ctx is NULL");
  ARG_CHECK(kind >= 0 && kind < N_KINDS, "unknown kind %d", kind);
  if (rows == 0) return 0;
  GemvCall call;
  call.seg[0] = GemvSeg{w_a, out_a, (int)rows, kind};
  call.seg[1] = GemvSeg{w_b, out_b, (int)rows, kind};
  call.nseg = 2;
  call.pair = 1;
  call.cols = cols;
  call.x = x;
  return launch_gemv(c, call);
}

int aotcu_matmul2(aotcu_ctx* c, int kind, float* out_a, float* out_b, const uint8_t* w_a, const uint8_t* w_b, const void* xs,
                  size_t m, size_t rows, size_t cols) {
  ARG_CHECK(c, "ctx is NULL");
  ARG_CHECK(kind >= 0 && kind < N_KINDS, "unknown kind %d", kind);
  if (rows == 0 || m == 0) return 0;
  GemvCall call;
  call.seg[0] = GemvSeg{w_a, out_a, (int)rows, kind};
  call.seg[1] = GemvSeg{w_b, out_b, (int)rows, kind};
  call.nseg = 2;
  call.pair = 1;
  call.cols = cols;
  call.x = xs;
  call.m = m;
  return launch_gemv(c, call);
}

int aotcu_matvec3(aotcu_ctx* c, const int kinds[3], float* const outs[3], const uint8_t* const ws[3], const void* x,
                  const size_t rows[3], size_t cols) {
  ARG_CHECK(c && kinds && outs && ws && rows, "NULL argument");
  GemvCall call;
  call.nseg = 0;
  for (int i = 0; i < 3; i++) {
    ARG_CHECK(kinds[i] >= 0 && kinds[i] < N_KINDS, "unknown kind %d", kinds[i]);
    if (rows[i] == 0) continue;
    call.seg[call.nseg++] = GemvSeg{ws[i], outs[i], (int)rows[i], kinds[i]};
  }
  if (call.nseg == 0) return 0;
  call.cols = cols;
  call.x = x;
  return launch_gemv(c, call);
}

int aotcu_block_sums(aotcu_ctx* c, int kind, const uint8_t* w, const void* x, size_t rows, size_t cols, int32_t* sumi,
                     int32_t* summ) {
  ARG_CHECK(c && w && x && sumi, "NULL argument");
  ARG_CHECK(kind >= AOTCU_Q4_0 && kind <= AOTCU_Q6_K, "kind %d has no integer block sums", kind);
  ARG_CHECK(cols % (size_t)kind_block(kind) == 0, "cols not a multiple of the block size");
  int nb = (int)(cols / kind_block(kind));
  if (rows == 0 || nb == 0) return 0;
  return launch(c, block_sums_kernel, dim3(grid_for(c, rows * nb, 128)), dim3(128), 0, kind, w, (const uint8_t*)x,
                (int)rows, nb, sumi, summ);
}

int aotcu_block_sums_of(aotcu_ctx* c, int kernel, int kind, const uint8_t* w, const void* x, size_t m, size_t rows, size_t cols,
                        int32_t* sumi, int32_t* summ) {
  ARG_CHECK(c && w && x && sumi && summ, "NULL argument");
  ARG_CHECK(kind == AOTCU_Q4_K || kind == AOTCU_Q5_K || kind == AOTCU_Q6_K, "kind %d is not a K-quant", kind);
  ARG_CHECK(cols > 0 && cols % 256 == 0 && rows > 0, "bad shape");
  ARG_CHECK(kernel == 0 || kernel == 1, "kernel: 0 = streaming single-row product, 1 = tcgen05 prompt product");
  if (int rc = ctx_set_device(c)) return rc;
  float* out = nullptr;
  CU_TRY(cudaMalloc(&out, m * rows * sizeof(float)));
  int rc = 0;
  if (kernel == 0) {
    if (m != 1) rc = fail(AOTCU_ERR_BAD_ARG, "the streaming product takes one activation row");
    GemvCall call;
    call.seg[0] = GemvSeg{w, out, (int)rows, kind};
    call.nseg = 1;
    call.cols = cols;
    call.x = x;
    call.x_mode = 0;
    call.m = 1;
    g_dbg_sumi = sumi;
    g_dbg_summ = summ;
    if (!rc) rc = launch_gemv_stream(c, call, rows);
    g_dbg_sumi = g_dbg_summ = nullptr;
  } else {
    if (kind == AOTCU_Q6_K || m < 1 || m > (size_t)TC_TOK) rc = fail(AOTCU_ERR_BAD_ARG, "the tcgen05 product takes Q4_K / Q5_K and 1..64 rows");
    GemvCall call;
    call.seg[0] = GemvSeg{w, out, (int)rows, kind};
    call.nseg = 1;
    call.cols = cols;
    call.x = x;
    call.x_mode = 0;
    call.m = m;
    g_dbg_sumi = sumi;
    g_dbg_summ = summ;
    if (!rc) rc = launch_gemm_tc(c, call);
    g_dbg_sumi = g_dbg_summ = nullptr;
  }
  if (!rc) rc = check_device_errors(c);
  cudaFree(out);
  return rc;
}

int aotcu_rmsnorm(aotcu_ctx* c, float* out, const float* x, const float* w, size_t n, size_t m, float eps) {
  ARG_CHECK(c && out && x && w, "NULL argument");
  if (n == 0 || m == 0) return 0;
  RmsnormParams P = {};
  P.x = x;
  P.w = w;
  P.out = out;
  P.n = (int)n;
  P.x_stride = P.out_stride = (int)n;
  P.eps = eps;
  size_t smem = (2 * n + 4) * sizeof(float);
  ARG_CHECK(smem <= c->max_smem, "row of %zu floats does not fit shared memory", n);
  return launch(c, rmsnorm_kernel, dim3((unsigned)m), dim3(512), smem, P);
}

int aotcu_rmsnorm_heads(aotcu_ctx* c, float* x, const float* w, size_t n_heads, size_t head_dim, float eps) {
  ARG_CHECK(c && x && w, "NULL argument");
  ARG_CHECK(head_dim >= 1 && head_dim <= 256, "head_dim %zu out of range (1..256)", head_dim);
  if (n_heads == 0) return 0;
  return launch(c, rmsnorm_heads_kernel, dim3((unsigned)n_heads), dim3(128), 0, x, w, (int)head_dim, eps);
}

int aotcu_rope(aotcu_ctx* c, float* x, size_t m, size_t n_heads, size_t head_dim, size_t rot_dim, const float* cs,
               int neox) {
  ARG_CHECK(c && x && cs, "NULL argument");
  ARG_CHECK(rot_dim <= head_dim && rot_dim % 2 == 0, "rot_dim %zu invalid for head_dim %zu", rot_dim, head_dim);
  size_t total = m * n_heads * (rot_dim / 2);
  if (total == 0) return 0;
  return launch(c, rope_kernel, dim3(grid_for(c, total, 256)), dim3(256), 0, x, (int)m, (int)n_heads, (int)head_dim,
                (int)rot_dim, cs, (int)rot_dim, neox);
}

int aotcu_silu_mul(aotcu_ctx* c, float* h, const float* up, size_t n) {
  ARG_CHECK(c && h && up, "NULL argument");
  if (n == 0) return 0;
  return launch(c, silu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, h, up, n);
}

int aotcu_gelu_mul(aotcu_ctx* c, float* h, const float* up, size_t n) {
  ARG_CHECK(c && h && up, "NULL argument");
  if (n == 0) return 0;
  return launch(c, gelu_mul_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, h, up, n);
}

int aotcu_add_inplace(aotcu_ctx* c, float* x, const float* y, size_t n) {
  ARG_CHECK(c && x && y, "NULL argument");
  if (n == 0) return 0;
  return launch(c, add_inplace_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, x, y, n);
}

int aotcu_add_bias_rows(aotcu_ctx* c, float* x, const float* b, size_t n, size_t m) {
  ARG_CHECK(c && x && b, "NULL argument");
  if (n * m == 0) return 0;
  return launch(c, add_bias_rows_kernel, dim3(grid_for(c, n * m, 256)), dim3(256), 0, x, b, n, m);
}

int aotcu_scale_inplace(aotcu_ctx* c, float* x, float s, size_t n) {
  ARG_CHECK(c && x, "NULL argument");
  if (n == 0) return 0;
  return launch(c, scale_inplace_kernel, dim3(grid_for(c, n, 256)), dim3(256), 0, x, s, n);
}

int aotcu_attention(aotcu_ctx* c, float* out, const float* q, const float* k_cache, const float* v_cache,
                    size_t n_head, size_t n_kv_head, size_t head_dim, size_t ctx_len, size_t pos0, size_t m,
                    size_t window) {
  ARG_CHECK(c && out && q && k_cache && v_cache, "NULL argument");
  ARG_CHECK(n_kv_head > 0 && n_head % n_kv_head == 0, "n_head must be a multiple of n_kv_head");
  ARG_CHECK(head_dim % 4 == 0 && head_dim <= 256, "head_dim %zu must be a multiple of 4, at most 256", head_dim);
  ARG_CHECK(pos0 + m <= ctx_len, "positions exceed the context");
  if (m == 0) return 0;
  ARG_CHECK(attn_smem_bytes(c, (int)n_head, (int)n_kv_head, (int)head_dim, pos0 + m, m) <= attn_smem_budget(c),
            "%zu positions are too many for the stand-alone attention entry point (scores are kept in shared memory)", pos0 + m);
  return launch_attention(c, out, q, k_cache, v_cache, nullptr, nullptr, pos0, m, (int)n_head, (int)n_kv_head,
                          (int)head_dim, ctx_len, window, (int)ctx_len);
}

int aotcu_argmax(aotcu_ctx* c, const float* x, size_t n, int32_t* out_token) {
  ARG_CHECK(c && x && out_token, "NULL argument");
  ARG_CHECK(n >= 1 && n < (1u << 31), "n out of range");
  return launch(c, argmax_kernel, dim3(1), dim3(1024), 0, x, (int)n, (int*)out_token, (int*)nullptr, (int*)nullptr, 0);
}

// ---- backend level -----------------------------------------------------------------------
int aotcu_gpu_new(aotcu_ctx* c, const aotcu_model_head* head, const aotcu_layer* layers, const uint8_t* weights,
                  size_t weights_len, size_t n_ctx, size_t max_batch, aotcu_gpu** out) {
  ARG_CHECK(c && head && layers && weights && out, "NULL argument");
  const aotcu_dims& d = head->dims;
  ARG_CHECK(d.dim > 0 && d.hidden > 0 && d.n_layer > 0 && d.n_head > 0 && d.n_kv_head > 0 && d.head_dim > 0 && d.vocab > 0,
            "dimensions must be positive");
  ARG_CHECK(d.n_head % d.n_kv_head == 0, "n_head must be a multiple of n_kv_head");
  ARG_CHECK(d.head_dim % 4 == 0 && d.head_dim <= 256, "head_dim %d must be a multiple of 4, at most 256", d.head_dim);
  ARG_CHECK(d.rot_dim % 2 == 0 && d.rot_dim <= d.head_dim, "rot_dim %d invalid", d.rot_dim);
  ARG_CHECK(n_ctx >= 1, "context must hold at least one token");
  if (int rc = ctx_set_device(c)) return rc;
  aotcu_gpu* g = new aotcu_gpu();
  g->c = c;
  c->gpus.push_back(g);
  g->head = *head;
  g->layers.assign(layers, layers + d.n_layer);
  g->n_ctx = n_ctx;
  g->max_batch = max_batch < 1 ? 1 : max_batch;
  g->weights_len = weights_len;

  auto bail = [&](int rc) {
    aotcu_gpu_free(g);
    return rc;
  };
  // Tensor table checks (the reference trusts its generator; a C caller may not be one).
  {
    struct N {
      const char* n;
      const aotcu_tensor* t;
      bool opt;
    };
    std::vector<N> ts = {{"token_embd", &g->head.token_embd, false}, {"output_norm", &g->head.output_norm, false},
                         {"output", &g->head.output, true}, {"rope_freqs", &g->head.rope_freqs, true}};
    for (auto& l : g->layers) {
      ts.push_back({"attn_norm", &l.attn_norm, false});
      ts.push_back({"wq", &l.wq, false});
      ts.push_back({"wk", &l.wk, false});
      ts.push_back({"wv", &l.wv, false});
      ts.push_back({"wo", &l.wo, false});
      ts.push_back({"ffn_norm", &l.ffn_norm, false});
      ts.push_back({"gate", &l.gate, false});
      ts.push_back({"up", &l.up, false});
      ts.push_back({"down", &l.down, false});
      ts.push_back({"bq", &l.bq, !d.qkv_bias});
      ts.push_back({"bk", &l.bk, !d.qkv_bias});
      ts.push_back({"bv", &l.bv, !d.qkv_bias});
      ts.push_back({"q_norm", &l.q_norm, !d.qk_norm});
      ts.push_back({"k_norm", &l.k_norm, !d.qk_norm});
      ts.push_back({"attn_post_norm", &l.attn_post_norm, !d.post_norms});
      ts.push_back({"ffn_post_norm", &l.ffn_post_norm, !d.post_norms});
    }
    for (auto& e : ts) {
      if (e.opt && !e.t->present) continue;
      if (int rc = tensor_check(g, *e.t, e.n)) return bail(rc);
      int a = kind_act(e.t->kind);
      if (e.t->rows > 1 || e.t == &g->head.token_embd) {
        g->need_q8k |= a == ACT_Q8_K;
        g->need_q80 |= a == ACT_Q8_0;
      }
    }
  }
  const size_t dim = d.dim, qd = (size_t)d.n_head * d.head_dim, kvd = (size_t)d.n_kv_head * d.head_dim;
  const size_t xbw = xb_width(d), b = g->max_batch > 1 ? g->max_batch : 0;
  const size_t lens[AOTCU_N_BUFS] = {dim, xbw, dim, qd, kvd, kvd, (size_t)d.hidden, (size_t)d.hidden, (size_t)d.vocab,
                                     (size_t)d.n_layer * n_ctx * kvd, (size_t)d.n_layer * n_ctx * kvd, (size_t)d.rot_dim,
                                     b * dim, b * xbw, b * dim, b * qd, b * kvd, b * kvd, b * d.hidden, b * d.hidden,
                                     b * d.rot_dim, d.swa_window > 0 ? (size_t)d.rot_dim : 0,
                                     d.swa_window > 0 ? b * d.rot_dim : 0};
  cudaError_t e;
#define G_TRY(expr)                                                                       \
  do {                                                                                    \
    e = (expr);                                                                           \
    if (e != cudaSuccess) return bail(fail(AOTCU_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e))); \
  } while (0)
  for (int i = 0; i < AOTCU_N_BUFS; i++) {
    g->buf_len[i] = lens[i];
    if (lens[i] == 0) continue;
    G_TRY(cudaMalloc(&g->bufs[i], lens[i] * sizeof(float) + 64));
    G_TRY(cudaMemsetAsync(g->bufs[i], 0, lens[i] * sizeof(float) + 64, c->stream));
  }
  // Weights: one upload, padded so aligned-superset tile copies stay inside.
  G_TRY(cudaMalloc(&g->d_weights, weights_len + WEIGHT_PAD));
  G_TRY(cudaMemcpyAsync(g->d_weights, weights, weights_len, cudaMemcpyHostToDevice, c->stream));
  G_TRY(cudaMemsetAsync(g->d_weights + weights_len, 0, WEIGHT_PAD, c->stream));
  // RoPE rows for every position (state.rs:308-319, ops.rs:28-34), host libm.
  {
    const size_t half = d.rot_dim / 2;
    std::vector<float> ff;
    if (g->head.rope_freqs.present) {
      ff.resize(half);
      memcpy(ff.data(), weights + g->head.rope_freqs.off, half * sizeof(float));
    }
    auto build = [&](float base, float scale, float** dev) -> cudaError_t {
      std::vector<float> inv(half), tab(n_ctx * d.rot_dim);
      for (size_t i = 0; i < half; i++) {
        float f = powf(base, -(2.0f * (float)i) / (float)d.rot_dim);
        if (!ff.empty()) f /= ff[i];
        inv[i] = f;
      }
      for (size_t p = 0; p < n_ctx; p++) {
        float pf = (float)p / scale;
        for (size_t i = 0; i < half; i++) {
          float a = pf * inv[i];
          tab[p * d.rot_dim + 2 * i] = cosf(a);
          tab[p * d.rot_dim + 2 * i + 1] = sinf(a);
        }
      }
      cudaError_t er = cudaMalloc(dev, tab.size() * sizeof(float));
      if (er != cudaSuccess) return er;
      er = cudaMemcpyAsync(*dev, tab.data(), tab.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream);
      if (er != cudaSuccess) return er;
      return cudaStreamSynchronize(c->stream);
    };
    G_TRY(build(d.rope_base, d.rope_scale, &g->rope_table));
    if (d.swa_window > 0) G_TRY(build(d.rope_base_local, d.rope_scale_local, &g->rope_table_local));
  }
  {
    size_t widest = xbw > (size_t)d.hidden ? xbw : (size_t)d.hidden;
    size_t rows = g->max_batch;
    G_TRY(cudaMalloc(&g->aqk, rows * (widest / 256 + 1) * XIMG_K));
    G_TRY(cudaMalloc(&g->aq0, rows * (widest / 32 + 1) * XIMG_0));
  }
  // Attention scores: shared memory when the context fits, else a global scratch.
  {
    if (attn_smem_bytes(c, d.n_head, d.n_kv_head, d.head_dim, n_ctx, g->max_batch) <= attn_smem_budget(c)) {
      g->smem_scores = (int)n_ctx;
    } else {
      g->smem_scores = 0;
      G_TRY(cudaMalloc(&g->attn_scratch, g->max_batch * d.n_head * ((n_ctx + 3) & ~(size_t)3) * sizeof(float)));
    }
  }
  g->history_cap = n_ctx;
  G_TRY(cudaMalloc(&g->d_step, 4 * sizeof(int)));
  G_TRY(cudaMemsetAsync(g->d_step, 0, 4 * sizeof(int), c->stream));
  G_TRY(cudaMalloc(&g->d_tokens, g->max_batch * sizeof(int)));
  G_TRY(cudaMalloc(&g->d_history, g->history_cap * sizeof(int)));
  G_TRY(cudaMalloc(&g->d_out_token, sizeof(int)));
  G_TRY(cudaMallocHost(&g->h_pinned, (g->max_batch + 8) * sizeof(int)));
  G_TRY(cudaMallocHost(&g->h_logits, (size_t)d.vocab * sizeof(float)));
  G_TRY(cudaStreamSynchronize(c->stream));
#undef G_TRY
  if (int rc = mega_setup(g)) return bail(rc);
  *out = g;
  return 0;
}

void aotcu_gpu_free(aotcu_gpu* g) {
  if (!g) return;
  {
    auto& v = g->c->gpus;
    v.erase(std::remove(v.begin(), v.end(), g), v.end());
  }
  cudaSetDevice(g->c->device);
  cudaStreamSynchronize(g->c->stream);
  drop_graphs(g);
  for (int i = 0; i < AOTCU_N_BUFS; i++) cudaFree(g->bufs[i]);
  cudaFree(g->d_weights);
  cudaFree(g->rope_table);
  cudaFree(g->rope_table_local);
  cudaFree(g->aqk);
  cudaFree(g->aq0);
  cudaFree(g->attn_scratch);
  cudaFree(g->d_step);
  cudaFree(g->d_tokens);
  cudaFree(g->d_history);
  cudaFree(g->d_out_token);
  cudaFree(g->d_step_layers);
  cudaFree(g->d_grid_bar);
  cudaFree(g->d_ll);
  if (g->tp) {
    if (g->tp->comm) g->tp->comm_destroy(g->tp->comm);
    delete g->tp;
  }
  for (void* p : g->tp_peer_map)
    if (p) cudaIpcCloseMemHandle(p);
  cudaFree(g->tp_inbox);
  cudaFree(g->tp_logits_full);
  for (auto& kv : g->prep) cudaFree(kv.second);
  if (g->h_pinned) cudaFreeHost(g->h_pinned);
  if (g->h_logits) cudaFreeHost(g->h_logits);
  delete g;
}

int aotcu_gpu_buf(aotcu_gpu* g, int buf, float** p, size_t* n) {
  ARG_CHECK(g && buf >= 0 && buf < AOTCU_N_BUFS, "bad buffer id %d", buf);
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  if (p) *p = g->bufs[buf];
  if (n) *n = g->buf_len[buf];
  return 0;
}

int aotcu_gpu_read(aotcu_gpu* g, int buf, size_t off, float* dst, size_t n) {
  ARG_CHECK(g && buf >= 0 && buf < AOTCU_N_BUFS && dst, "bad argument");
  ARG_CHECK(off + n <= g->buf_len[buf], "read of %zu floats at %zu exceeds buffer %d (%zu)", n, off, buf, g->buf_len[buf]);
  return aotcu_d2h(g->c, dst, g->bufs[buf] + off, n * sizeof(float));
}

int aotcu_gpu_write(aotcu_gpu* g, int buf, size_t off, const float* src, size_t n) {
  ARG_CHECK(g && buf >= 0 && buf < AOTCU_N_BUFS && src, "bad argument");
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  ARG_CHECK(off + n <= g->buf_len[buf], "write of %zu floats at %zu exceeds buffer %d (%zu)", n, off, buf, g->buf_len[buf]);
  note_write(g, g->bufs[buf]);
  return aotcu_h2d(g->c, g->bufs[buf] + off, src, n * sizeof(float));
}

int aotcu_gpu_begin(aotcu_gpu* g) {
  ARG_CHECK(g, "gpu is NULL");
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  g->qsrc = aotcu_gpu::QSrc();
  return ctx_set_device(g->c);
}

int aotcu_gpu_finish(aotcu_gpu* g) {
  ARG_CHECK(g, "gpu is NULL");
  return check_device_errors(g->c);
}

static int buf_ptr(aotcu_gpu* g, int buf, size_t off, size_t need, float** p) {
  ARG_CHECK(buf >= 0 && buf < AOTCU_N_BUFS, "bad buffer id %d", buf);
  ARG_CHECK(off + need <= g->buf_len[buf], "range %zu+%zu exceeds buffer %d (%zu floats)", off, need, buf, g->buf_len[buf]);
  *p = g->bufs[buf] + off;
  return 0;
}

int aotcu_gpu_rmsnorm(aotcu_gpu* g, int dst, size_t dst_off, int src, size_t src_off, const aotcu_tensor* w, size_t n,
                      size_t m, float eps, int accumulate) {
  ARG_CHECK(g && w, "NULL argument");
  if (int rc = tensor_check(g, *w, "norm weight")) return rc;
  ARG_CHECK(w->kind == AOTCU_F32 && w->rows * w->cols >= n, "norm weights must be f32 with at least n elements");
  float *pd, *ps;
  if (int rc = buf_ptr(g, dst, dst_off, n * m, &pd)) return rc;
  if (int rc = buf_ptr(g, src, src_off, n * m, &ps)) return rc;
  return gpu_rmsnorm(g, pd, n, ps, n, wf32(g, *w), n, m, eps, accumulate, true);
}

int aotcu_gpu_matmul(aotcu_gpu* g, int dst, size_t dst_off, const aotcu_tensor* w, int src, size_t src_off, size_t m,
                     int accumulate) {
  ARG_CHECK(g && w, "NULL argument");
  ARG_CHECK(m >= 1 && m <= g->max_batch, "m (%zu) out of range 1..%zu", m, g->max_batch);
  if (int rc = tensor_check(g, *w, "matrix")) return rc;
  float *pd, *ps;
  if (int rc = buf_ptr(g, dst, dst_off, w->rows * m, &pd)) return rc;
  if (int rc = buf_ptr(g, src, src_off, w->cols * m, &ps)) return rc;
  return gpu_matmul(g, pd, *w, ps, m, accumulate);
}

int aotcu_gpu_mv3(aotcu_gpu* g, const int dst[3], const size_t dst_off[3], const aotcu_tensor* const w[3], int src,
                  size_t m) {
  ARG_CHECK(g && dst && dst_off && w, "NULL argument");
  ARG_CHECK(m >= 1 && m <= g->max_batch, "m (%zu) out of range 1..%zu", m, g->max_batch);
  float* pd[3];
  float* ps;
  for (int i = 0; i < 3; i++) {
    if (int rc = tensor_check(g, *w[i], "q/k/v matrix")) return rc;
    ARG_CHECK(w[i]->cols == w[0]->cols, "q/k/v matrices must share cols");
    if (int rc = buf_ptr(g, dst[i], dst_off[i], w[i]->rows * m, &pd[i])) return rc;
  }
  if (int rc = buf_ptr(g, src, 0, w[0]->cols * m, &ps)) return rc;
  return gpu_mv3(g, pd, w, ps, m);
}

int aotcu_gpu_gate_up(aotcu_gpu* g, int dst, const aotcu_tensor* gate, const aotcu_tensor* up, int src, size_t m) {
  ARG_CHECK(g && gate && up, "NULL argument");
  ARG_CHECK(m >= 1 && m <= g->max_batch, "m (%zu) out of range 1..%zu", m, g->max_batch);
  if (int rc = tensor_check(g, *gate, "gate")) return rc;
  if (int rc = tensor_check(g, *up, "up")) return rc;
  ARG_CHECK(gate->rows == up->rows && gate->cols == up->cols, "gate and up must have the same shape");
  const bool batch = dst == AOTCU_BUF_BHB;
  ARG_CHECK(dst == AOTCU_BUF_HB || dst == AOTCU_BUF_BHB, "gate_up writes Hb or Bhb");
  float *pd, *p2, *ps;
  if (int rc = buf_ptr(g, dst, 0, gate->rows * m, &pd)) return rc;
  if (int rc = buf_ptr(g, batch ? AOTCU_BUF_BHB2 : AOTCU_BUF_HB2, 0, gate->rows * m, &p2)) return rc;
  if (int rc = buf_ptr(g, src, 0, gate->cols * m, &ps)) return rc;
  return gpu_gate_up(g, pd, p2, *gate, *up, ps, m);
}

int aotcu_gpu_qk_post(aotcu_gpu* g, size_t layer, size_t pos0, size_t m) {
  ARG_CHECK(g, "gpu is NULL");
  ARG_CHECK(layer < (size_t)g->head.dims.n_layer, "layer %zu out of range", layer);
  ARG_CHECK(m >= 1 && m <= g->max_batch && pos0 + m <= g->n_ctx, "positions exceed the context");
  return gpu_qk_post(g, layer, nullptr, pos0, m, m > 1);
}

int aotcu_gpu_attention(aotcu_gpu* g, int dst, int q, size_t layer, size_t pos0, size_t m, size_t window) {
  ARG_CHECK(g, "gpu is NULL");
  const aotcu_dims& d = g->head.dims;
  ARG_CHECK(layer < (size_t)d.n_layer, "layer %zu out of range", layer);
  ARG_CHECK(m >= 1 && m <= g->max_batch && pos0 + m <= g->n_ctx, "positions exceed the context");
  float *pd, *pq;
  size_t qd = (size_t)d.n_head * d.head_dim;
  if (int rc = buf_ptr(g, dst, 0, qd * m, &pd)) return rc;
  if (int rc = buf_ptr(g, q, 0, qd * m, &pq)) return rc;
  return gpu_attention(g, pd, pq, layer, nullptr, pos0, m, window);
}

// ---- step level ----------------------------------------------------------------------------
static int set_step(aotcu_gpu* g, uint32_t token, size_t pos, int n_generated) {
  aotcu_ctx* c = g->c;
  // The staging words may still be in flight from the previous step.
  CU_TRY(cudaStreamSynchronize(c->stream));
  g->h_pinned[0] = (int)token;
  g->h_pinned[1] = (int)pos;
  g->h_pinned[2] = n_generated;
  g->h_pinned[3] = 0;
  CU_TRY(cudaMemcpyAsync(g->d_step, g->h_pinned, 4 * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  return 0;
}

int aotcu_forward(aotcu_gpu* g, uint32_t token, size_t pos, int want_logits) {
  ARG_CHECK(g, "gpu is NULL");
  const aotcu_dims& d = g->head.dims;
  // emit.rs:467-468
  ARG_CHECK(token < (uint32_t)d.vocab, "token id out of range");
  ARG_CHECK(pos < g->n_ctx, "position exceeds the context");
  if (int rc = ctx_set_device(g->c)) return rc;
  if (int rc = set_step(g, token, pos, 0)) return rc;
  want_logits = want_logits ? 1 : 0;
  g->split_now = mega_split(g, pos);
  if (g->use_graph) {
    const int gi = want_logits + 2 * g->split_now;
    if (!g->decode_graph[gi])
      if (int rc = capture_graph(g, &g->decode_graph[gi], &g->decode_graph_kernels[gi], want_logits, false)) return rc;
    CU_TRY(cudaGraphLaunch(g->decode_graph[gi], g->c->stream));
    g->c->launches += g->decode_graph_kernels[gi];
  } else {
    if (int rc = enqueue_decode(g, want_logits, false)) return rc;
  }
  // One wait per step: the error word and, when logits were asked for, the logits themselves
  // come back into pinned memory behind the step; aotcu_logits then copies host to host.
  aotcu_ctx* c = g->c;
  g->h_logits_fresh = false;
  CU_TRY(cudaMemcpyAsync(g->h_pinned + 4, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  const bool fetch = want_logits && !g->head_sharded;
  if (fetch)
    CU_TRY(cudaMemcpyAsync(g->h_logits, g->bufs[AOTCU_BUF_LOGITS], (size_t)d.vocab * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  if (const int h = g->h_pinned[4]) {
    CU_TRY(cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream));
    if (h & (DEVERR_MBAR_TIMEOUT | DEVERR_GRID_TIMEOUT))
      return fail(AOTCU_ERR_TIMEOUT, "a bounded device-side wait expired (error word %d)", h);
    return fail(AOTCU_ERR_CUDA, "device error word %d", h);
  }
  g->h_logits_fresh = fetch;
  return 0;
}

int aotcu_forward_batch(aotcu_gpu* g, const uint32_t* tokens, size_t n, size_t pos0, int want_logits) {
  ARG_CHECK(g && tokens, "NULL argument");
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  const aotcu_dims& d = g->head.dims;
  // emit.rs:493-494
  ARG_CHECK(g->max_batch > 1 && n >= 1 && n <= g->max_batch, "batch size out of range");
  ARG_CHECK(pos0 + n <= g->n_ctx, "positions exceed the context");
  for (size_t i = 0; i < n; i++) ARG_CHECK(tokens[i] < (uint32_t)d.vocab, "token id out of range");
  aotcu_ctx* c = g->c;
  if (int rc = ctx_set_device(c)) return rc;
  CU_TRY(cudaStreamSynchronize(c->stream));
  for (size_t i = 0; i < n; i++) g->h_pinned[8 + i] = (int)tokens[i];
  CU_TRY(cudaMemcpyAsync(g->d_tokens, g->h_pinned + 8, n * sizeof(int), cudaMemcpyHostToDevice, c->stream));
  g->qsrc = aotcu_gpu::QSrc();
  if (n >= 8)
    if (int rc = ensure_prepared(g)) return rc;
  if (int rc = embed(g, g->bufs[AOTCU_BUF_BX], g->d_tokens, n)) return rc;
  for (int i = 0; i < d.n_layer; i++)
    if (int rc = layer_forward(g, (size_t)i, nullptr, pos0, n, true)) return rc;
  if (want_logits)
    if (int rc = logits_from(g, g->bufs[AOTCU_BUF_BX] + (n - 1) * d.dim)) return rc;
  g->qsrc = aotcu_gpu::QSrc();
  return check_device_errors(c);
}

int aotcu_logits(aotcu_gpu* g, float* host_dst) {
  ARG_CHECK(g && host_dst, "NULL argument");
  if (g->head_sharded) {
    // collective: every rank of the group calls this after the same forward call
    if (int rc = ctx_set_device(g->c)) return rc;
    if (int rc = tp_gather_logits(g)) return rc;
    return aotcu_d2h(g->c, host_dst, g->tp_logits_full, (size_t)g->head.dims.vocab * sizeof(float));
  }
  if (g->h_logits_fresh) {  // fetched with the step (aotcu_forward)
    memcpy(host_dst, g->h_logits, (size_t)g->head.dims.vocab * sizeof(float));
    return 0;
  }
  return aotcu_d2h(g->c, host_dst, g->bufs[AOTCU_BUF_LOGITS], (size_t)g->head.dims.vocab * sizeof(float));
}


// ---- saved KV cache (prefix.rs) ----------------------------------------------------------------
constexpr size_t KV_HEADER = 24;
static size_t kv_data_off(size_t n_tokens) { return (KV_HEADER + 4 * n_tokens + 63) / 64 * 64; }
static void put_u32(uint8_t* p, uint32_t v) {
  p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); p[2] = (uint8_t)(v >> 16); p[3] = (uint8_t)(v >> 24);
}
static uint32_t get_u32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

size_t aotcu_kv_blob_size(const aotcu_gpu* g, size_t n_tokens, size_t n_cached) {
  if (!g) return 0;
  const aotcu_dims& d = g->head.dims;
  n_cached = std::min(n_cached, n_tokens);
  return kv_data_off(n_tokens) + (size_t)d.n_layer * 2 * n_cached * ((size_t)d.n_kv_head * d.head_dim) * 4;
}

int aotcu_kv_save(aotcu_gpu* g, const uint32_t* tokens, size_t n_tokens, size_t n_cached, uint8_t* out, size_t out_cap,
                  size_t* out_len) {
  ARG_CHECK(g && out && out_len && (tokens || n_tokens == 0), "NULL argument");
  const aotcu_dims& d = g->head.dims;
  n_cached = std::min(n_cached, n_tokens);
  ARG_CHECK(n_cached <= g->n_ctx, "%zu cached positions exceed the context (%zu)", n_cached, g->n_ctx);
  ARG_CHECK(n_tokens <= 0xFFFFFFFFu, "too many tokens");
  const size_t kvd = (size_t)d.n_kv_head * d.head_dim, rows = n_cached * kvd;
  const size_t need = aotcu_kv_blob_size(g, n_tokens, n_cached);
  ARG_CHECK(out_cap >= need, "the blob needs %zu bytes, the buffer holds %zu", need, out_cap);
  if (int rc = ctx_set_device(g->c)) return rc;
  memcpy(out, "AOTP", 4);
  put_u32(out + 4, 2);
  put_u32(out + 8, (uint32_t)n_tokens);
  put_u32(out + 12, (uint32_t)d.n_layer);
  put_u32(out + 16, (uint32_t)kvd);
  put_u32(out + 20, (uint32_t)n_cached);
  for (size_t i = 0; i < n_tokens; i++) put_u32(out + KV_HEADER + 4 * i, tokens[i]);
  const size_t off = kv_data_off(n_tokens);
  memset(out + KV_HEADER + 4 * n_tokens, 0, off - (KV_HEADER + 4 * n_tokens));
  // device floats are little-endian IEEE words already: the rows go out as they are
  for (int l = 0; l < d.n_layer && rows; l++) {
    const size_t at = (size_t)l * g->n_ctx * kvd;
    CU_TRY(cudaMemcpyAsync(out + off + ((size_t)l * 2) * rows * 4, g->bufs[AOTCU_BUF_KCACHE] + at, rows * 4, cudaMemcpyDeviceToHost,
                           g->c->stream));
    CU_TRY(cudaMemcpyAsync(out + off + ((size_t)l * 2 + 1) * rows * 4, g->bufs[AOTCU_BUF_VCACHE] + at, rows * 4, cudaMemcpyDeviceToHost,
                           g->c->stream));
  }
  CU_TRY(cudaStreamSynchronize(g->c->stream));
  *out_len = need;
  return 0;
}

int aotcu_kv_load(aotcu_gpu* g, const uint8_t* blob, size_t blob_len, uint32_t* tokens_out, size_t tokens_cap,
                  size_t* n_tokens, size_t* n_cached) {
  ARG_CHECK(g && blob && n_tokens && n_cached && (tokens_out || tokens_cap == 0), "NULL argument");
  const aotcu_dims& d = g->head.dims;
  const size_t kvd = (size_t)d.n_kv_head * d.head_dim;
  ARG_CHECK(blob_len >= KV_HEADER && !memcmp(blob, "AOTP", 4), "not a saved KV cache (no AOTP header)");
  const uint32_t version = get_u32(blob + 4);
  ARG_CHECK(version == 1 || version == 2, "saved KV cache of unknown version %u", version);
  const size_t n = get_u32(blob + 8), nl = get_u32(blob + 12), kv = get_u32(blob + 16);
  const size_t nc = version == 1 ? n : get_u32(blob + 20);
  ARG_CHECK(nl == (size_t)d.n_layer && kv == kvd && n > 0 && nc <= n,
            "the saved KV cache is not of this model (layers %zu/%d, kv_dim %zu/%zu, tokens %zu, cached %zu)", nl, d.n_layer, kv, kvd, n, nc);
  ARG_CHECK(blob_len >= KV_HEADER + 4 * n, "saved KV cache is truncated");
  const size_t off = kv_data_off(n), rows = nc * kvd;
  ARG_CHECK(blob_len >= off + nl * 2 * rows * 4, "saved KV cache is truncated");
  ARG_CHECK(nc <= g->n_ctx, "the saved cache holds %zu positions, the context %zu", nc, g->n_ctx);
  if (int rc = ctx_set_device(g->c)) return rc;
  for (size_t l = 0; l < nl && rows; l++) {
    const size_t at = l * g->n_ctx * kvd;
    CU_TRY(cudaMemcpyAsync(g->bufs[AOTCU_BUF_KCACHE] + at, blob + off + (l * 2) * rows * 4, rows * 4, cudaMemcpyHostToDevice, g->c->stream));
    CU_TRY(cudaMemcpyAsync(g->bufs[AOTCU_BUF_VCACHE] + at, blob + off + (l * 2 + 1) * rows * 4, rows * 4, cudaMemcpyHostToDevice,
                           g->c->stream));
  }
  CU_TRY(cudaStreamSynchronize(g->c->stream));
  for (size_t i = 0; i < n && i < tokens_cap; i++) tokens_out[i] = get_u32(blob + KV_HEADER + 4 * i);
  *n_tokens = n;
  *n_cached = nc;
  return 0;
}

int aotcu_generate(aotcu_gpu* g, uint32_t token, size_t pos, size_t n_steps, uint32_t* out_tokens, float* elapsed_ms) {
  ARG_CHECK(g && out_tokens, "NULL argument");
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  const aotcu_dims& d = g->head.dims;
  ARG_CHECK(token < (uint32_t)d.vocab, "token id out of range");
  ARG_CHECK(pos + n_steps <= g->n_ctx, "positions exceed the context");
  ARG_CHECK(n_steps <= g->history_cap, "too many steps");
  if (n_steps == 0) return 0;
  aotcu_ctx* c = g->c;
  if (int rc = ctx_set_device(c)) return rc;
  if (int rc = set_step(g, token, pos, 0)) return rc;
  if (g->use_graph)
    for (int v = mega_split(g, pos); v <= mega_split(g, pos + n_steps - 1); v++) {
      g->split_now = v;
      if (!g->gen_graph[v])
        if (int rc = capture_graph(g, &g->gen_graph[v], &g->gen_graph_kernels[v], 1, true)) return rc;
    }
  cudaEvent_t e0, e1;
  CU_TRY(cudaEventCreate(&e0));
  CU_TRY(cudaEventCreate(&e1));
  CU_TRY(cudaEventRecord(e0, c->stream));
  for (size_t s = 0; s < n_steps; s++) {
    g->split_now = mega_split(g, pos + s);  // the device advances the position by one per step
    if (g->use_graph) {
      CU_TRY(cudaGraphLaunch(g->gen_graph[g->split_now], c->stream));
      c->launches += g->gen_graph_kernels[g->split_now];
    } else {
      if (int rc = enqueue_decode(g, 1, true)) return rc;
    }
  }
  CU_TRY(cudaEventRecord(e1, c->stream));
  CU_TRY(cudaMemcpyAsync(out_tokens, g->d_history, n_steps * sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  if (elapsed_ms) CU_TRY(cudaEventElapsedTime(elapsed_ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return check_device_errors(c);
}

int aotcu_tp_unique_id(const char* nccl_library, uint8_t out_id[128]) {
  ARG_CHECK(out_id, "NULL argument");
  TpState t;
  if (int rc = tp_load(&t, nccl_library)) return rc;
  NcclId id;
  const int r = t.get_unique_id(&id);
  if (r != 0) return fail(AOTCU_ERR_CUDA, "ncclGetUniqueId: %s", t.get_error_string(r));
  memcpy(out_id, id.bytes, 128);
  return 0;  // the library stays loaded
}


int aotcu_tp_inbox_handle(aotcu_gpu* g, uint8_t out_handle[64]) {
  ARG_CHECK(g && out_handle, "NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (int rc = ctx_set_device(g->c)) return rc;
  if (!g->tp_inbox) {
    const size_t words = (size_t)2 * TP_MAX_WORLD * g->head.dims.dim + 2 * TP_MAX_WORLD;  // partial rows, argmax slots
    CU_TRY(cudaMalloc(&g->tp_inbox, words * sizeof(LLWord)));
    CU_TRY(cudaMemset(g->tp_inbox, 0, words * sizeof(LLWord)));
  }
  cudaIpcMemHandle_t h;
  CU_TRY(cudaIpcGetMemHandle(&h, g->tp_inbox));
  memcpy(out_handle, &h, 64);
  return 0;
}

int aotcu_tp_attach(aotcu_gpu* g, const char* nccl_library, int rank, int world, const uint8_t id[128],
                    const uint8_t* peer_handles) {
  ARG_CHECK(g && id, "NULL argument");
  ARG_CHECK(world >= 1 && world <= TP_MAX_WORLD && rank >= 0 && rank < world, "bad rank %d of %d (at most %d ranks)", rank,
            world, TP_MAX_WORLD);
  ARG_CHECK(!g->tp, "this Gpu already belongs to a tensor-parallel group");
  if (int rc = ctx_set_device(g->c)) return rc;
  CU_TRY(cudaStreamSynchronize(g->c->stream));
  const aotcu_tensor& out_t = g->head.output.present ? g->head.output : g->head.token_embd;
  const size_t vocab = (size_t)g->head.dims.vocab;
  ARG_CHECK((size_t)out_t.rows == vocab || (size_t)out_t.rows * world == vocab,
            "the output head has %zu rows: neither the vocabulary (%zu) nor one of %d equal slices", (size_t)out_t.rows, vocab, world);
  if ((size_t)out_t.rows != vocab) {
    g->head_sharded = true;
    g->head_row0 = (size_t)rank * out_t.rows;
    CU_TRY(cudaMalloc(&g->tp_logits_full, vocab * sizeof(float)));
  }
  // Peers' inboxes first, the (blocking, collective) communicator second: once any rank is
  // back from this call, every rank has mapped every inbox.
  const bool fused = world > 1 && peer_handles && g->tp_inbox && g->mega_ok;
  if (fused) {
    TpExchange& x = g->step_params.tp;
    x.world = world;
    x.rank = rank;
    x.dim = g->head.dims.dim;
    x.head_sharded = g->head_sharded ? 1 : 0;
    x.head_row0 = (int)g->head_row0;
    x.arg_off = 2 * TP_MAX_WORLD * x.dim;
    for (int r = 0; r < world; r++) {
      if (r == rank) {
        x.inbox[r] = g->tp_inbox;
        continue;
      }
      cudaIpcMemHandle_t h;
      memcpy(&h, peer_handles + (size_t)r * 64, 64);
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
      g->tp_peer_map[r] = p;
      x.inbox[r] = reinterpret_cast<LLWord*>(p);
    }
    // ranks step together: bound the waits at about half a minute instead of two seconds
    g->step_params.spin_limit = 1 << 25;
    // every rank counts launches from the same value, so tags agree across GPUs
    const unsigned one = 1;
    CU_TRY(cudaMemcpy(g->d_grid_bar + 1, &one, sizeof(unsigned), cudaMemcpyHostToDevice));
  }
  TpState* t = new TpState();
  t->rank = rank;
  t->world = world;
  if (world > 1) {
    if (int rc = tp_load(t, nccl_library)) {
      delete t;
      return rc;
    }
    NcclId nid;
    memcpy(nid.bytes, id, 128);
    const int r = t->comm_init_rank(&t->comm, world, nid, rank);
    if (r != 0) {
      int rc = fail(AOTCU_ERR_CUDA, "ncclCommInitRank: %s", t->get_error_string(r));
      delete t;
      return rc;
    }
  }
  drop_graphs(g);
  g->tp = t;
  // Without mapped inboxes the one-kernel step has no exchange between ranks: the sharded
  // model then takes the per-operator path with NCCL all-reduces.
  if (world > 1 && !fused) g->mega_ok = false;
  return 0;
}

uint64_t aotcu_gpu_dispatches(aotcu_gpu* g) { return g ? g->c->launches : 0; }

int aotcu_gpu_set_option(aotcu_gpu* g, const char* name, int value) {
  ARG_CHECK(g && name, "NULL argument");
  if (!strcmp(name, "graph")) {
    g->use_graph = value != 0;
    return 0;
  }
  if (!strcmp(name, "prepared_operands")) {
    // 0: prompt chunks unpack the weights in every launch; 1 (default): Q4_K / Q5_K layer
    // matrices are expanded once into tensor-core operand tiles when memory allows
    CU_TRY(cudaStreamSynchronize(g->c->stream));
    if (!value) {
      for (auto& kv : g->prep) cudaFree(kv.second);
      g->prep.clear();
      g->prep_state = -1;
    } else if (g->prep_state == -1) {
      g->prep_state = 0;
    }
    return 0;
  }
  if (!strcmp(name, "prepared_bytes")) {  // query: bytes held by the prepared operands
    size_t total = 0;
    for (const auto& l : g->layers) {
      const aotcu_tensor* c7[7] = {&l.wq, &l.wk, &l.wv, &l.wo, &l.gate, &l.up, &l.down};
      for (auto t : c7)
        if (g->prep.count(t->off)) total += tc_prep_bytes(t->rows, t->cols);
    }
    return (int)std::min<size_t>(total >> 20, 0x7fffffff);  // MiB
  }
  if (!strcmp(name, "mega")) {
    if (value && !g->mega_ok) return fail(AOTCU_ERR_UNSUPPORTED, "this model cannot use the one-kernel decode step");
    if (g->use_mega != (value != 0)) {
      CU_TRY(cudaStreamSynchronize(g->c->stream));
      drop_graphs(g);
    }
    g->use_mega = value != 0;
    return 0;
  }
  if (!strcmp(name, "mega_available")) return g->mega_ok ? 1 : 0;
  if (!strcmp(name, "wide_rows")) {  // process-wide: rows per CTA from which single-row products use one lane per super-block
    ARG_CHECK(value >= 1, "wide_rows must be at least 1");
    g_wide_rows = value;
    return 0;
  }
  if (!strcmp(name, "q80_chunks")) {  // process-wide: Q4_0 / Q5_0 / Q8_0 products on the chunk-streaming kernel (1, default)
    g_q80_chunks = value != 0;
    return 0;
  }
  if (!strcmp(name, "wide_multi_work")) {  // process-wide: see launch_gemv
    ARG_CHECK(value >= 0, "wide_multi_work must not be negative");
    g_wide_multi_work = value;
    return 0;
  }
  if (!strcmp(name, "wide_multi")) {  // process-wide: K-quant prompt chunks of few tiles (and Q6_K) on gemv_stream_kernel<3> (1, default)
    g_wide_multi = value != 0;
    return 0;
  }
  if (!strcmp(name, "float_rows4")) {  // process-wide: four weight rows per lane in the float chunk kernel at 9..16 activation rows (1, default)
    g_float_rows4 = value != 0;
    return 0;
  }
  if (!strcmp(name, "float_chunks")) {  // process-wide: F16 / BF16 / F32 products on the chunk-streaming kernel (1, default)
    g_float_chunks = value != 0;
    return 0;
  }
  if (!strcmp(name, "q80_rows_per_lane")) {  // process-wide: 0 by shape, 1 or 2 forced (single activation row, no pair)
    ARG_CHECK(value >= 0 && value <= 2, "q80_rows_per_lane is 0, 1 or 2");
    g_q80_rows_per_lane = value;
    return 0;
  }
  if (!strcmp(name, "tc_gemm")) {
    // process-wide: prompt chunks of Q4_K / Q5_K matrices on tcgen05 (2: always, 1: when the
    // launch has enough 128-row tiles to occupy the GPU) or on mma.sync tiles (0)
    g_use_tc = value != 0;
    g_tc_force = value >= 2 ? 1 : 0;
    return 0;
  }
  if (!strcmp(name, "fast") || !strcmp(name, "exact") || !strcmp(name, "spin_limit")) {
    // Parameters of the one-kernel step are baked into the captured graphs: drop them.
    CU_TRY(cudaStreamSynchronize(g->c->stream));
    drop_graphs(g);
    if (!strcmp(name, "spin_limit")) {
      ARG_CHECK(value >= 1, "spin_limit must be at least 1");
      g->step_params.spin_limit = value;
    } else if (!strcmp(name, "fast")) {
      ARG_CHECK(value >= 0 && value <= 3, "fast is a mask of bits 1 and 2");
      g->step_params.fast = value;
    } else {
      g->step_params.fast = value ? 0 : 3;
    }
    return 0;
  }
  if (!strcmp(name, "pdl")) {
    if (g->c->pdl != (value != 0)) {
      // Captured graphs bake the launch attributes in; drop them.
      CU_TRY(cudaStreamSynchronize(g->c->stream));
      drop_graphs(g);
    }
    g->c->pdl = value != 0;
    return 0;
  }
  return fail(AOTCU_ERR_BAD_ARG, "unknown option %s", name);
}


// Times only the matrix products of one decode step (q/k/v, wo, gate/up, down of every
// layer, then the output head), back to back in one CUDA graph, `iters` replays. The
// layers' weights are distinct and together far larger than L2, so every launch
// streams from HBM. Used by the benchmark to quote the GEMV kernel's bandwidth.
int aotcu_bench_matmul(aotcu_ctx* c, int kind, float* out, const uint8_t* w, size_t copy_stride, size_t n_copies,
                       const void* xs, size_t m, size_t rows, size_t cols, int iters, float* ms_per_launch) {
  ARG_CHECK(c && out && w && xs && ms_per_launch, "NULL argument");
  ARG_CHECK(iters >= 1 && n_copies >= 1 && m >= 1, "iters, n_copies and m must be at least 1");
  if (int rc = ctx_set_device(c)) return rc;
  auto one = [&](int i) -> int {
    const uint8_t* wi = w + (size_t)(i % (int)n_copies) * copy_stride;
    return m == 1 ? aotcu_matvec(c, kind, out, wi, xs, rows, cols) : aotcu_matmul(c, kind, out, wi, xs, m, rows, cols);
  };
  for (int i = 0; i < 3; i++)
    if (int rc = one(i)) return rc;
  cudaEvent_t e0, e1;
  CU_TRY(cudaEventCreate(&e0));
  CU_TRY(cudaEventCreate(&e1));
  // iters == 1 times one launch alone: the stream is drained first, so nothing of a
  // predecessor overlaps it (no dependent-launch overlap, cold pipeline)
  if (iters == 1) CU_TRY(cudaStreamSynchronize(c->stream));
  CU_TRY(cudaEventRecord(e0, c->stream));
  int rc = 0;
  for (int i = 0; i < iters && !rc; i++) rc = one(i + 3);
  cudaEventRecord(e1, c->stream);
  cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0.0f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "bench_matmul: %s", cudaGetErrorString(e));
  *ms_per_launch = ms / (float)iters;
  return check_device_errors(c);
}

int aotcu_bench_gemv_sweep(aotcu_gpu* g, int iters, float* ms_per_sweep, uint64_t* launches_per_sweep,
                           uint64_t* bytes_per_sweep) {
  ARG_CHECK(g && iters >= 1 && ms_per_sweep, "bad argument");
  aotcu_ctx* c = g->c;
  const aotcu_dims& d = g->head.dims;
  if (int rc = ctx_set_device(c)) return rc;
  uint64_t bytes = 0;
  auto tensor_bytes = [&](const aotcu_tensor& t) { bytes += t.len + 4 * t.cols + 4 * t.rows; };
  auto one = [&](const aotcu_tensor& t, float* dst) -> int {
    ARG_CHECK(kind_act(t.kind) == ACT_Q8_K, "the sweep handles K-quant matrices only");
    GemvCall call;
    call.seg[0] = GemvSeg{wptr(g, t), dst, (int)t.rows, t.kind};
    call.cols = t.cols;
    call.x = g->aqk;
    call.x_mode = 1;
    tensor_bytes(t);
    return launch_gemv(c, call);
  };
  CU_TRY(cudaMemsetAsync(g->aqk, 0, (xb_width(d) > (size_t)d.hidden ? xb_width(d) : (size_t)d.hidden) / 256 * XIMG_K, c->stream));
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t before = c->launches;
  CU_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  int rc = 0;
  for (int li = 0; li < d.n_layer && !rc; li++) {
    const aotcu_layer& l = g->layers[li];
    GemvCall qkv;
    qkv.nseg = 3;
    const aotcu_tensor* w3[3] = {&l.wq, &l.wk, &l.wv};
    float* o3[3] = {g->bufs[AOTCU_BUF_Q], g->bufs[AOTCU_BUF_K], g->bufs[AOTCU_BUF_V]};
    for (int i = 0; i < 3; i++) {
      if (kind_act(w3[i]->kind) != ACT_Q8_K) rc = fail(AOTCU_ERR_UNSUPPORTED, "the sweep handles K-quant matrices only");
      qkv.seg[i] = GemvSeg{wptr(g, *w3[i]), o3[i], (int)w3[i]->rows, w3[i]->kind};
      tensor_bytes(*w3[i]);
    }
    qkv.cols = l.wq.cols;
    qkv.x = g->aqk;
    qkv.x_mode = 1;
    if (!rc) rc = launch_gemv(c, qkv);
    if (!rc) rc = one(l.wo, g->bufs[AOTCU_BUF_XB2]);
    if (!rc) {
      GemvCall gu;
      gu.seg[0] = GemvSeg{wptr(g, l.gate), g->bufs[AOTCU_BUF_HB], (int)l.gate.rows, l.gate.kind};
      gu.seg[1] = GemvSeg{wptr(g, l.up), g->bufs[AOTCU_BUF_HB2], (int)l.up.rows, l.up.kind};
      gu.nseg = 2;
      gu.pair = l.gate.kind == l.up.kind ? 1 : 0;
      gu.cols = l.gate.cols;
      gu.x = g->aqk;
      gu.x_mode = 1;
      gu.epilogue = gu.pair ? EPI_SILU_MUL : EPI_STORE;
      tensor_bytes(l.gate);
      tensor_bytes(l.up);
      if (kind_act(l.gate.kind) != ACT_Q8_K || kind_act(l.up.kind) != ACT_Q8_K) rc = fail(AOTCU_ERR_UNSUPPORTED, "the sweep handles K-quant matrices only");
      if (!rc) rc = launch_gemv(c, gu);
    }
    if (!rc) rc = one(l.down, g->bufs[AOTCU_BUF_XB2]);
  }
  if (!rc) rc = one(g->head.output.present ? g->head.output : g->head.token_embd, g->bufs[AOTCU_BUF_LOGITS]);
  cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
  uint64_t n_launch = c->launches - before;
  c->launches = before;
  if (rc) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (int i = 0; i < 2; i++) cudaGraphLaunch(exec, c->stream);  // warm-up
  cudaEventRecord(e0, c->stream);
  for (int i = 0; i < iters; i++) cudaGraphLaunch(exec, c->stream);
  cudaEventRecord(e1, c->stream);
  e = cudaStreamSynchronize(c->stream);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaGraphExecDestroy(exec);
  if (e != cudaSuccess) return fail(AOTCU_ERR_CUDA, "gemv sweep: %s", cudaGetErrorString(e));
  c->launches += n_launch * (uint64_t)(iters + 2);
  *ms_per_sweep = ms / (float)iters;
  if (launches_per_sweep) *launches_per_sweep = n_launch;
  if (bytes_per_sweep) *bytes_per_sweep = bytes;
  g->qsrc = aotcu_gpu::QSrc();
  return check_device_errors(c);
}


// Runs one decode step of the one-kernel path with phase timestamps: out[0..15] are the
// SM cycles CTA `cta` spent in each phase, summed over layers (0 embed, 1 attn norm,
// 2 q/k/v, 3 barrier, 4 attention, 5 barrier, 6 quantize, 7 wo, 8 barrier, 9 ffn norm,
// 10 gate/up, 11 barrier, 12 quantize, 13 down, 14 barrier, 15 head).
int aotcu_gpu_profile_step(aotcu_gpu* g, uint32_t token, size_t pos, int cta, uint64_t out[32]) {
  ARG_CHECK(g && out, "NULL argument");
  g->h_logits_fresh = false;  // anything but aotcu_forward may change the logits behind the host copy
  ARG_CHECK(g->mega_ok, "this model cannot use the one-kernel decode step");
  ARG_CHECK(token < (uint32_t)g->head.dims.vocab && pos < g->n_ctx, "token or position out of range");
  aotcu_ctx* c = g->c;
  if (int rc = ctx_set_device(c)) return rc;
  unsigned long long* d = nullptr;
  CU_TRY(cudaMalloc(&d, 32 * sizeof(unsigned long long)));
  CU_TRY(cudaMemsetAsync(d, 0, 32 * sizeof(unsigned long long), c->stream));
  int rc = set_step(g, token, pos, 0);
  g->split_now = mega_split(g, pos);
  if (!rc) rc = enqueue_mega(g, 1, false, d, cta);
  if (!rc) rc = check_device_errors(c);
  if (!rc) {
    cudaError_t e = cudaMemcpy(out, d, 32 * sizeof(uint64_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail(AOTCU_ERR_CUDA, "profile copy: %s", cudaGetErrorString(e));
  }
  cudaFree(d);
  return rc;
}


}  // extern "C"

extern "C" int aotcu_gpu_timeline_step(aotcu_gpu* g, uint32_t token, size_t pos, int layer, uint64_t* out, int* n_cta) {
  ARG_CHECK(g && out && n_cta, "NULL argument");
  g->h_logits_fresh = false;
  ARG_CHECK(g->mega_ok, "this model cannot use the one-kernel decode step");
  ARG_CHECK(token < (uint32_t)g->head.dims.vocab && pos < g->n_ctx, "token or position out of range");
  ARG_CHECK(layer >= 0 && layer < g->head.dims.n_layer && g->c->n_sm <= 256, "layer out of range");
  aotcu_ctx* c = g->c;
  if (int rc = ctx_set_device(c)) return rc;
  const size_t bytes = (size_t)c->n_sm * 16 * sizeof(unsigned long long);
  unsigned long long* d = nullptr;
  CU_TRY(cudaMalloc(&d, bytes));
  CU_TRY(cudaMemsetAsync(d, 0, bytes, c->stream));
  int rc = set_step(g, token, pos, 0);
  g->split_now = mega_split(g, pos);
  if (!rc) rc = enqueue_mega(g, 1, false, nullptr, 0, d, layer);
  if (!rc) rc = check_device_errors(c);
  if (!rc) {
    cudaError_t e = cudaMemcpy(out, d, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail(AOTCU_ERR_CUDA, "timeline copy: %s", cudaGetErrorString(e));
  }
  cudaFree(d);
  *n_cta = c->n_sm;
  return rc;
}

// ---- a matrix-vector product for callers that may not allocate ---------------------------
// The f32 activation vector has to be quantized to Q8_K block images before the product
// can run, and those images need somewhere to live. The ordinary route
// (aotcu_quantize_q8_k into a buffer from aotcu_malloc, then aotcu_matvec_*) makes the
// caller own that buffer. Here the images go into a fixed array inside the library's
// device image instead: every GPU that loads the library carries these 19,456 bytes until
// the process exits, and in exchange the call below never asks the CUDA allocator for
// anything.
constexpr size_t STATIC_MAX_COLS = 16384;  // 64 super-blocks
static __device__ __align__(256) uint8_t g_static_xq[(STATIC_MAX_COLS / 256) * XIMG_K];

// In host code `g_static_xq` is only a handle for the runtime, not a device address. The
// address is looked up once per device, with that device current, and cached here.
constexpr int STATIC_MAX_DEVICES = 64;
static uint8_t* g_static_xq_addr[STATIC_MAX_DEVICES] = {};

extern "C" int aotcu_matvec_k_static(aotcu_ctx* c, int kind, float* out, const uint8_t* w, const float* x,
                                     size_t rows, size_t cols) {
  ARG_CHECK(c && out && w && x, "NULL argument");
  ARG_CHECK(kind == AOTCU_Q4_K || kind == AOTCU_Q5_K || kind == AOTCU_Q6_K, "kind %d is not a K-quant", kind);
  ARG_CHECK(cols > 0 && cols % 256 == 0, "cols (%zu) must be a positive multiple of 256", cols);
  ARG_CHECK(cols <= STATIC_MAX_COLS,
            "cols (%zu) exceeds the %zu columns the built-in activation area holds; use aotcu_quantize_q8_k + "
            "aotcu_matvec with a buffer of your own",
            cols, STATIC_MAX_COLS);
  ARG_CHECK(c->device >= 0 && c->device < STATIC_MAX_DEVICES, "device index %d out of range", c->device);
  if (rows == 0) return 0;
  if (int rc = ctx_set_device(c)) return rc;
  uint8_t* xq = g_static_xq_addr[c->device];
  if (!xq) {
    // First call on this device: resolve the array's device address.
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_xq);
    if (e != cudaSuccess || !p)
      return fail(AOTCU_ERR_CUDA, "cudaGetSymbolAddress(g_static_xq): %s", cudaGetErrorString(e));
    xq = g_static_xq_addr[c->device] = static_cast<uint8_t*>(p);
  }
  const int nblk = (int)(cols / 256);
  // Every block image of the vector is rewritten in full, so nothing left by an earlier
  // call is read.
  if (int rc = launch(c, quantize_q8k_kernel, dim3(grid_for(c, nblk, 8)), dim3(256), 0, x, xq, nblk, 1)) return rc;
  GemvCall call;
  call.seg[0] = GemvSeg{w, out, (int)rows, kind};
  call.nseg = 1;
  call.cols = cols;
  call.x = xq;
  call.x_mode = 1;
  call.m = 1;
  return launch_gemv(c, call);
}
