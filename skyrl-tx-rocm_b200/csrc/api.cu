// Host side of the C ABI: error reporting, TMA descriptor encoding and the
// operator entry points that chain the stage kernels on the caller's stream.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace skyrl {

static thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

static int encode(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides, const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(SKYRL_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SKYRL_ERR_INVALID_ARGUMENT, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SKYRL_OK;
}

int encode_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer) {
  (void)elem_bytes;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  return encode(map, dtype, 2, base, dims, strides, box);
}

int encode_tmap_3d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0,
                   uint32_t box1, uint32_t box2) {
  (void)elem_bytes;
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
  const cuuint32_t box[3] = {box0, box1, box2};
  return encode(map, dtype, 3, base, dims, strides, box);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- workspace carving -------------------------------------------------------
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int MAX_CHUNKS = 16;
constexpr int SCHED_WORDS = 8;  // room for four {claimed, finished} pairs of the GEMMs' dynamic tile scheduler

// Tiles one chunk of `rows` sorted rows can hold: every adapter may end a partial tile inside it.
static inline int tile_cap(int rows, int num_adapters) {
  return (rows + SKYRL_TILE_ROWS - 1) / SKYRL_TILE_ROWS + (num_adapters > 0 ? num_adapters : 1) + 1;
}
static inline int max_tiles_for(int m, int num_adapters) { return tile_cap(m, num_adapters); }
// Capacity of the tile buffer: the unchunked list, or MAX_CHUNKS per-chunk lists, whichever is larger.
static inline size_t tile_buffer_slots(int m, int num_adapters) {
  const size_t whole = static_cast<size_t>(max_tiles_for(m, num_adapters));
  const size_t chunked = static_cast<size_t>(m) / SKYRL_TILE_ROWS + 2 * MAX_CHUNKS +
                         static_cast<size_t>(MAX_CHUNKS) * ((num_adapters > 0 ? num_adapters : 1) + 1);
  return whole > chunked ? whole : chunked;
}

struct Carver {
  unsigned char* base;
  size_t off = 0;
  explicit Carver(void* b) : base(static_cast<unsigned char*>(b)) {}
  template <typename T>
  T* take(size_t count) {
    off = align_up(off, 1024);
    T* p = base != nullptr ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
  size_t total() const { return align_up(off, 1024); }
};

// Batches of at most this many rows take the row-wise LoRA path (no adapter sort, one M tile).
constexpr int ROWS_PATH_MAX_M = SKYRL_TILE_ROWS;

struct LinearWs {
  int32_t* perm;
  int32_t* tiles;
  int32_t* num_tiles;
  int8_t* xq;
  float* sx;
  uint16_t* xn;
  uint16_t* z_parts;  // bf16 [m, 6, 64]; the row-wise path keeps fp32 [m, 64] here instead
  int32_t* acc;       // int32 [m, n] accumulator, row-wise path only
  int32_t* sched;     // tile-claim counters of the GEMM launch (zeroed by the routing kernel, left at zero by the GEMM)
  size_t bytes;
};

static LinearWs carve_linear(void* ws, int m, int n, int k, int num_adapters) {
  Carver c(ws);
  LinearWs w;
  const int mt = max_tiles_for(m, num_adapters);
  w.perm = c.take<int32_t>(m);
  w.tiles = c.take<int32_t>(4 * static_cast<size_t>(mt));
  w.num_tiles = c.take<int32_t>(4);
  w.sched = c.take<int32_t>(SCHED_WORDS);
  w.xq = c.take<int8_t>(static_cast<size_t>(m) * k);
  w.sx = c.take<float>(m);
  w.z_parts = c.take<uint16_t>(SKYRL_Z_PARTS * static_cast<size_t>(m) * SKYRL_LORA_RANK_PAD);
  if (m <= ROWS_PATH_MAX_M) {
    w.xn = nullptr;
    w.acc = c.take<int32_t>(static_cast<size_t>(m) * n * plan_gemm(m, n, k, SKYRL_EPI_ACC_I32, MAX_SPLIT_K_SLABS).k_splits);
  } else {
    w.xn = c.take<uint16_t>(static_cast<size_t>(m) * k);
    w.acc = nullptr;
  }
  w.bytes = c.total();
  return w;
}

struct MlpWs {
  int32_t* perm;
  int32_t* tiles;
  int32_t* num_tiles;
  int8_t* xq;
  float* sx;
  uint16_t* xn;
  uint16_t* z_parts;
  uint16_t* h;
  int8_t* hq;
  float* sh;
  int32_t* acc;  // int32 [m, max(2I, H)] accumulator, row-wise path only
  float* h_amax; // fp32 [m]: absmax of every row of h, collected by the gate_up epilogue
  int32_t* sched; // tile-claim counters: words 0-1 gate_up GEMM, 2-3 down GEMM, 4-7 the same for odd chunks (zeroed by the routing kernel)
  size_t bytes;
};

static MlpWs carve_mlp(void* ws, int m, int hidden, int inter, int num_adapters) {
  Carver c(ws);
  MlpWs w;
  const int mt = max_tiles_for(m, num_adapters);
  w.perm = c.take<int32_t>(m);
  (void)mt;
  w.tiles = c.take<int32_t>(4 * tile_buffer_slots(m, num_adapters));
  w.num_tiles = c.take<int32_t>(MAX_CHUNKS + 4);
  w.sched = c.take<int32_t>(SCHED_WORDS);
  w.xq = c.take<int8_t>(static_cast<size_t>(m) * hidden);
  w.sx = c.take<float>(m);
  w.z_parts = c.take<uint16_t>(SKYRL_Z_PARTS * static_cast<size_t>(m) * SKYRL_LORA_RANK_PAD);
  w.h = c.take<uint16_t>(static_cast<size_t>(m) * inter);
  w.hq = c.take<int8_t>(static_cast<size_t>(m) * inter);
  w.sh = c.take<float>(m);
  w.xn = c.take<uint16_t>(static_cast<size_t>(m) * hidden);
  if (m <= ROWS_PATH_MAX_M) {
    const size_t gu = static_cast<size_t>(m) * 2 * inter *
                      plan_gemm(m, 2 * inter, hidden, SKYRL_EPI_ACC_I32, MAX_SPLIT_K_SLABS).k_splits;
    const size_t dn = static_cast<size_t>(m) * hidden *
                      plan_gemm(m, hidden, inter, SKYRL_EPI_ACC_I32, MAX_SPLIT_K_SLABS).k_splits;
    w.acc = c.take<int32_t>(gu > dn ? gu : dn);
  } else {
    w.acc = nullptr;
  }
  w.h_amax = c.take<float>(m);
  w.bytes = c.total();
  return w;
}

static int check_ws(const void* ws, size_t have, size_t need, const char* who) {
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 1023u) != 0)
    return fail(SKYRL_ERR_WORKSPACE, "%s: workspace must be non-null and 1024-byte aligned", who);
  if (have < need) return fail(SKYRL_ERR_WORKSPACE, "%s: workspace has %zu bytes, needs %zu", who, have, need);
  return SKYRL_OK;
}

// One W8A8 LoRA projection on rows that are already laid out as the GEMM wants them.
//   tensor-core route (m > 128): rows adapter-sorted, z planes from lora_a_proj, LoRA inside the GEMM epilogue
//   row-wise route (m <= 128): rows in token order; the GEMM leaves the int32 accumulator in global
//   memory (split over K when that fills the GPU better) and a row-wise kernel applies scales, LoRA,
//   the cast and the SwiGLU / residual step
struct Projection {
  const void* x;          // bf16 [m, k] source rows
  int64_t x_stride;
  const void* rms_delta;  // nullable
  float eps;
  const int32_t* gather;  // row gather for the quantiser (sorted route) or NULL
  bool keep_xn;           // sorted route: x must be re-laid out (gathered / normalised) for the projection MMA
  int m, n, k, rank, na, mt;
  int q_row0, q_rows;     // sorted rows the quantiser stage covers (a chunk of the block, or all m rows)
  int list_row0;          // first sorted row of the tile list `tiles` (0, or the first row of the call's chunk)
  bool skip_quant;        // the quantiser stage of these rows already ran (its outputs are in xq / sx / z_parts)
  int gemm_variant;       // SKYRL_GEMM_VARIANT_* forced on the GEMM (0: the library chooses)
  bool two_step_rows;     // row-wise route: GEMM to an int32 accumulator in memory + finalize kernel (default)
  const float* known_amax;  // absmax of every source row, if the producer of x collected it (sorted route)
  float* row_amax;          // SwiGLU epilogue: collect the absmax of every output row here
  int cta_limit;
  void* const* scatter_bases;  // row scatter of the fp32 partial sums (see SkyrlW8A8GemmArgs) or NULL
  int scatter_row0, scatter_rows;

  const void* wq;
  const float* sw;
  const void* a_packed;
  const void* b_packed;
  const void* b_rows;     // dense [A, n, b_rows_rank] LoRA-B table for the row-wise route, or NULL
  int b_rows_rank;
  const float* scaling;
  const int32_t* ids;     // token-order adapter ids (row-wise route)
  int8_t* xq;
  float* sx;
  uint16_t* xn;
  uint16_t* z_parts;
  int32_t* acc;
  const int32_t* tiles;
  const int32_t* num_tiles;
  int epilogue;
  const int32_t* out_row_map;
  const void* residual;
  int64_t residual_stride;
  void* out;
  int64_t out_stride;
  int32_t* status;
  int32_t* sched;         // {claimed, finished} words of the GEMM launch inside the caller's workspace
  const void* prefetch;   // row-wise route: bytes the GEMM asks into L2 after its own loads (the next GEMM's weights)
  int64_t prefetch_bytes;
  void* ev_begin;
  void* ev_end;
};

// Quantiser stage of the sorted route for rows [q_row0, q_row0 + q_rows): RMSNorm + int8 codes + scales
// (+ the normalised bf16 rows the LoRA-A projection reads), then the LoRA-A projection of those rows.
static int run_quant_stage(const Projection& q, cudaStream_t stream) {
  const bool lora = q.rank > 0;
  const bool need_xn = lora && q.keep_xn;
  const int r0 = q.q_row0, rows = q.q_rows > 0 ? q.q_rows : q.m;
  int rc;
  // a gather reads rows perm[r0 ...] of x; without one the chunk's rows are rows r0 ... of x itself
  const unsigned char* xsrc = static_cast<const unsigned char*>(q.x) +
                              (q.gather != nullptr ? 0 : static_cast<size_t>(r0) * q.x_stride * 2);
  if (q.known_amax != nullptr && q.rms_delta == nullptr && q.gather == nullptr && !need_xn && q.x_stride == q.k) {
    // the rows' absmax came with them: one streaming pass
    if ((rc = launch_quant_stream(xsrc, q.known_amax + r0, rows, q.k, q.xq + static_cast<size_t>(r0) * q.k, q.sx + r0,
                                  stream)))
      return rc;
  } else if ((rc = launch_rms_quant(xsrc, q.x_stride, q.rms_delta, q.eps,
                                    q.gather != nullptr ? q.gather + r0 : nullptr, rows, q.k,
                                    q.xq + static_cast<size_t>(r0) * q.k, q.sx + r0,
                                    need_xn ? q.xn + static_cast<size_t>(r0) * q.k : nullptr, stream))) {
    return rc;
  }
  if (lora) {
    const void* xa = need_xn ? static_cast<const void*>(q.xn) : q.x;
    if ((rc = launch_lora_a_proj(xa, q.m, q.k, q.a_packed, q.scaling, q.na, q.rank, q.tiles, q.num_tiles, q.mt,
                                 q.z_parts, q.status, stream, r0, r0 + rows, nullptr, 0, q.list_row0)))
      return rc;
  }
  return SKYRL_OK;
}

static int run_projection(const Projection& q, cudaStream_t stream) {
  const bool lora = q.rank > 0;
  const bool rows_path = q.m <= ROWS_PATH_MAX_M;
  int rc;
  SkyrlW8A8GemmArgs g = {};
  if (rows_path && lora && q.epilogue != SKYRL_EPI_ACC_I32) {
    float* z_rows = reinterpret_cast<float*>(q.z_parts);
    if ((rc = launch_rms_quant_rows(q.x, q.x_stride, q.rms_delta, q.eps, q.ids, q.na, q.a_packed, q.scaling, q.rank, q.m,
                                    q.k, q.xq, q.sx, z_rows, q.status, stream, true, q.keep_xn ? q.xn : nullptr)))
      return rc;
    const bool dense = q.b_rows != nullptr;
    const int brow = dense ? q.b_rows_rank : SKYRL_LORA_RANK_PAD;
    // timing events between the launches would cut the programmatic chain: use ordinary launches then
    const bool chain = q.ev_begin == nullptr && q.ev_end == nullptr;
    g.struct_size = sizeof(g);
    g.m = q.m;
    g.n = q.n;
    g.k = q.k;
    g.num_adapters = q.na;
    g.max_tiles = q.mt;
    g.xq = q.xq;
    g.sx = q.sx;
    g.wq = q.wq;
    g.sw = q.sw;
    g.tiles = q.tiles;
    g.num_tiles = q.num_tiles;
    g.status = q.status;
    g.sched = q.sched;
    g.prefetch = q.prefetch;
    g.prefetch_bytes = q.prefetch_bytes;
    if (!q.two_step_rows) {
      // one kernel: the GEMM's epilogue warps evaluate the per-row LoRA term while the weights stream and apply
      // scales, LoRA, the cast and the SwiGLU / residual step from tensor memory
      g.epilogue = q.epilogue;
      g.rank = q.rank;
      g.z_rows = z_rows;
      g.row_adapter_ids = q.ids;
      g.lora_b_rows = dense ? q.b_rows : q.b_packed;
      g.lora_b_rows_rank = brow;
      g.residual = q.residual;
      g.residual_row_stride = q.residual_stride;
      g.out = q.out;
      g.out_row_stride = q.out_stride;
      if (q.ev_begin != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_begin), stream);
      rc = launch_gemm(g, stream, chain);
      if (q.ev_end != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_end), stream);
      return rc;
    }
    // two steps (the default: faster at decode shapes): int32 accumulator to global memory, split over K when
    // that fills the GPU better, then a row-wise kernel run by a whole grid
    const int slabs = plan_gemm(q.m, q.n, q.k, SKYRL_EPI_ACC_I32, MAX_SPLIT_K_SLABS).k_splits;
    g.epilogue = SKYRL_EPI_ACC_I32;
    g.split_k_slabs = MAX_SPLIT_K_SLABS;
    g.rank = 0;
    g.out = q.acc;
    g.out_row_stride = q.n;
    if (q.ev_begin != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_begin), stream);
    rc = launch_gemm(g, stream, chain);
    if (q.ev_end != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_end), stream);
    if (rc) return rc;
    return launch_finalize_rows(q.epilogue, q.acc, slabs, q.sx, q.sw, z_rows, q.ids, q.na,
                                dense ? q.b_rows : q.b_packed, static_cast<int64_t>(q.n) * brow, brow, q.rank, q.m, q.n,
                                q.residual, q.residual_stride, q.out, q.out_stride, q.status, stream, chain);
  }
  {
    if (!q.skip_quant && (rc = run_quant_stage(q, stream))) return rc;
    g.rank = q.rank;
    g.z_parts = lora ? q.z_parts : nullptr;
  }
  g.struct_size = sizeof(g);
  g.epilogue = q.epilogue;
  g.m = q.m;
  g.n = q.n;
  g.k = q.k;
  g.num_adapters = q.na;
  g.max_tiles = q.mt;
  g.xq = q.xq;
  g.sx = q.sx;
  g.wq = q.wq;
  g.sw = q.sw;
  g.lora_b_packed = q.b_packed;
  g.tiles = q.tiles;
  g.num_tiles = q.num_tiles;
  g.out_row_map = q.out_row_map;
  g.residual = q.residual;
  g.out = q.out;
  g.out_row_stride = q.out_stride;
  g.residual_row_stride = q.residual_stride;
  g.status = q.status;
  g.sched = q.sched;
  g.variant = q.gemm_variant;
  g.cta_limit = q.cta_limit;
  if (q.row_amax != nullptr && q.epilogue == SKYRL_EPI_SWIGLU) {
    const int r0 = q.q_row0, rows = q.q_rows > 0 ? q.q_rows : q.m;
    cudaError_t e = cudaMemsetAsync(q.row_amax + r0, 0, static_cast<size_t>(rows) * sizeof(float), stream);
    if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "row_amax memset: %s", cudaGetErrorString(e));
    g.row_amax = q.row_amax;
  }
  if (q.scatter_bases != nullptr && q.scatter_rows > 0) {
    for (int o = 0; o < 8; ++o) g.scatter_bases[o] = q.scatter_bases[o];
    g.scatter_row0 = q.scatter_row0;
    g.scatter_rows = q.scatter_rows;
  }
  if (q.ev_begin != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_begin), stream);
  rc = launch_gemm(g, stream);
  if (q.ev_end != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(q.ev_end), stream);
  return rc;
}

}  // namespace skyrl

using namespace skyrl;

extern "C" int skyrl_w8a8_abi_version(void) { return SKYRL_W8A8_ABI_VERSION; }
extern "C" const char* skyrl_w8a8_last_error(void) { return g_last_error; }

extern "C" size_t skyrl_w8a8_linear_workspace_bytes(int32_t m, int32_t n, int32_t k, int32_t num_adapters) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  return carve_linear(nullptr, m, n, k, num_adapters).bytes;
}

extern "C" size_t skyrl_w8a8_mlp_workspace_bytes(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters) {
  if (m <= 0 || hidden <= 0 || inter <= 0) return 0;
  return carve_mlp(nullptr, m, hidden, inter, num_adapters).bytes;
}

extern "C" int skyrl_w8a8_lora_forward_sm100_v1(const SkyrlW8A8LinearArgs* a, skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: args is null");
  if (a->struct_size != sizeof(SkyrlW8A8LinearArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: struct_size %u does not match ABI v%d (%zu)", a->struct_size,
                SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8LinearArgs));
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: non-positive shape");
  if (a->x == nullptr || a->wq == nullptr || a->sw == nullptr || a->out == nullptr || a->status == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: null buffer");
  if (a->rank < 0 || a->rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "linear: LoRA rank must be in [0, %d], got %d", SKYRL_LORA_RANK_PAD, a->rank);
  const bool lora = a->rank > 0;
  if (lora && (a->lora_a_packed == nullptr || a->lora_b_packed == nullptr || a->lora_scaling == nullptr ||
               a->num_adapters <= 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: LoRA tables missing");
  if (a->adapter_ids != nullptr && a->num_adapters <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "linear: adapter ids given without adapters");
  const int na = a->num_adapters > 0 ? a->num_adapters : 1;
  const LinearWs w = carve_linear(a->workspace, a->m, a->n, a->k, na);
  int rc = check_ws(a->workspace, a->workspace_bytes, w.bytes, "linear");
  if (rc) return rc;
  const int mt = max_tiles_for(a->m, na);
  const bool rows_path = a->m <= ROWS_PATH_MAX_M;
  const bool routed = a->adapter_ids != nullptr && !rows_path;

  if ((rc = launch_route(routed ? a->adapter_ids : nullptr, a->m, na, w.perm, w.tiles, w.num_tiles, mt, a->status,
                         stream, 0, 0, w.sched, SCHED_WORDS)))
    return rc;
  Projection q = {};
  q.x = a->x;
  q.x_stride = a->x_row_stride;
  q.rms_delta = a->rms_delta;
  q.eps = a->rms_eps;
  q.gather = routed ? w.perm : nullptr;
  q.keep_xn = routed || a->rms_delta != nullptr || a->x_row_stride != a->k;
  q.two_step_rows = (a->flags & SKYRL_LINEAR_FUSED_ROWS) == 0;
  q.gemm_variant = static_cast<int>((a->flags >> SKYRL_FLAGS_GEMM_VARIANT_SHIFT) & 7u);
  q.m = a->m;
  q.n = a->n;
  q.k = a->k;
  q.rank = a->rank;
  q.na = na;
  q.mt = mt;
  q.wq = a->wq;
  q.sw = a->sw;
  q.a_packed = a->lora_a_packed;
  q.b_packed = a->lora_b_packed;
  q.scaling = a->lora_scaling;
  q.ids = a->adapter_ids;
  q.xq = w.xq;
  q.sx = w.sx;
  q.xn = w.xn;
  q.z_parts = w.z_parts;
  q.acc = w.acc;
  q.b_rows = a->lora_b_rows;
  q.b_rows_rank = a->lora_b_rows_rank;
  q.tiles = w.tiles;
  q.num_tiles = w.num_tiles;
  q.epilogue = a->epilogue;
  q.out_row_map = routed ? w.perm : nullptr;
  q.residual = a->residual;
  q.residual_stride = a->residual_row_stride;
  q.out = a->out;
  q.out_stride = a->out_row_stride;
  q.status = a->status;
  q.sched = w.sched;
  q.ev_begin = a->timing_events[0];
  q.ev_end = a->timing_events[1];
  return run_projection(q, stream);
}

// One exported target per fused variant: thin wrappers that check what the variant needs and fix the epilogue.
extern "C" int skyrl_rms_gate_up_w8a8_lora_swiglu_sm100_v1(const SkyrlW8A8LinearArgs* a, skyrl_stream_t stream) {
  if (a == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_gate_up_swiglu: args is null");
  if (a->struct_size != sizeof(SkyrlW8A8LinearArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_gate_up_swiglu: struct_size %u does not match ABI v%d (%zu)",
                a->struct_size, SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8LinearArgs));
  if (a->residual != nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_gate_up_swiglu: takes no residual");
  if (a->n % 2 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_gate_up_swiglu: n must count (gate, up) pairs");
  SkyrlW8A8LinearArgs b = *a;
  b.epilogue = SKYRL_EPI_SWIGLU;
  return skyrl_w8a8_lora_forward_sm100_v1(&b, stream);
}

extern "C" int skyrl_down_w8a8_lora_residual_sm100_v1(const SkyrlW8A8LinearArgs* a, skyrl_stream_t stream) {
  if (a == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "down_residual: args is null");
  if (a->struct_size != sizeof(SkyrlW8A8LinearArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "down_residual: struct_size %u does not match ABI v%d (%zu)",
                a->struct_size, SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8LinearArgs));
  if (a->residual == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "down_residual: residual is null");
  if (a->rms_delta != nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "down_residual: takes no RMSNorm weights");
  SkyrlW8A8LinearArgs b = *a;
  b.epilogue = SKYRL_EPI_RESIDUAL;
  return skyrl_w8a8_lora_forward_sm100_v1(&b, stream);
}

namespace skyrl {

// What one MLP call works on: the carved workspace and the chunk of sorted rows with its tile list.
struct MlpPlan {
  MlpWs w;
  int na;
  bool rows_path, routed, chunked;
  const int32_t* perm;
  int chunk_rows, chunk_cap, mt, row0, rows;
  const int32_t* tiles;
  const int32_t* num_tiles;
};

static int plan_mlp(const SkyrlW8A8MlpArgs* a, const char* who, MlpPlan* pl) {
  if (a == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: args is null", who);
  if (a->struct_size != sizeof(SkyrlW8A8MlpArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: struct_size %u does not match ABI v%d (%zu)", who, a->struct_size,
                SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8MlpArgs));
  if (a->m <= 0 || a->hidden <= 0 || a->inter <= 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: non-positive shape", who);
  if (a->x == nullptr || a->gu_wq == nullptr || a->gu_sw == nullptr || a->dn_wq == nullptr || a->dn_sw == nullptr ||
      a->out == nullptr || a->status == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: null buffer", who);
  if (a->down_epilogue != SKYRL_EPI_RESIDUAL && a->down_epilogue != SKYRL_EPI_PARTIAL_F32 &&
      a->down_epilogue != SKYRL_EPI_LINEAR)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: down_epilogue must be RESIDUAL, LINEAR or PARTIAL_F32", who);
  if (a->rank < 0 || a->rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "%s: LoRA rank must be in [0, %d], got %d", who, SKYRL_LORA_RANK_PAD, a->rank);
  const bool lora = a->rank > 0;
  if (lora && (a->gu_a_packed == nullptr || a->gu_b_packed == nullptr || a->gu_scaling == nullptr ||
               a->dn_a_packed == nullptr || a->dn_b_packed == nullptr || a->dn_scaling == nullptr ||
               a->num_adapters <= 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: LoRA tables missing", who);
  pl->na = a->num_adapters > 0 ? a->num_adapters : 1;
  pl->w = carve_mlp(a->workspace, a->m, a->hidden, a->inter, pl->na);
  int rc = check_ws(a->workspace, a->workspace_bytes, pl->w.bytes, who);
  if (rc) return rc;
  pl->rows_path = a->m <= ROWS_PATH_MAX_M;
  pl->routed = a->adapter_ids != nullptr && !pl->rows_path;
  pl->perm = pl->routed ? pl->w.perm : nullptr;
  pl->chunked = a->num_chunks > 1 && !pl->rows_path;
  if (pl->chunked && (a->num_chunks > MAX_CHUNKS || a->chunk_index < 0 || a->chunk_index >= a->num_chunks))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "%s: num_chunks must be <= %d and chunk_index inside it", who, MAX_CHUNKS);
  pl->chunk_rows = pl->chunked ? ((a->m + a->num_chunks - 1) / a->num_chunks + SKYRL_TILE_ROWS - 1) / SKYRL_TILE_ROWS *
                                     SKYRL_TILE_ROWS
                               : 0;
  pl->chunk_cap = pl->chunked ? tile_cap(pl->chunk_rows, pl->na) : 0;
  pl->mt = pl->chunked ? pl->chunk_cap : max_tiles_for(a->m, pl->na);
  pl->row0 = pl->chunked ? a->chunk_index * pl->chunk_rows : 0;
  pl->rows = pl->chunked ? (a->m - pl->row0 < pl->chunk_rows ? a->m - pl->row0 : pl->chunk_rows) : a->m;
  pl->tiles = pl->chunked ? pl->w.tiles + 4 * static_cast<size_t>(a->chunk_index) * pl->chunk_cap : pl->w.tiles;
  pl->num_tiles = pl->chunked ? pl->w.num_tiles + a->chunk_index : pl->w.num_tiles;
  return SKYRL_OK;
}

static int route_mlp(const SkyrlW8A8MlpArgs* a, const MlpPlan& pl, cudaStream_t stream) {
  if ((a->flags & SKYRL_MLP_REUSE_ROUTING) != 0) return SKYRL_OK;
  return launch_route(pl.routed ? a->adapter_ids : nullptr, a->m, pl.na, pl.w.perm, pl.w.tiles, pl.w.num_tiles,
                      static_cast<int>(tile_buffer_slots(a->m, pl.na)), a->status, stream, pl.chunk_rows, pl.chunk_cap,
                      pl.w.sched, SCHED_WORDS);
}

// front half: RMSNorm -> quant -> gate_up W8A8 LoRA -> SwiGLU; h keeps the row order of the GEMM
static Projection front_projection(const SkyrlW8A8MlpArgs* a, const MlpPlan& pl) {
  const MlpWs& w = pl.w;
  Projection q = {};
  q.x = a->x;
  q.x_stride = a->hidden;
  q.rms_delta = a->rms_delta;
  q.eps = a->rms_eps;
  q.gather = pl.perm;
  // small batches need no re-laid-out copy of x; they write one only when asked to (stage checks)
  q.keep_xn = pl.rows_path ? (a->flags & SKYRL_MLP_KEEP_NORMALIZED) != 0 : (pl.routed || a->rms_delta != nullptr);
  q.two_step_rows = (a->flags & SKYRL_MLP_FUSED_ROWS) == 0;
  q.gemm_variant = static_cast<int>((a->flags >> SKYRL_FLAGS_GEMM_VARIANT_SHIFT) & 7u);
  q.m = a->m;
  q.n = 2 * a->inter;
  q.k = a->hidden;
  q.rank = a->rank;
  q.na = pl.na;
  q.mt = pl.mt;
  q.q_row0 = pl.row0;
  q.q_rows = pl.rows;
  q.list_row0 = pl.row0;
  q.cta_limit = a->gemm_cta_limit;
  q.wq = a->gu_wq;
  q.sw = a->gu_sw;
  q.a_packed = a->gu_a_packed;
  q.b_packed = a->gu_b_packed;
  q.scaling = a->gu_scaling;
  q.ids = a->adapter_ids;
  q.xq = w.xq;
  q.sx = w.sx;
  q.xn = w.xn;
  q.z_parts = w.z_parts;
  q.acc = w.acc;
  q.b_rows = a->gu_b_rows;
  q.b_rows_rank = a->b_rows_rank;
  q.tiles = pl.tiles;
  q.num_tiles = pl.num_tiles;
  q.epilogue = SKYRL_EPI_SWIGLU;
  q.out_row_map = nullptr;
  q.out = w.h;
  q.out_stride = a->inter;
  q.status = a->status;
  // odd and even chunks claim tiles through counter pairs of their own, so that two chunks of one block may run
  // on two streams at the same time
  q.sched = w.sched + (pl.chunked ? (a->chunk_index & 1) * 4 : 0);
  q.ev_begin = a->timing_events[0];
  q.ev_end = a->timing_events[1];
  return q;
}

}  // namespace skyrl

extern "C" int skyrl_w8a8_mlp_block_sm100_v1(const SkyrlW8A8MlpArgs* a, skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MlpPlan pl;
  int rc = plan_mlp(a, "mlp", &pl);
  if (rc) return rc;
  if (pl.rows <= 0) return SKYRL_OK;  // more chunks than rows: nothing to do for this one
  const bool prepared = (a->flags & SKYRL_MLP_INPUT_PREPARED) != 0;
  if (prepared && pl.rows_path)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "mlp: SKYRL_MLP_INPUT_PREPARED needs more than %d rows", ROWS_PATH_MAX_M);
  if ((rc = route_mlp(a, pl, stream))) return rc;
  const MlpWs& w = pl.w;

  Projection q = front_projection(a, pl);
  q.skip_quant = prepared;
  // sorted route: the gate_up epilogue collects the absmax of every row of h, so that quantising h is one
  // streaming pass (SKYRL_MLP_NO_ROW_AMAX keeps the two-pass quantiser; the two must agree bit for bit)
  const bool collect = !pl.rows_path && (a->flags & SKYRL_MLP_NO_ROW_AMAX) == 0;
  q.row_amax = collect ? w.h_amax : nullptr;
  if (pl.rows_path && a->prefetch_down_bytes > 0) {
    // the down weights travel to L2 while the row-wise kernels behind gate_up run
    const int64_t dn_bytes = static_cast<int64_t>((a->inter + SKYRL_WEIGHT_KBLOCK - 1) / SKYRL_WEIGHT_KBLOCK) * a->hidden * SKYRL_WEIGHT_KBLOCK;
    q.prefetch = a->dn_wq;
    q.prefetch_bytes = (a->prefetch_down_bytes < dn_bytes ? a->prefetch_down_bytes : dn_bytes) / 16 * 16;
  }
  if ((rc = run_projection(q, stream))) return rc;

  // back half: quant(h) -> down W8A8 LoRA -> + residual, rows scattered back to token order
  q.skip_quant = false;
  q.row_amax = nullptr;
  q.known_amax = collect ? w.h_amax : nullptr;
  q.x = w.h;
  q.x_stride = a->inter;
  q.rms_delta = nullptr;
  q.gather = nullptr;
  q.keep_xn = false;
  q.n = a->hidden;
  q.k = a->inter;
  q.wq = a->dn_wq;
  q.sw = a->dn_sw;
  q.a_packed = a->dn_a_packed;
  q.b_packed = a->dn_b_packed;
  q.b_rows = a->dn_b_rows;
  q.scaling = a->dn_scaling;
  q.xq = w.hq;
  q.sx = w.sh;
  q.sched += 2;
  q.prefetch = nullptr;
  q.prefetch_bytes = 0;
  if (pl.rows_path && a->prefetch_next != nullptr && a->prefetch_next_bytes > 0) {
    q.prefetch = a->prefetch_next;
    q.prefetch_bytes = a->prefetch_next_bytes;
  }
  q.epilogue = a->down_epilogue;
  q.out_row_map = a->down_epilogue == SKYRL_EPI_PARTIAL_F32 ? nullptr : pl.perm;
  q.residual = a->residual != nullptr ? a->residual : a->x;
  q.residual_stride = a->hidden;
  q.out = a->out;
  q.out_stride = a->hidden;
  if (a->tp_scatter_rows > 0) {
    if (a->down_epilogue != SKYRL_EPI_PARTIAL_F32 || pl.rows_path)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "mlp: tp_scatter_rows needs down_epilogue PARTIAL_F32 and more than %d rows",
                  ROWS_PATH_MAX_M);
    q.scatter_bases = a->tp_scatter_bases;
    q.scatter_row0 = pl.row0;
    q.scatter_rows = a->tp_scatter_rows;
  }
  q.ev_begin = a->timing_events[2];
  q.ev_end = a->timing_events[3];
  return run_projection(q, stream);
}

extern "C" int skyrl_w8a8_mlp_tp_prepare_sm100_v1(const SkyrlW8A8MlpArgs* a, int32_t row_begin, int32_t row_count,
                                                   skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MlpPlan pl;
  int rc = plan_mlp(a, "tp_prepare", &pl);
  if (rc) return rc;
  if (pl.rows_path)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_prepare: needs more than %d rows", ROWS_PATH_MAX_M);
  if (row_count <= 0 || row_begin < pl.row0 || row_begin + row_count > pl.row0 + pl.rows)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_prepare: rows [%d, %d) are not inside chunk rows [%d, %d)", row_begin,
                row_begin + row_count, pl.row0, pl.row0 + pl.rows);
  if ((rc = route_mlp(a, pl, stream))) return rc;
  Projection q = front_projection(a, pl);
  q.q_row0 = row_begin;
  q.q_rows = row_count;
  return run_quant_stage(q, stream);
}

extern "C" int skyrl_w8a8_mlp_workspace_regions(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters,
                                                 size_t* offsets) {
  if (m <= 0 || hidden <= 0 || inter <= 0 || offsets == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "workspace_regions: bad argument");
  unsigned char* const base = reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(1024));
  const MlpWs w = carve_mlp(base, m, hidden, inter, num_adapters > 0 ? num_adapters : 1);
  offsets[0] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.xq) - base);
  offsets[1] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.sx) - base);
  offsets[2] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.z_parts) - base);
  return SKYRL_OK;
}

extern "C" int skyrl_w8a8_tp_signal_sm100_v1(int32_t* const* flags, int32_t count, int32_t value, skyrl_stream_t stream) {
  return launch_tp_signal(flags, count, value, static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_w8a8_tp_wait_sm100_v1(const int32_t* flags, int32_t count, int32_t value, int32_t* status,
                                            skyrl_stream_t stream) {
  return launch_tp_wait(flags, count, value, status, static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_w8a8_mlp_tp_exchange_sm100_v1(const SkyrlW8A8MlpArgs* blk, const SkyrlW8A8MlpArgs* next,
                                                    const SkyrlW8A8TpExchangeArgs* x, skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (x == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: exchange args are null");
  if (x->struct_size != sizeof(SkyrlW8A8TpExchangeArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: struct_size %u does not match ABI v%d (%zu)", x->struct_size,
                SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8TpExchangeArgs));
  if (x->tp < 1 || x->tp > 8) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: tp must be in [1, 8], got %d", x->tp);
  if (x->out == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: out is null");
  MlpPlan pl;
  int rc = plan_mlp(blk, "tp_exchange", &pl);
  if (rc) return rc;
  if (pl.rows_path) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: needs more than %d rows", ROWS_PATH_MAX_M);
  if (x->row_count <= 0 || x->row_begin < 0 || x->row_begin + x->row_count > blk->m)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: rows [%d, %d) are outside [0, %d)", x->row_begin,
                x->row_begin + x->row_count, blk->m);
  TpExchangeLaunch e = {};
  e.tp = x->tp;
  for (int s = 0; s < x->tp; ++s) e.partial[s] = x->partials[s];
  e.row_begin = x->row_begin;
  e.row_count = x->row_count;
  e.hidden = blk->hidden;
  e.perm = pl.perm;
  e.residual = blk->residual != nullptr ? blk->residual : blk->x;
  e.out = x->out;
  e.out_sorted = (blk->flags & SKYRL_MLP_FINALIZE_SORTED) != 0;
  e.wait_flags = x->wait_flags;
  e.wait_value = x->wait_value;
  e.status = blk->status;
  if (static_cast<int64_t>(blk->m) * (blk->hidden >> 3) > 0x7fffffffLL)
    return fail(SKYRL_ERR_UNSUPPORTED, "tp_exchange: m * hidden / 8 must fit 31 bits");
  e.grid_ctas = x->grid_ctas;
  e.single_kernel = (x->flags & SKYRL_TP_EXCHANGE_SINGLE_KERNEL) != 0;
  e.multimem = (x->flags & SKYRL_TP_EXCHANGE_MULTIMEM) != 0;
  e.profile = (x->flags & SKYRL_TP_EXCHANGE_PROFILE) != 0;
  e.wide = (x->flags & SKYRL_TP_EXCHANGE_WIDE) != 0;
  MlpPlan np;
  const bool lora = next != nullptr && next->rank > 0;
  if (next != nullptr) {
    if ((rc = plan_mlp(next, "tp_exchange (next block)", &np))) return rc;
    if (next->m != blk->m || next->hidden != blk->hidden)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: the next block has another shape");
    if (x->row_begin < np.row0 || x->row_begin + x->row_count > np.row0 + np.rows)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: rows [%d, %d) are not inside the next block's chunk [%d, %d)",
                  x->row_begin, x->row_begin + x->row_count, np.row0, np.row0 + np.rows);
    unsigned char* const local = static_cast<unsigned char*>(next->workspace);
    const size_t off_xq = reinterpret_cast<unsigned char*>(np.w.xq) - local;
    const size_t off_sx = reinterpret_cast<unsigned char*>(np.w.sx) - local;
    e.quantize = true;
    e.delta = next->rms_delta;
    e.eps = next->rms_eps;
    e.xn = np.w.xn;  // the LoRA-A projection reads it; without LoRA it is still the scratch of the warp-per-row quantiser
    for (int r = 0; r < x->tp; ++r) {
      if (x->peer_workspaces[r] == nullptr || (reinterpret_cast<uintptr_t>(x->peer_workspaces[r]) & 1023u) != 0)
        return fail(SKYRL_ERR_WORKSPACE, "tp_exchange: workspace of rank %d is null or not 1024-byte aligned", r);
      unsigned char* const base = static_cast<unsigned char*>(x->peer_workspaces[r]);
      e.xq_dst[r] = reinterpret_cast<int8_t*>(base + off_xq);
      e.sx_dst[r] = reinterpret_cast<float*>(base + off_sx);
    }
  }
  if ((rc = launch_tp_exchange(e, stream))) return rc;
  if (lora) {
    // LoRA-A projection of the rows just normalised, its parts stored into every rank's workspace
    unsigned char* const local = static_cast<unsigned char*>(next->workspace);
    const size_t off_z = reinterpret_cast<unsigned char*>(np.w.z_parts) - local;
    void* extra[8];
    int extra_count = 0;
    for (int r = 0; r < x->tp; ++r) {
      void* dst = static_cast<unsigned char*>(x->peer_workspaces[r]) + off_z;
      if (dst != static_cast<void*>(np.w.z_parts)) extra[extra_count++] = dst;
    }
    if (extra_count > 7) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: this rank's workspace is not among peer_workspaces");
    if ((rc = launch_lora_a_proj(np.w.xn, next->m, next->hidden, next->gu_a_packed, next->gu_scaling, np.na, next->rank,
                                 np.tiles, np.num_tiles, np.mt, np.w.z_parts, next->status, stream, x->row_begin,
                                 x->row_begin + x->row_count, extra, extra_count, np.row0)))
      return rc;
  }
  bool any = false;
  for (int r = 0; r < x->tp; ++r) any = any || x->signal_flags[r] != nullptr;
  if (any) return launch_tp_signal(x->signal_flags, x->tp, x->signal_value, stream);
  return SKYRL_OK;
}

extern "C" int skyrl_w8a8_mlp_workspace_stage_regions(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters,
                                                       size_t* offsets) {
  if (m <= 0 || hidden <= 0 || inter <= 0 || offsets == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "workspace_stage_regions: bad argument");
  unsigned char* const base = reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(1024));
  const MlpWs w = carve_mlp(base, m, hidden, inter, num_adapters > 0 ? num_adapters : 1);
  offsets[0] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.perm) - base);
  offsets[1] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.h) - base);
  offsets[2] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.hq) - base);
  offsets[3] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.sh) - base);
  offsets[4] = static_cast<size_t>(reinterpret_cast<unsigned char*>(w.xn) - base);
  return SKYRL_OK;
}

extern "C" int skyrl_w8a8_mlp_tp_unsort_sm100_v1(const SkyrlW8A8MlpArgs* a, const void* sorted_rows, void* out,
                                                  skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MlpPlan pl;
  int rc = plan_mlp(a, "tp_unsort", &pl);
  if (rc) return rc;
  return launch_unsort_rows(sorted_rows, pl.perm, out, a->m, a->hidden, stream);
}

extern "C" int skyrl_w8a8_mlp_tp_finalize_sm100_v1(const SkyrlW8A8MlpArgs* a, const float* reduced, void* out,
                                                    int32_t row_begin, int32_t row_count, skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || reduced == nullptr || out == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize: null argument");
  if (a->struct_size != sizeof(SkyrlW8A8MlpArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize: struct_size does not match ABI v%d", SKYRL_W8A8_ABI_VERSION);
  if (a->m <= 0 || a->hidden <= 0 || a->hidden % 8 != 0 || row_begin < 0 || row_count <= 0 ||
      row_begin + row_count > a->m)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize: bad shape or row range");
  const int na = a->num_adapters > 0 ? a->num_adapters : 1;
  const MlpWs w = carve_mlp(a->workspace, a->m, a->hidden, a->inter, na);
  int rc = check_ws(a->workspace, a->workspace_bytes, w.bytes, "tp_finalize");
  if (rc) return rc;
  const void* residual = a->residual != nullptr ? a->residual : a->x;
  const bool routed = a->adapter_ids != nullptr && a->m > ROWS_PATH_MAX_M;
  return launch_tp_finalize(reduced, routed ? w.perm : nullptr, residual, out, a->hidden, row_begin, row_count, stream,
                            (a->flags & SKYRL_MLP_FINALIZE_SORTED) != 0);
}

extern "C" int skyrl_w8a8_mlp_tp_finalize_slabs_sm100_v1(const SkyrlW8A8MlpArgs* a, const float* const* slabs,
                                                          int32_t num_slabs, void* out, int32_t row_begin,
                                                          int32_t row_count, skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || slabs == nullptr || out == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: null argument");
  if (a->struct_size != sizeof(SkyrlW8A8MlpArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: struct_size does not match ABI v%d",
                SKYRL_W8A8_ABI_VERSION);
  if (a->m <= 0 || a->hidden <= 0 || a->hidden % 8 != 0 || row_begin < 0 || row_count <= 0 ||
      row_begin + row_count > a->m)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: bad shape or row range");
  const int na = a->num_adapters > 0 ? a->num_adapters : 1;
  const MlpWs w = carve_mlp(a->workspace, a->m, a->hidden, a->inter, na);
  int rc = check_ws(a->workspace, a->workspace_bytes, w.bytes, "tp_finalize_slabs");
  if (rc) return rc;
  const void* residual = a->residual != nullptr ? a->residual : a->x;
  const bool routed = a->adapter_ids != nullptr && a->m > ROWS_PATH_MAX_M;
  return launch_tp_finalize_slabs(slabs, num_slabs, routed ? w.perm : nullptr, residual, out, a->hidden, row_begin,
                                  row_count, stream, (a->flags & SKYRL_MLP_FINALIZE_SORTED) != 0);
}

// ---------------------------------------------------------------------------
// W8A8 LoRA linear without a caller workspace: the scratch is a fixed array in
// this library's device image.  `g_noalloc_scratch` below is, in host code, only
// a handle for the symbol; the address kernels can use is looked up once per
// device with cudaGetSymbolAddress and cached.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[SKYRL_NOALLOC_SCRATCH_BYTES];

namespace skyrl {

static int noalloc_scratch(unsigned char** base, size_t* bytes) {
  static std::mutex mu;
  static unsigned char* cached[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return fail(SKYRL_ERR_LAUNCH, "noalloc: no current CUDA device (%s)", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // address of the array on the CURRENT device
    if (e != cudaSuccess || p == nullptr)
      return fail(SKYRL_ERR_LAUNCH, "noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    cached[dev] = static_cast<unsigned char*>(p);
  }
  // the operator carves its scratch on 1024-byte boundaries; the array is only 256-byte aligned
  const uintptr_t raw = reinterpret_cast<uintptr_t>(cached[dev]);
  const uintptr_t aligned = (raw + 1023u) & ~static_cast<uintptr_t>(1023u);
  *base = reinterpret_cast<unsigned char*>(aligned);
  *bytes = SKYRL_NOALLOC_SCRATCH_BYTES - static_cast<size_t>(aligned - raw);
  return SKYRL_OK;
}

}  // namespace skyrl

extern "C" int skyrl_w8a8_lora_forward_noalloc_sm100_v1(const SkyrlW8A8LinearArgs* a, skyrl_stream_t stream_) {
  if (a == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "noalloc linear: args is null");
  if (a->struct_size != sizeof(SkyrlW8A8LinearArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "noalloc linear: struct_size %u does not match ABI v%d (%zu)",
                a->struct_size, SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8LinearArgs));
  if (a->m <= 0 || a->n <= 0 || a->k <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "noalloc linear: non-positive shape");
  unsigned char* base = nullptr;
  size_t avail = 0;
  int rc = noalloc_scratch(&base, &avail);
  if (rc) return rc;
  const int na = a->num_adapters > 0 ? a->num_adapters : 1;
  const LinearWs w = carve_linear(base, a->m, a->n, a->k, na);
  if (w.bytes > avail)
    return fail(SKYRL_ERR_WORKSPACE,
                "noalloc linear: m=%d, n=%d, k=%d needs %zu bytes of scratch, the built-in array holds %zu "
                "(SKYRL_NOALLOC_SCRATCH_BYTES = %u); use skyrl_w8a8_lora_forward_sm100_v1 with a workspace",
                a->m, a->n, a->k, w.bytes, avail, SKYRL_NOALLOC_SCRATCH_BYTES);
  // The array keeps the previous call's contents.  Nothing in it is accumulated into, but the
  // tile count is cleared so that a failed routing pass can never expose a stale count.
  cudaError_t e = cudaMemsetAsync(w.num_tiles, 0, 4 * sizeof(int32_t), static_cast<cudaStream_t>(stream_));
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "noalloc linear: memset: %s", cudaGetErrorString(e));
  SkyrlW8A8LinearArgs b = *a;
  b.workspace = base;
  b.workspace_bytes = avail;
  return skyrl_w8a8_lora_forward_sm100_v1(&b, stream_);
}
