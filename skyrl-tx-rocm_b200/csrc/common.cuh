// Host-side helpers shared by the translation units of the C-ABI library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/skyrl_w8a8_sm100.h"

namespace skyrl {

// Records the message returned by skyrl_w8a8_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// cuTensorMapEncodeTiled resolved through the runtime (no link-time libcuda
// dependency, so the library loads on a machine without a driver).
// 2-D / 3-D row-major tensors, 128-byte swizzle, zero fill out of bounds.
int encode_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer);
int encode_tmap_3d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0,
                   uint32_t box1, uint32_t box2 = 1);

int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Kernel launch, optionally with programmatic stream serialization (see pdl_wait / pdl_trigger): the
// kernel may then begin, up to its pdl_wait, before the previous kernel of the stream has finished.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool programmatic, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The opt-in to more than 48 KB of dynamic shared memory is an attribute of the function PER DEVICE
// (a single process may drive several GPUs, as an XLA host does): `done` is the caller's
// function-local `static bool[MAX_DEVICES]`, indexed by the current device.  A benign race only
// repeats the idempotent call.
constexpr int MAX_DEVICES = 64;
template <typename Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, bool (&done)[MAX_DEVICES]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= MAX_DEVICES) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[dev] = true;
  return e;
}
#endif

// kernel launchers implemented in the .cu files
// `zero_words` (nullable): `zero_count` int32 words the routing kernel clears (the workspace's tile-claim counters).
int launch_route(const int32_t* ids, int m, int num_adapters, int32_t* perm, int32_t* tiles, int32_t* num_tiles,
                 int max_tiles, int32_t* status, cudaStream_t stream, int chunk_rows = 0, int chunk_cap = 0,
                 int32_t* zero_words = nullptr, int zero_count = 0);
int launch_grad_quant(const void* dy, int64_t dy_row_stride, const float* col_scale, const int32_t* row_map, int m, int n,
                      void* q1, float* s1, void* q2, float* s2, cudaStream_t stream);
int launch_rms_quant(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* row_map,
                     int m, int k, void* xq, float* sx, void* xn, cudaStream_t stream);
// rows [m, k] contiguous (row pitch k) with their absmax known: codes and scales in one streaming pass
int launch_quant_stream(const void* x, const float* row_amax, int m, int k, void* xq, float* sx, cudaStream_t stream);
int launch_lora_a_proj(const void* x, int m, int k, const void* a_packed, const float* scaling, int num_adapters,
                       int rank, const int32_t* tiles, const int32_t* num_tiles, int max_tiles, void* z_parts,
                       int32_t* status, cudaStream_t stream, int row_lo = 0, int row_hi = -1,
                       void* const* extra_dests = nullptr, int extra_count = 0, int list_row0 = -1);  // extra copies of the rows written
// Tile width and K split the GEMM launcher chooses for a shape (deterministic per device).
struct GemmPlan {
  int bn_eff;
  int k_splits;
  int kb_per_split;
};
GemmPlan plan_gemm(int m, int n, int k, int epilogue, int max_slabs);
constexpr int MAX_SPLIT_K_SLABS = 16;
int launch_gemm(const SkyrlW8A8GemmArgs& a, cudaStream_t stream, bool programmatic = false);
// `programmatic`: launch with programmatic stream serialization (small-batch chain of short kernels)
// Adapter ids outside [0, num_adapters) are clamped and STATUS_BAD_ADAPTER_ID is recorded in `status`.
int launch_rms_quant_rows(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* ids,
                          int num_adapters, const void* a_packed, const float* scaling, int rank, int m, int k, void* xq,
                          float* sx, float* z_rows, int32_t* status, cudaStream_t stream, bool programmatic = false,
                          void* xn_out = nullptr);  // xn_out: optional bf16 [m, k] copy of the normalised rows
int launch_finalize_rows(int epilogue, const int32_t* acc, int slabs, const float* sx, const float* sw, const float* z_rows,
                         const int32_t* ids, int num_adapters, const void* b_table, int64_t b_adapter_stride,
                         int b_row_stride, int rank, int m, int n, const void* residual, int64_t res_stride, void* out,
                         int64_t out_stride, int32_t* status, cudaStream_t stream, bool programmatic = false);
int launch_tp_finalize(const float* reduced, const int32_t* perm, const void* residual, void* out, int hidden,
                       int row_begin, int row_count, cudaStream_t stream, bool out_sorted = false);
int launch_tp_finalize_slabs(const float* const* slabs, int num_slabs, const int32_t* perm, const void* residual,
                             void* out, int hidden, int row_begin, int row_count, cudaStream_t stream, bool out_sorted);
// Tensor-parallel exchange between two blocks (tp_exchange_sm100.cu).
struct TpExchangeLaunch {
  int tp;
  const float* partial[8];
  int row_begin, row_count, hidden;
  const int32_t* perm;
  const void* residual;
  void* out;
  bool out_sorted;
  bool quantize;
  const void* delta;
  float eps;
  int8_t* xq_dst[8];
  float* sx_dst[8];
  void* xn;
  const int32_t* wait_flags;
  int32_t wait_value;
  int32_t* status;
  int grid_ctas;
  bool profile;        // CTA 0 of the two-launch kernels adds its wait / sum / quantiser times to status[1..3]
  bool wide;           // two-launch form as many small CTAs on all SMs instead of fat CTAs on the spare ones
  bool multimem;       // partial[0] is a multicast address: the sum over ranks is one multimem.ld_reduce per vector
  bool single_kernel;  // true: one kernel sums, finalizes and quantises row by row; false: a streaming sum kernel, then the row-wise one
};
int launch_tp_exchange(const TpExchangeLaunch& a, cudaStream_t stream);
int launch_tp_signal(int32_t* const* flags, int count, int32_t value, cudaStream_t stream);
int launch_tp_wait(const int32_t* flags, int count, int32_t value, int32_t* status, cudaStream_t stream);
int launch_unsort_rows(const void* sorted_rows, const int32_t* perm, void* out, int m, int hidden, cudaStream_t stream);

}  // namespace skyrl
