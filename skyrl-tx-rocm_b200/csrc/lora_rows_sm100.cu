// Row-wise kernels for small batches (decode shapes: a few dozen token rows,
// almost every row with its own adapter).  Sorting rows by adapter and spending
// one 128-row tensor-core tile per adapter would multiply the weight traffic by
// the number of adapters, so here every row carries its adapter id:
//
//   rms_quant_rows_kernel<R> ... a cluster of 8 CTAs per token row: RMSNorm, absmax, int8 codes and
//                                z[m, :] = s[a] * (n[m, :] @ A[a]); every CTA owns one eighth of K and
//                                the row-wide reductions go through distributed shared memory (two exchanges)
//   finalize_rows_kernel<EPI> .. v = (f32(acc) * sx[m]) * sw[n] + sum_j z[m, j] * B[a(m)][n, j], then the
//                                single bf16 cast and SwiGLU / residual, from the int32 accumulator the
//                                GEMM left in global memory
//
// Both are HBM/L2-bound CUDA-core kernels; the arithmetic is the reference's
// (skyrl/tx/kernels/quantized_lora.py:199-212, 248-252, 301-304) evaluated per
// token as in skyrl/tx/layers/lora.py:142-157.
#include <cooperative_groups.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace cg = cooperative_groups;

namespace skyrl {

#ifndef SKYRL_FINALIZE_PAIRS
#define SKYRL_FINALIZE_PAIRS 1  // column pairs per thread of the finalize kernel on wide projections (1, 2 or 4; measured on the c2 step: 2.58, 2.68, 2.79 ms)
#endif

constexpr int ROWQ_THREADS = 128;
constexpr int ROWQ_CLUSTER = 8;

__device__ __forceinline__ float rowq_block_reduce(float v, bool is_max, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < ROWQ_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

// Each thread owns up to VMAX 8-element vectors of its CTA's K slice and keeps them in registers; every
// global load (activations, RMSNorm weights, and with PREFETCH_A the LoRA-A slice) is issued before the
// first reduction, so the kernel pays one memory latency plus the cluster barriers (sum of squares; then absmax and
// projection together; one more so that no CTA leaves while its shared memory is read).
template <int R, int VMAX, bool PREFETCH_A>
__global__ void __cluster_dims__(ROWQ_CLUSTER, 1, 1) __launch_bounds__(ROWQ_THREADS)
rms_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_row_stride,
                      const __nv_bfloat16* __restrict__ delta, float eps, const int32_t* __restrict__ ids,
                      int num_adapters, const __nv_bfloat16* __restrict__ a_packed,
                      const float* __restrict__ scaling, int k, int8_t* __restrict__ xq, float* __restrict__ sx,
                      float* __restrict__ z_rows, int32_t* status, __nv_bfloat16* __restrict__ xn_out) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[ROWQ_THREADS / 32];
  __shared__ float zwarp[ROWQ_THREADS / 32][R];
  __shared__ float part_ss, part_amax;   // this CTA's partial results, read by the whole cluster
  __shared__ float part_z[R];

  const int m = blockIdx.x / ROWQ_CLUSTER;
  const int crank = static_cast<int>(cluster.block_rank());
  const int nvec = k >> 3;
  const int per = (nvec + ROWQ_CLUSTER - 1) / ROWQ_CLUSTER;
  const int v0 = crank * per;
  const int cnt = max(0, min(per, nvec - v0));
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(m) * x_row_stride) + v0;
  const bool norm = delta != nullptr;
  // an id outside the tables is clamped (so that no load leaves them) and reported, as the routing kernel does
  int adapter = ids != nullptr ? __ldg(ids + m) : 0;
  if (adapter < 0 || adapter >= num_adapters) {
    if (threadIdx.x == 0 && crank == 0) atomicCAS(status, 0, STATUS_BAD_ADAPTER_ID);
    adapter = min(max(adapter, 0), num_adapters - 1);
  }
  const uint4* a_base =
      reinterpret_cast<const uint4*>(a_packed + static_cast<int64_t>(adapter) * SKYRL_LORA_RANK_PAD * k) + v0;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

  uint4 xr[VMAX], dr[VMAX];
  uint4 ar[PREFETCH_A ? VMAX : 1][PREFETCH_A ? R : 1];
  // parameters (RMSNorm weights, LoRA-A) first; the activations are the previous kernel's output
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int v = threadIdx.x + i * ROWQ_THREADS;
    const bool valid = v < cnt;
    dr[i] = (valid && norm) ? __ldg(reinterpret_cast<const uint4*>(delta) + v0 + v) : zero4;
    if (PREFETCH_A) {
#pragma unroll
      for (int j = 0; j < R; ++j) ar[i][j] = valid ? __ldg(a_base + static_cast<int64_t>(j) * nvec + v) : zero4;
    }
  }
  pdl_wait();
  pdl_trigger();
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int v = threadIdx.x + i * ROWQ_THREADS;
    xr[i] = v < cnt ? ld_stream16(src + v) : zero4;
  }

  float xv[VMAX][8];
  float ss = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const uint32_t w[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      xv[i][2 * j] = bf16_lo(w[j]);
      xv[i][2 * j + 1] = bf16_hi(w[j]);
      ss = fmaf(xv[i][2 * j], xv[i][2 * j], ss);
      ss = fmaf(xv[i][2 * j + 1], xv[i][2 * j + 1], ss);
    }
  }
  if (norm) {
    ss = rowq_block_reduce(ss, false, red);
    if (threadIdx.x == 0) part_ss = ss;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < ROWQ_CLUSTER; ++r) total += *cluster.map_shared_rank(&part_ss, r);  // fixed order
    const float var = __fdiv_rn(total, static_cast<float>(k));
    const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
#pragma unroll
    for (int i = 0; i < VMAX; ++i) {
      const uint32_t dw[4] = {dr[i].x, dr[i].y, dr[i].z, dr[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xv[i][2 * j] = round_bf16(__fmul_rn(__fmul_rn(xv[i][2 * j], rinv), __fadd_rn(1.0f, bf16_lo(dw[j]))));
        xv[i][2 * j + 1] = round_bf16(__fmul_rn(__fmul_rn(xv[i][2 * j + 1], rinv), __fadd_rn(1.0f, bf16_hi(dw[j]))));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VMAX; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(xv[i][e]));
  // The projection z = n A[a] needs the normalised row but not its absmax, so it is evaluated HERE, before the
  // absmax is exchanged: its LoRA-A loads are in flight during the block reductions, and the partial absmax and
  // the partial z of every CTA cross the cluster behind ONE barrier instead of two.
  float acc[R];
#pragma unroll
  for (int j = 0; j < R; ++j) acc[j] = 0.f;
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int v = threadIdx.x + i * ROWQ_THREADS;
    if (v < cnt) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const uint4 aw = PREFETCH_A ? ar[i][j] : __ldg(a_base + static_cast<int64_t>(j) * nvec + v);
        const uint32_t av[4] = {aw.x, aw.y, aw.z, aw.w};
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          acc[j] = fmaf(xv[i][2 * qd], bf16_lo(av[qd]), acc[j]);
          acc[j] = fmaf(xv[i][2 * qd + 1], bf16_hi(av[qd]), acc[j]);
        }
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    float v = acc[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) zwarp[warp][j] = v;
  }
  amax = rowq_block_reduce(amax, true, red);   // (its barriers also publish zwarp)
  if (threadIdx.x == 0) part_amax = amax;
  if (threadIdx.x < R) {
    float z = 0.f;
#pragma unroll
    for (int w = 0; w < ROWQ_THREADS / 32; ++w) z += zwarp[w][threadIdx.x];
    part_z[threadIdx.x] = z;
  }
  cluster.sync();
  float row_amax = 0.f;
#pragma unroll
  for (int r = 0; r < ROWQ_CLUSTER; ++r) row_amax = fmaxf(row_amax, *cluster.map_shared_rank(&part_amax, r));
  if (crank == 0 && threadIdx.x < SKYRL_LORA_RANK_PAD) {
    float z = 0.f;
    if (threadIdx.x < R) {
#pragma unroll
      for (int r = 0; r < ROWQ_CLUSTER; ++r) z += cluster.map_shared_rank(part_z, r)[threadIdx.x];  // fixed order
      z = __fmul_rn(z, __ldg(scaling + adapter));
    }
    z_rows[static_cast<int64_t>(m) * SKYRL_LORA_RANK_PAD + threadIdx.x] = z;
  }
  const float scale = row_amax > 0.f ? __fdiv_rn(row_amax, 127.0f) : 1.0f;
  const float rcp = quant_rcp(scale);
  if (crank == 0 && threadIdx.x == 0) sx[m] = scale;
  uint2* dst = reinterpret_cast<uint2*>(xq + static_cast<int64_t>(m) * k) + v0;
  uint4* ndst = xn_out != nullptr ? reinterpret_cast<uint4*>(xn_out + static_cast<int64_t>(m) * k) + v0 : nullptr;
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int v = threadIdx.x + i * ROWQ_THREADS;
    if (v < cnt) {
      if (ndst != nullptr)  // the (normalised) bf16 activations both the quantiser and the LoRA term saw, for stage checks
        ndst[v] = make_uint4(pack_bf16x2(xv[i][0], xv[i][1]), pack_bf16x2(xv[i][2], xv[i][3]),
                             pack_bf16x2(xv[i][4], xv[i][5]), pack_bf16x2(xv[i][6], xv[i][7]));
      int q[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) q[e] = quant_code(xv[i][e], scale, rcp);
      dst[v] = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
    }
  }
  cluster.sync();  // no CTA may leave while another still reads its shared memory
}

// P column pairs per thread (pairs j * 256 + threadIdx.x of the CTA's run of 256 * P pairs), rank <= 8 * RV.
// Every load is issued before the first value is used: the scales, the residual and the RAW LoRA-B rows
// before the wait for the GEMM in front of this kernel (CTAs that are resident while that GEMM still runs
// hide them completely), the accumulator right after it, and only then is the LoRA term evaluated.  A CTA
// that starts after the GEMM has finished therefore pays one memory latency, not two in a row.
template <int EPI, int P, int RV>
__global__ void __launch_bounds__(256)
finalize_rows_kernel(const int32_t* __restrict__ acc, int slabs, int64_t slab_stride, const float* __restrict__ sx,
                     const float* __restrict__ sw,
                     const float* __restrict__ z_rows, const int32_t* __restrict__ ids, int num_adapters,
                     const __nv_bfloat16* __restrict__ b_table, int64_t b_adapter_stride, int b_row_stride,
                     int rank_vecs, int n, const __nv_bfloat16* __restrict__ residual, int64_t res_stride,
                     void* __restrict__ out, int64_t out_stride, int32_t* status) {
  __shared__ float zs[SKYRL_LORA_RANK_PAD];
  const int m = blockIdx.y;
  if (rank_vecs > 0 && threadIdx.x < SKYRL_LORA_RANK_PAD)
    zs[threadIdx.x] = z_rows[static_cast<int64_t>(m) * SKYRL_LORA_RANK_PAD + threadIdx.x];
  __syncthreads();
  const int base = 2 * (blockIdx.x * 256 * P + threadIdx.x);  // pair j of this thread: columns base + 512 j, + 1
  const float sxm = __ldg(sx + m);
  int adapter = 0;
  if (rank_vecs > 0) {
    adapter = ids != nullptr ? ids[m] : 0;
    if (adapter < 0 || adapter >= num_adapters) {  // clamped and reported, never used as an index
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(status, 0, STATUS_BAD_ADAPTER_ID);
      adapter = min(max(adapter, 0), num_adapters - 1);
    }
  }
  float2 w2[P];
  uint32_t rv[P];
  uint4 braw[P][2][RV];
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int n0 = base + 512 * j;
    const bool live = n0 < n;
    w2[j] = live ? __ldg(reinterpret_cast<const float2*>(sw + n0)) : make_float2(0.f, 0.f);
    rv[j] = (EPI == SKYRL_EPI_RESIDUAL && live)
                ? __ldg(reinterpret_cast<const uint32_t*>(residual + static_cast<int64_t>(m) * res_stride + n0))
                : 0u;
    const __nv_bfloat16* b0 = b_table + static_cast<int64_t>(adapter) * b_adapter_stride +
                              static_cast<int64_t>(live ? n0 : 0) * b_row_stride;
#pragma unroll
    for (int q = 0; q < RV; ++q) {
      const bool use = live && q < rank_vecs;
      braw[j][0][q] = use ? __ldg(reinterpret_cast<const uint4*>(b0) + q) : zero4;
      braw[j][1][q] = use ? __ldg(reinterpret_cast<const uint4*>(b0 + b_row_stride) + q) : zero4;
    }
  }
  pdl_wait();
  pdl_trigger();
  int2 a2[P];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int n0 = base + 512 * j;
    a2[j] = n0 < n ? ld_stream_int2(acc + static_cast<int64_t>(m) * n + n0) : make_int2(0, 0);
  }
  float l0[P], l1[P];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    l0[j] = 0.f;
    l1[j] = 0.f;
#pragma unroll
    for (int q = 0; q < RV; ++q) {
      if (q < rank_vecs) {  // same order of additions as a loop over q = 0 .. rank_vecs - 1
        const uint32_t c0[4] = {braw[j][0][q].x, braw[j][0][q].y, braw[j][0][q].z, braw[j][0][q].w};
        const uint32_t c1[4] = {braw[j][1][q].x, braw[j][1][q].y, braw[j][1][q].z, braw[j][1][q].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          l0[j] = fmaf(zs[8 * q + 2 * e], bf16_lo(c0[e]), l0[j]);
          l0[j] = fmaf(zs[8 * q + 2 * e + 1], bf16_hi(c0[e]), l0[j]);
          l1[j] = fmaf(zs[8 * q + 2 * e], bf16_lo(c1[e]), l1[j]);
          l1[j] = fmaf(zs[8 * q + 2 * e + 1], bf16_hi(c1[e]), l1[j]);
        }
      }
    }
  }
  for (int sl = 1; sl < slabs; ++sl) {  // split-K partial sums: int32 addition is exact
#pragma unroll
    for (int j = 0; j < P; ++j) {
      const int n0 = base + 512 * j;
      if (n0 < n) {
        const int2 t2 = ld_stream_int2(acc + sl * slab_stride + static_cast<int64_t>(m) * n + n0);
        a2[j].x += t2.x;
        a2[j].y += t2.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int n0 = base + 512 * j;
    if (n0 >= n) continue;
    float f0 = __fmul_rn(__fmul_rn(__int2float_rn(a2[j].x), sxm), w2[j].x);
    float f1 = __fmul_rn(__fmul_rn(__int2float_rn(a2[j].y), sxm), w2[j].y);
    if (rank_vecs > 0) {
      f0 = __fadd_rn(f0, l0[j]);
      f1 = __fadd_rn(f1, l1[j]);
    }
    if (EPI == SKYRL_EPI_PARTIAL_F32) {
      *reinterpret_cast<float2*>(static_cast<float*>(out) + static_cast<int64_t>(m) * out_stride + n0) =
          make_float2(f0, f1);
    } else if (EPI == SKYRL_EPI_SWIGLU) {
      const float g = round_bf16(f0), u = round_bf16(f1);
      const float h = __fmul_rn(__fdiv_rn(g, 1.0f + expf(-g)), u);
      static_cast<__nv_bfloat16*>(out)[static_cast<int64_t>(m) * out_stride + (n0 >> 1)] = __float2bfloat16_rn(h);
    } else if (EPI == SKYRL_EPI_RESIDUAL) {
      *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(out) + static_cast<int64_t>(m) * out_stride + n0) =
          pack_bf16x2(__fadd_rn(round_bf16(f0), bf16_lo(rv[j])), __fadd_rn(round_bf16(f1), bf16_hi(rv[j])));
    } else {
      *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(out) + static_cast<int64_t>(m) * out_stride + n0) =
          pack_bf16x2(f0, f1);
    }
  }
}

template <int R, int VMAX, bool PREFETCH_A>
static int launch_rows_variant(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* ids,
                               int num_adapters, const void* a_packed, const float* scaling, int m, int k, void* xq,
                               float* sx, float* z_rows, int32_t* status, void* xn_out, cudaStream_t stream,
                               bool programmatic) {
  cudaError_t e = launch_kernel(rms_quant_rows_kernel<R, VMAX, PREFETCH_A>, dim3(m * ROWQ_CLUSTER), dim3(ROWQ_THREADS), 0,
                                stream, programmatic, static_cast<const __nv_bfloat16*>(x), x_row_stride,
                                static_cast<const __nv_bfloat16*>(rms_delta), eps, ids, num_adapters,
                                static_cast<const __nv_bfloat16*>(a_packed), scaling, k, static_cast<int8_t*>(xq), sx,
                                z_rows, status, static_cast<__nv_bfloat16*>(xn_out));
  if (e == cudaSuccess) e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "rms_quant_rows launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

int launch_rms_quant_rows(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* ids,
                          int num_adapters, const void* a_packed, const float* scaling, int rank, int m, int k, void* xq,
                          float* sx, float* z_rows, int32_t* status, cudaStream_t stream, bool programmatic,
                          void* xn_out) {
  if (x == nullptr || xq == nullptr || sx == nullptr || a_packed == nullptr || scaling == nullptr ||
      z_rows == nullptr || status == nullptr || m <= 0 || k <= 0 || num_adapters <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: null buffer or non-positive shape");
  if (k % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: K must be a multiple of 16, got %d", k);
  if (x_row_stride < k || x_row_stride % 8 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: row stride must be >= K and a multiple of 8 elements");
  if (!aligned16(x) || !aligned16(xq) || !aligned16(a_packed) || (rms_delta != nullptr && !aligned16(rms_delta)))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: buffers must be 16-byte aligned");
  const int per_cta = ((k >> 3) + ROWQ_CLUSTER - 1) / ROWQ_CLUSTER;  // 8-element vectors per CTA of the cluster
  if (per_cta > 4 * ROWQ_THREADS)
    return fail(SKYRL_ERR_UNSUPPORTED, "rms_quant_rows: K=%d exceeds %d", k, 4 * ROWQ_THREADS * ROWQ_CLUSTER * 8);
  if (rank <= 0 || rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "rms_quant_rows: rank must be in [1, %d], got %d", SKYRL_LORA_RANK_PAD, rank);
#define SKYRL_ROWS(R, V, P) \
  return launch_rows_variant<R, V, P>(x, x_row_stride, rms_delta, eps, ids, num_adapters, a_packed, scaling, m, k, xq, sx, \
                                      z_rows, status, xn_out, stream, programmatic)
  if (per_cta <= 2 * ROWQ_THREADS) {
    if (rank <= 16) SKYRL_ROWS(16, 2, false);
    if (rank <= 32) SKYRL_ROWS(32, 2, false);
    SKYRL_ROWS(64, 2, false);
  }
  if (rank <= 16) SKYRL_ROWS(16, 4, false);
  if (rank <= 32) SKYRL_ROWS(32, 4, false);
  SKYRL_ROWS(64, 4, false);
#undef SKYRL_ROWS
}

int launch_finalize_rows(int epilogue, const int32_t* acc, int slabs, const float* sx, const float* sw,
                         const float* z_rows, const int32_t* ids, int num_adapters, const void* b_table,
                         int64_t b_adapter_stride, int b_row_stride, int rank, int m, int n, const void* residual,
                         int64_t res_stride, void* out, int64_t out_stride, int32_t* status, cudaStream_t stream,
                         bool programmatic) {
  if (acc == nullptr || sx == nullptr || sw == nullptr || out == nullptr || status == nullptr || m <= 0 || n <= 0 ||
      n % 2 != 0 || m > 65535 || num_adapters <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "finalize_rows: null buffer or bad shape");
  if (rank > 0 && (z_rows == nullptr || b_table == nullptr || !aligned16(b_table) || b_row_stride % 8 != 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "finalize_rows: LoRA operands missing or misaligned");
  if (epilogue == SKYRL_EPI_RESIDUAL && residual == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "finalize_rows: residual missing");
  // pairs per thread: 4 (16 or 20 independent 16-byte loads in flight per thread) for wide projections with rank <= 16,
  // else 1 (rank up to 64: the raw LoRA-B rows of one pair are already 64 registers)
  const int rank_vecs = (rank + 7) / 8;
  const bool wide_rank = rank_vecs > 2;
  const int pairs = (!wide_rank && static_cast<int64_t>(n / 2) * m >= 4 * 256 * sm_count()) ? SKYRL_FINALIZE_PAIRS : 1;
  dim3 grid((n / 2 + 256 * pairs - 1) / (256 * pairs), m);
  const __nv_bfloat16* bt = static_cast<const __nv_bfloat16*>(b_table);
  const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(residual);
  cudaError_t le = cudaSuccess;
#define SKYRL_FINALIZE_P(E, PP, RR)                                                                                  \
  le = launch_kernel(finalize_rows_kernel<E, PP, RR>, grid, dim3(256), 0, stream, programmatic, acc, slabs,          \
                     static_cast<int64_t>(m) * n, sx, sw, z_rows, ids, num_adapters, bt, b_adapter_stride, b_row_stride, \
                     rank_vecs, n, res, res_stride, out, out_stride, status)
#define SKYRL_FINALIZE(E)                                \
  if (wide_rank) {                                       \
    SKYRL_FINALIZE_P(E, 1, 8);                           \
  } else if (pairs == 4) {                               \
    SKYRL_FINALIZE_P(E, 4, 2);                           \
  } else if (pairs == 2) {                               \
    SKYRL_FINALIZE_P(E, 2, 2);                           \
  } else {                                               \
    SKYRL_FINALIZE_P(E, 1, 2);                           \
  }
  switch (epilogue) {
    case SKYRL_EPI_LINEAR: SKYRL_FINALIZE(SKYRL_EPI_LINEAR); break;
    case SKYRL_EPI_SWIGLU: SKYRL_FINALIZE(SKYRL_EPI_SWIGLU); break;
    case SKYRL_EPI_RESIDUAL: SKYRL_FINALIZE(SKYRL_EPI_RESIDUAL); break;
    case SKYRL_EPI_PARTIAL_F32: SKYRL_FINALIZE(SKYRL_EPI_PARTIAL_F32); break;
    default: return fail(SKYRL_ERR_INVALID_ARGUMENT, "finalize_rows: unsupported epilogue %d", epilogue);
  }
#undef SKYRL_FINALIZE_P
#undef SKYRL_FINALIZE
  cudaError_t e = le != cudaSuccess ? le : cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "finalize_rows launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

}  // namespace skyrl
