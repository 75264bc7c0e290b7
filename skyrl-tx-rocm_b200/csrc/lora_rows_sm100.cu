// Row-wise LoRA kernels for small batches (decode shapes: a few dozen token
// rows, almost every row with its own adapter).  Sorting rows by adapter and
// spending one 128-row tensor-core tile per adapter would multiply the weight
// traffic by the number of adapters, so here every row carries its adapter id:
//
//   rms_quant_rows_kernel<R> ... K1 of the main path (RMSNorm, absmax, int8 codes)
//                                plus z[m, :] = s[a] * (n[m, :] @ A[a]) while the
//                                normalised row is still in shared memory
//   lora_b_rows_kernel ......... addend[m, n] = sum_j z[m, j] * B[a(m)][n, j] (fp32),
//                                consumed by the GEMM epilogue before the single cast
//
// Both are HBM/L2-bound CUDA-core kernels; the arithmetic is the reference's
// fp32 LoRA term (skyrl/tx/kernels/quantized_lora.py:301-304) evaluated per
// token as in skyrl/tx/layers/lora.py:142-157.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace skyrl {

constexpr int ROWS_THREADS = 256;

__device__ __forceinline__ float rows_block_reduce(float v, bool is_max, float* red) {
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
  for (int w = 1; w < ROWS_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

template <int R>
__global__ void __launch_bounds__(ROWS_THREADS)
rms_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_row_stride,
                      const __nv_bfloat16* __restrict__ delta, float eps, const int32_t* __restrict__ ids,
                      const __nv_bfloat16* __restrict__ a_packed, const float* __restrict__ scaling, int k,
                      int8_t* __restrict__ xq, float* __restrict__ sx, float* __restrict__ z_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* row = reinterpret_cast<uint4*>(smem_raw);
  __shared__ float red[ROWS_THREADS / 32];
  __shared__ float zred[ROWS_THREADS / 32][R];

  const int m = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(m) * x_row_stride);
  const int nvec = k >> 3;
  const bool norm = delta != nullptr;

  float ss = 0.f, amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += ROWS_THREADS) {
    const uint4 u = __ldg(src + v);
    row[v] = u;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = bf16_lo(w[j]), b = bf16_hi(w[j]);
      if (norm) {
        ss = fmaf(a, a, ss);
        ss = fmaf(b, b, ss);
      } else {
        amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
      }
    }
  }
  if (norm) {
    ss = rows_block_reduce(ss, false, red);
    const float var = __fdiv_rn(ss, static_cast<float>(k));
    const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    const uint4* dvec = reinterpret_cast<const uint4*>(delta);
    for (int v = threadIdx.x; v < nvec; v += ROWS_THREADS) {
      const uint4 u = row[v];
      const uint4 d = __ldg(dvec + v);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __fmul_rn(__fmul_rn(bf16_lo(w[j]), rinv), __fadd_rn(1.0f, bf16_lo(dw[j])));
        const float b = __fmul_rn(__fmul_rn(bf16_hi(w[j]), rinv), __fadd_rn(1.0f, bf16_hi(dw[j])));
        o[j] = pack_bf16x2(a, b);
        amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(o[j])), fabsf(bf16_hi(o[j]))));
      }
      row[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  amax = rows_block_reduce(amax, true, red);  // also orders the writes to `row` before the reads below
  const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  if (threadIdx.x == 0) sx[m] = scale;

  const int adapter = ids != nullptr ? ids[m] : 0;
  const uint4* a_base = reinterpret_cast<const uint4*>(a_packed + static_cast<int64_t>(adapter) * SKYRL_LORA_RANK_PAD * k);
  float acc[R];
#pragma unroll
  for (int j = 0; j < R; ++j) acc[j] = 0.f;

  uint2* dst = reinterpret_cast<uint2*>(xq + static_cast<int64_t>(m) * k);
  for (int v = threadIdx.x; v < nvec; v += ROWS_THREADS) {
    const uint4 u = row[v];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float xv[8];
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      xv[2 * j] = bf16_lo(w[j]);
      xv[2 * j + 1] = bf16_hi(w[j]);
      int qa = __float2int_rn(__fdiv_rn(xv[2 * j], scale));
      int qb = __float2int_rn(__fdiv_rn(xv[2 * j + 1], scale));
      qa = max(-127, min(127, qa));
      qb = max(-127, min(127, qb));
      const uint32_t two = (static_cast<uint32_t>(qa) & 0xffu) | ((static_cast<uint32_t>(qb) & 0xffu) << 8);
      packed[j >> 1] |= two << ((j & 1) * 16);
    }
    dst[v] = make_uint2(packed[0], packed[1]);
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const uint4 aw = __ldg(a_base + static_cast<int64_t>(j) * nvec + v);
      const uint32_t av[4] = {aw.x, aw.y, aw.z, aw.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[j] = fmaf(xv[2 * q], bf16_lo(av[q]), acc[j]);
        acc[j] = fmaf(xv[2 * q + 1], bf16_hi(av[q]), acc[j]);
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    float v = acc[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) zred[warp][j] = v;
  }
  __syncthreads();
  if (threadIdx.x < SKYRL_LORA_RANK_PAD) {
    float z = 0.f;
    if (threadIdx.x < R) {
#pragma unroll
      for (int w = 0; w < ROWS_THREADS / 32; ++w) z += zred[w][threadIdx.x];
      z = __fmul_rn(z, __ldg(scaling + adapter));
    }
    z_rows[static_cast<int64_t>(m) * SKYRL_LORA_RANK_PAD + threadIdx.x] = z;
  }
}

__global__ void __launch_bounds__(ROWS_THREADS)
lora_b_rows_kernel(const float* __restrict__ z_rows, const int32_t* __restrict__ ids,
                   const __nv_bfloat16* __restrict__ b_packed, int n, int rank_vecs, float* __restrict__ addend,
                   int64_t addend_stride) {
  __shared__ float zs[SKYRL_LORA_RANK_PAD];
  const int m = blockIdx.y;
  if (threadIdx.x < SKYRL_LORA_RANK_PAD) zs[threadIdx.x] = z_rows[static_cast<int64_t>(m) * SKYRL_LORA_RANK_PAD + threadIdx.x];
  __syncthreads();
  const int nn = blockIdx.x * ROWS_THREADS + threadIdx.x;
  if (nn >= n) return;
  const int adapter = ids != nullptr ? ids[m] : 0;
  const uint4* brow = reinterpret_cast<const uint4*>(b_packed + (static_cast<int64_t>(adapter) * n + nn) * SKYRL_LORA_RANK_PAD);
  float acc = 0.f;
  for (int q = 0; q < rank_vecs; ++q) {
    const uint4 w = __ldg(brow + q);
    const uint32_t bv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc = fmaf(zs[8 * q + 2 * j], bf16_lo(bv[j]), acc);
      acc = fmaf(zs[8 * q + 2 * j + 1], bf16_hi(bv[j]), acc);
    }
  }
  addend[static_cast<int64_t>(m) * addend_stride + nn] = acc;
}

template <int R>
static int launch_rows_variant(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* ids,
                               const void* a_packed, const float* scaling, int m, int k, void* xq, float* sx,
                               float* z_rows, cudaStream_t stream) {
  auto kernel = rms_quant_rows_kernel<R>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "rms_quant_rows attribute: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  kernel<<<m, ROWS_THREADS, static_cast<size_t>(k) * 2, stream>>>(
      static_cast<const __nv_bfloat16*>(x), x_row_stride, static_cast<const __nv_bfloat16*>(rms_delta), eps, ids,
      static_cast<const __nv_bfloat16*>(a_packed), scaling, k, static_cast<int8_t*>(xq), sx, z_rows);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "rms_quant_rows launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

int launch_rms_quant_rows(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* ids,
                          const void* a_packed, const float* scaling, int rank, int m, int k, void* xq, float* sx,
                          float* z_rows, cudaStream_t stream) {
  if (x == nullptr || xq == nullptr || sx == nullptr || a_packed == nullptr || scaling == nullptr ||
      z_rows == nullptr || m <= 0 || k <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: null buffer or non-positive shape");
  if (k % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: K must be a multiple of 16, got %d", k);
  if (x_row_stride < k || x_row_stride % 8 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: row stride must be >= K and a multiple of 8 elements");
  if (!aligned16(x) || !aligned16(xq) || !aligned16(a_packed) || (rms_delta != nullptr && !aligned16(rms_delta)))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant_rows: buffers must be 16-byte aligned");
  if (static_cast<size_t>(k) * 2 > 200 * 1024)
    return fail(SKYRL_ERR_UNSUPPORTED, "rms_quant_rows: K=%d exceeds the staged-row limit", k);
  if (rank <= 0 || rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "rms_quant_rows: rank must be in [1, %d], got %d", SKYRL_LORA_RANK_PAD, rank);
  if (rank <= 16)
    return launch_rows_variant<16>(x, x_row_stride, rms_delta, eps, ids, a_packed, scaling, m, k, xq, sx, z_rows, stream);
  if (rank <= 32)
    return launch_rows_variant<32>(x, x_row_stride, rms_delta, eps, ids, a_packed, scaling, m, k, xq, sx, z_rows, stream);
  return launch_rows_variant<64>(x, x_row_stride, rms_delta, eps, ids, a_packed, scaling, m, k, xq, sx, z_rows, stream);
}

int launch_lora_b_rows(const float* z_rows, const int32_t* ids, const void* b_packed, int rank, int m, int n,
                       float* addend, int64_t addend_stride, cudaStream_t stream) {
  if (z_rows == nullptr || b_packed == nullptr || addend == nullptr || m <= 0 || n <= 0 || m > 65535)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_b_rows: null buffer or bad shape");
  if (!aligned16(b_packed) || addend_stride < n)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_b_rows: misaligned table or short addend stride");
  dim3 grid((n + ROWS_THREADS - 1) / ROWS_THREADS, m);
  lora_b_rows_kernel<<<grid, ROWS_THREADS, 0, stream>>>(z_rows, ids, static_cast<const __nv_bfloat16*>(b_packed), n,
                                                        (rank + 7) / 8, addend, addend_stride);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "lora_b_rows launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

}  // namespace skyrl
