// Row-wise RMSNorm + per-token int8 quantiser shared by rms_quant_kernel and the tensor-parallel
// exchange kernel: both must produce the same bits for the same row, so the arithmetic (and the
// order of the block-wide reductions) lives here once.
#pragma once

#include "ptx_sm100.cuh"

namespace skyrl {

constexpr int QUANT_THREADS = 256;
constexpr int QUANT_MAX_DESTS = 8;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();  // protects `red` against the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < QUANT_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

// Where the codes and the scale of one row go: up to QUANT_MAX_DESTS copies (a tensor-parallel rank
// hands its rows to every peer's workspace; one destination otherwise).
struct QuantDests {
  int8_t* xq[QUANT_MAX_DESTS];   // row pointers (already offset to the row)
  float* sx[QUANT_MAX_DESTS];    // scale pointers (already offset to the row)
  int count;
};

// One row of k bf16 values staged in shared memory (`row`, k / 8 vectors), QUANT_THREADS threads.
// Arithmetic follows the reference exactly: fp32 mean of squares, (x * rinv) * (1 + delta) rounded to
// bf16 (skyrl/tx/models/qwen3_5.py:274-278), then amax / 127 and rint(x / scale) with IEEE division
// (skyrl/tx/kernels/quantized_lora.py:207-211).  `ss` / `amax` are this thread's partial sum of
// squares (norm) or partial absmax (no norm) over the vectors v = threadIdx.x, + QUANT_THREADS, ...
// accumulated in that order.  `xn_row` (nullable) receives the normalised (or copied) row.
__device__ __forceinline__ void quant_row_from_smem(uint4* row, int k, const __nv_bfloat16* __restrict__ delta,
                                                    float eps, float ss, float amax, float* red,
                                                    const QuantDests& dst, uint4* xn_row) {
  const int nvec = k >> 3;
  const bool norm = delta != nullptr;
  if (norm) {
    ss = block_reduce(ss, false, red);
    const float var = __fdiv_rn(ss, static_cast<float>(k));
    const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    const uint4* dvec = reinterpret_cast<const uint4*>(delta);
    for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
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
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      row[v] = ov;
      if (xn_row != nullptr) xn_row[v] = ov;
    }
  } else if (xn_row != nullptr) {
    for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) xn_row[v] = row[v];
  }
  amax = block_reduce(amax, true, red);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float rcp = quant_rcp(scale);
  if (threadIdx.x == 0) {
    for (int d = 0; d < dst.count; ++d) *dst.sx[d] = scale;
  }
  for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
    const uint4 u = row[v];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    int q[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      q[2 * j] = quant_code(bf16_lo(w[j]), scale, rcp);
      q[2 * j + 1] = quant_code(bf16_hi(w[j]), scale, rcp);
    }
    const uint2 packed = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
    for (int d = 0; d < dst.count; ++d) reinterpret_cast<uint2*>(dst.xq[d])[v] = packed;
  }
}

}  // namespace skyrl
