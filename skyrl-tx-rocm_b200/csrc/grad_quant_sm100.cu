// Quantiser of the output cotangent for the input gradient of the W8A8 linear.
//
// The straight-through backward of y = deq(xq wq^T) + s (x A) B needs dx = dy deq(W)^T + R A^T with
// deq(W)[k, n] = wq[k, n] * sw[n] (skyrl/tx/kernels/quantized_lora.py:337-394).  The contraction runs
// over n, where the weight scale varies, so the scale moves to the left operand: g[m, n] = dy[m, n] * sw[n]
// and dx = g wq^T.  g is then split into int8 planes per row, g ~= s1 * q1 + s2 * q2 with
//   s1 = amax(g) / 127,  q1 = rint(g / s1),  r = g - s1 * q1 (|r| <= s1 / 2),  s2 = amax(r) / 127,  q2 = rint(r / s2),
// so that two passes of the int8 tensor-core GEMM over the transposed packed weight reproduce the fp32
// product to ~2^-15 relative (one plane: ~2^-8); the int8 pipe runs at twice the bf16 rate, so two planes
// cost what one bf16 GEMM would.  One CTA per row; the scaled row is staged in shared memory as fp32, so
// dy is read from HBM once.
#include "common.cuh"
#include "quant_row.cuh"

namespace skyrl {

namespace {

__global__ void __launch_bounds__(QUANT_THREADS)
grad_quant_kernel(const __nv_bfloat16* __restrict__ dy, int64_t dy_row_stride, const float* __restrict__ col_scale,
                  const int32_t* __restrict__ row_map, int n, int8_t* __restrict__ q1, float* __restrict__ s1,
                  int8_t* __restrict__ q2, float* __restrict__ s2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* g = reinterpret_cast<float4*>(smem_raw);  // n / 4 vectors
  __shared__ float red[QUANT_THREADS / 32];

  const int out_row = blockIdx.x;
  const int64_t src_row = row_map != nullptr ? row_map[out_row] : out_row;
  const uint4* src = reinterpret_cast<const uint4*>(dy + src_row * dy_row_stride);
  const float4* cs = reinterpret_cast<const float4*>(col_scale);
  const int nvec = n >> 3;

  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
    const uint4 u = __ldg(src + v);
    const float4 c0 = __ldg(cs + 2 * v), c1 = __ldg(cs + 2 * v + 1);
    float4 a, b;
    a.x = __fmul_rn(bf16_lo(u.x), c0.x);
    a.y = __fmul_rn(bf16_hi(u.x), c0.y);
    a.z = __fmul_rn(bf16_lo(u.y), c0.z);
    a.w = __fmul_rn(bf16_hi(u.y), c0.w);
    b.x = __fmul_rn(bf16_lo(u.z), c1.x);
    b.y = __fmul_rn(bf16_hi(u.z), c1.y);
    b.z = __fmul_rn(bf16_lo(u.w), c1.z);
    b.w = __fmul_rn(bf16_hi(u.w), c1.w);
    g[2 * v] = a;
    g[2 * v + 1] = b;
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
  }
  amax = block_reduce(amax, true, red);
  const float scale1 = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float rcp1 = quant_rcp(scale1);
  if (threadIdx.x == 0) s1[out_row] = scale1;

  uint2* dst1 = reinterpret_cast<uint2*>(q1 + static_cast<int64_t>(out_row) * n);
  float amax2 = 0.f;
  for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
    const float4 a = g[2 * v], b = g[2 * v + 1];
    float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    int q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      q[j] = quant_code(e[j], scale1, rcp1);
      const float code = static_cast<float>(static_cast<int8_t>(q[j] & 0xff));
      e[j] = fmaf(-code, scale1, e[j]);  // residual, exact to one rounding
      amax2 = fmaxf(amax2, fabsf(e[j]));
    }
    dst1[v] = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
    if (q2 != nullptr) {
      g[2 * v] = make_float4(e[0], e[1], e[2], e[3]);
      g[2 * v + 1] = make_float4(e[4], e[5], e[6], e[7]);
    }
  }
  if (q2 == nullptr) return;

  amax2 = block_reduce(amax2, true, red);
  const float scale2 = amax2 > 0.f ? __fdiv_rn(amax2, 127.0f) : 1.0f;
  const float rcp2 = quant_rcp(scale2);
  if (threadIdx.x == 0) s2[out_row] = scale2;
  uint2* dst2 = reinterpret_cast<uint2*>(q2 + static_cast<int64_t>(out_row) * n);
  for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
    const float4 a = g[2 * v], b = g[2 * v + 1];
    const float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    int q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = quant_code(e[j], scale2, rcp2);
    dst2[v] = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
  }
}

}  // namespace

int launch_grad_quant(const void* dy, int64_t dy_row_stride, const float* col_scale, const int32_t* row_map, int m, int n,
                      void* q1, float* s1, void* q2, float* s2, cudaStream_t stream) {
  if (dy == nullptr || col_scale == nullptr || q1 == nullptr || s1 == nullptr || m <= 0 || n <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "grad_quant: null buffer or non-positive shape");
  if ((q2 == nullptr) != (s2 == nullptr))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "grad_quant: the second plane needs both its codes and its scales");
  if (n % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "grad_quant: N must be a multiple of 16, got %d", n);
  if (dy_row_stride < n || dy_row_stride % 8 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "grad_quant: row stride must be >= N and a multiple of 8 elements");
  if (!aligned16(dy) || !aligned16(col_scale) || !aligned16(q1) || (q2 != nullptr && !aligned16(q2)))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "grad_quant: buffers must be 16-byte aligned");
  const size_t smem = static_cast<size_t>(n) * 4;
  if (smem > 200 * 1024) return fail(SKYRL_ERR_UNSUPPORTED, "grad_quant: N=%d exceeds the staged-row limit", n);
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(grad_quant_kernel, 200 * 1024, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "grad_quant attribute: %s", cudaGetErrorString(e));
  grad_quant_kernel<<<m, QUANT_THREADS, smem, stream>>>(static_cast<const __nv_bfloat16*>(dy), dy_row_stride, col_scale,
                                                        row_map, n, static_cast<int8_t*>(q1), s1,
                                                        static_cast<int8_t*>(q2), s2);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "grad_quant launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

}  // namespace skyrl

extern "C" int skyrl_w8a8_grad_quant_sm100_v1(const void* dy, int64_t dy_row_stride, const float* col_scale,
                                              const int32_t* row_map, int32_t m, int32_t n, void* q1, float* s1,
                                              void* q2, float* s2, skyrl_stream_t stream) {
  return skyrl::launch_grad_quant(dy, dy_row_stride, col_scale, row_map, m, n, q1, s1, q2, s2,
                                  static_cast<cudaStream_t>(stream));
}
