// Tensor-parallel exchange between two MLP blocks, fused into one kernel per rank and row chunk.
//
// The reference shards gate_up by output features and down by input features and lets GSPMD add one
// all-reduce behind down_proj (skyrl/tx/models/qwen3_5.py:633,644).  Every stage between the down GEMM of
// block l and the gate_up GEMM of block l + 1 is row-wise, so a rank owns 1/tp of a chunk's adapter-sorted
// rows there, and this kernel does for those rows, in one pass over NVLink:
//
//   pull     the fp32 partial sums of the row from EVERY rank's buffer (plain peer loads, no collective),
//            added in ascending rank order: the fp32 group sum of skyrl/tx/kernels/quantized_lora.py:253
//   finalize bf16(sum) + residual in bf16 (quantized_lora.py:304, qwen3_5.py:784) -> the block's output row
//   prepare  the next block's RMSNorm(1 + delta), per-token absmax, int8 codes (qwen3_5.py:274-278,
//            quantized_lora.py:199-212), same code as rms_quant_kernel
//   push     the codes and the scale of the row into EVERY rank's workspace (plain peer stores), the
//            normalised bf16 row into this rank's, for the LoRA-A projection that follows
//
// Ordering between ranks is by flag words in each rank's memory, never by a collective: a rank raises
// "partial sums of (block, chunk) complete" on every peer after its down GEMM, and "prepared rows of
// (block + 1, chunk) delivered" after its pushes.  Flag values only grow (one sequence number per block and
// chunk), so nothing is ever reset.  Every wait is bounded: when the limit runs out the kernel records
// STATUS_TIMEOUT_PEER in the caller's status word and carries on (its rows are then wrong, the context is
// intact, and no GPU is left waiting).  No TMA and no multicast touches peer memory anywhere.
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "quant_row.cuh"

namespace skyrl {

constexpr int XCH_MAX_RANKS = 8;

struct ExchangeParams {
  const float* partial[XCH_MAX_RANKS];  // rank s's fp32 [m, hidden] partial sums, sorted rows (own or peer mapping)
  int tp;
  int row_begin, row_count;             // this rank's rows of the chunk (sorted positions)
  int hidden;
  const int32_t* perm;                  // sorted position -> token row (NULL: identity)
  const __nv_bfloat16* residual;        // bf16 [m, hidden], token order
  __nv_bfloat16* out;                   // bf16 [m, hidden]: row perm[i], or row i when out_sorted
  int out_sorted;
  int from_out;                         // 1: the finalized row is already in `out` (tp_sum_kernel ran): no partial sums are read
  int quantize;                         // 1: run the next block's quantiser stage on the finalized row
  const __nv_bfloat16* delta;           // next block's RMSNorm weights (NULL: no normalisation)
  float eps;
  int8_t* xq_dst[XCH_MAX_RANKS];        // every rank's int8 code region [m, hidden] (NULL entries are skipped)
  float* sx_dst[XCH_MAX_RANKS];         // every rank's fp32 scale region [m]
  __nv_bfloat16* xn;                    // this rank's normalised-row region [m, hidden] or NULL
  const int32_t* wait_flags;            // tp words in this rank's memory, word s raised by rank s
  int32_t wait_value;
  int32_t* status;
};

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Partial sums another GPU wrote (or this GPU's own GEMM, one kernel earlier): a system-scope load, served by
// the owning GPU's L2, never by a line an earlier pass left in this SM's L1.
__device__ __forceinline__ float4 ld_peer16(const float4* p) {
  float4 v;
  // volatile (never hoisted above the flag wait and the barrier behind it) but no memory clobber: the loads of
  // one vector are independent and should all be in flight together
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// Waits until every one of `count` flag words has reached `value` (values only grow; the comparison is on
// the signed difference so that a wrap of the counter is harmless).  Bounded by WAIT_LIMIT_NS.
__device__ __forceinline__ bool wait_flags_reach(const int32_t* flags, int count, int32_t value, int32_t* status) {
  unsigned long long t0 = 0;
  for (int s = 0; s < count; ++s) {
    uint32_t spins = 0;
    while (ld_acquire_sys(flags + s) - value < 0) {
      if ((++spins & 0x3fu) == 0u) {
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > WAIT_LIMIT_NS) {
          atomicCAS(status, 0, STATUS_TIMEOUT_PEER);
          return false;
        }
        __nanosleep(200);
      }
    }
  }
  return true;
}

template <int TP>
__global__ void __launch_bounds__(QUANT_THREADS) tp_exchange_kernel(const __grid_constant__ ExchangeParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* row = reinterpret_cast<uint4*>(smem_raw);  // hidden / 8 vectors of 8 bf16: the finalized row
  __shared__ float red[QUANT_THREADS / 32];

  if (threadIdx.x == 0 && p.wait_flags != nullptr) wait_flags_reach(p.wait_flags, TP, p.wait_value, p.status);
  __syncthreads();

  const int nvec = p.hidden >> 3;   // 8-element vectors per row
  for (int r = blockIdx.x; r < p.row_count; r += gridDim.x) {
    const int64_t srow = p.row_begin + r;
    const int64_t trow = p.perm != nullptr ? p.perm[srow] : srow;
    const uint4* res = reinterpret_cast<const uint4*>(p.residual + trow * p.hidden);
    uint4* dst = reinterpret_cast<uint4*>(p.out + (p.out_sorted ? srow : trow) * p.hidden);
    const bool norm = p.delta != nullptr;
    float ss = 0.f, amax = 0.f;
    if (p.from_out) {
      // second phase of the two-kernel form: the streaming kernel wrote the finalized row, this pass only stages it
      // and accumulates what the quantiser needs, with the same values in the same order as the fused pass below
      for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
        const uint4 ov = ld_stream16(dst + v);
        const uint32_t o[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float x0 = bf16_lo(o[j]), x1 = bf16_hi(o[j]);
          if (norm) {
            ss = fmaf(x0, x0, ss);
            ss = fmaf(x1, x1, ss);
          } else {
            amax = fmaxf(amax, fmaxf(fabsf(x0), fabsf(x1)));
          }
        }
        row[v] = ov;
      }
    } else {
      // Every rank's two float4 of this vector are requested before the first is used: TP x 32 bytes in
      // flight per thread, which is what keeps the NVLink loads streaming.
      for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
        float4 lo[TP], hi[TP];
  #pragma unroll
        for (int s = 0; s < TP; ++s) {
          const float4* src = reinterpret_cast<const float4*>(p.partial[s] + srow * p.hidden) + 2 * v;
          lo[s] = ld_peer16(src);
          hi[s] = ld_peer16(src + 1);
        }
        const uint4 rv = __ldg(res + v);
        float4 a = lo[0], b = hi[0];
  #pragma unroll
        for (int s = 1; s < TP; ++s) {  // ascending rank order, one fp32 addition per rank
          a.x = __fadd_rn(a.x, lo[s].x); a.y = __fadd_rn(a.y, lo[s].y); a.z = __fadd_rn(a.z, lo[s].z); a.w = __fadd_rn(a.w, lo[s].w);
          b.x = __fadd_rn(b.x, hi[s].x); b.y = __fadd_rn(b.y, hi[s].y); b.z = __fadd_rn(b.z, hi[s].z); b.w = __fadd_rn(b.w, hi[s].w);
        }
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
        uint32_t o[4];
  #pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[j] = pack_bf16x2(__fadd_rn(round_bf16(f[2 * j]), bf16_lo(rw[j])),
                             __fadd_rn(round_bf16(f[2 * j + 1]), bf16_hi(rw[j])));
          const float x0 = bf16_lo(o[j]), x1 = bf16_hi(o[j]);
          if (norm) {
            ss = fmaf(x0, x0, ss);
            ss = fmaf(x1, x1, ss);
          } else {
            amax = fmaxf(amax, fmaxf(fabsf(x0), fabsf(x1)));
          }
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        dst[v] = ov;
        row[v] = ov;
      }
    }
    if (p.quantize) {
      QuantDests qd;
      qd.count = 0;
#pragma unroll
      for (int s = 0; s < TP; ++s) {
        if (p.xq_dst[s] != nullptr) {
          qd.xq[qd.count] = p.xq_dst[s] + srow * p.hidden;
          qd.sx[qd.count] = p.sx_dst[s] + srow;
          ++qd.count;
        }
      }
      quant_row_from_smem(row, p.hidden, p.delta, p.eps, ss, amax, red, qd,
                          p.xn != nullptr ? reinterpret_cast<uint4*>(p.xn + srow * p.hidden) : nullptr);
    }
    __syncthreads();  // the staged row is reused by the next iteration
  }
  __threadfence_system();  // this thread's peer stores are performed before the kernel counts as finished
}

// First phase of the two-kernel form: out = bf16(sum over ranks, ascending) + residual for this rank's rows,
// as a pure streaming pass.  Nothing here is row-wide, so every thread keeps TP x 32 bytes of loads in flight
// all the time (the fused kernel above alternates between a load phase and the quantiser's reductions, which
// leaves the few SMs the GEMMs spare idle half of the time); the quantiser then runs as a second pass over the
// bf16 rows, an eighth to a sixteenth of the bytes.
template <int TP>
__global__ void __launch_bounds__(256) tp_sum_kernel(const __grid_constant__ ExchangeParams p) {
  if (threadIdx.x == 0 && p.wait_flags != nullptr) wait_flags_reach(p.wait_flags, TP, p.wait_value, p.status);
  __syncthreads();
  const int nvec = p.hidden >> 3;
  const int64_t total = static_cast<int64_t>(p.row_count) * nvec;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int r = static_cast<int>(i / nvec);
    const int v = static_cast<int>(i - static_cast<int64_t>(r) * nvec);
    const int64_t srow = p.row_begin + r;
    const int64_t trow = p.perm != nullptr ? p.perm[srow] : srow;
    float4 lo[TP], hi[TP];
#pragma unroll
    for (int s = 0; s < TP; ++s) {
      const float4* src = reinterpret_cast<const float4*>(p.partial[s] + srow * p.hidden) + 2 * v;
      lo[s] = ld_peer16(src);
      hi[s] = ld_peer16(src + 1);
    }
    const uint4 rv = __ldg(reinterpret_cast<const uint4*>(p.residual + trow * p.hidden) + v);
    float4 a = lo[0], b = hi[0];
#pragma unroll
    for (int s = 1; s < TP; ++s) {  // ascending rank order, one fp32 addition per rank
      a.x = __fadd_rn(a.x, lo[s].x); a.y = __fadd_rn(a.y, lo[s].y); a.z = __fadd_rn(a.z, lo[s].z); a.w = __fadd_rn(a.w, lo[s].w);
      b.x = __fadd_rn(b.x, hi[s].x); b.y = __fadd_rn(b.y, hi[s].y); b.z = __fadd_rn(b.z, hi[s].z); b.w = __fadd_rn(b.w, hi[s].w);
    }
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(__fadd_rn(round_bf16(f[2 * j]), bf16_lo(rw[j])), __fadd_rn(round_bf16(f[2 * j + 1]), bf16_hi(rw[j])));
    reinterpret_cast<uint4*>(p.out + (p.out_sorted ? srow : trow) * p.hidden)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// One warp: after everything enqueued before it on the stream has completed, raise `value` in up to eight
// flag words (each in some rank's memory).
struct SignalParams {
  int32_t* flag[XCH_MAX_RANKS];
  int count;
  int32_t value;
};
__global__ void __launch_bounds__(32) tp_signal_kernel(const SignalParams p) {
  __threadfence_system();
  if (static_cast<int>(threadIdx.x) < p.count && p.flag[threadIdx.x] != nullptr) st_release_sys(p.flag[threadIdx.x], p.value);
}

// One thread: returns once `count` local flag words have reached `value`, or the limit ran out (status).
__global__ void __launch_bounds__(32) tp_wait_kernel(const int32_t* flags, int count, int32_t value, int32_t* status) {
  if (threadIdx.x == 0) wait_flags_reach(flags, count, value, status);
}

int launch_tp_signal(int32_t* const* flags, int count, int32_t value, cudaStream_t stream) {
  if (flags == nullptr || count < 1 || count > XCH_MAX_RANKS)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_signal: 1 to %d flag addresses wanted, got %d", XCH_MAX_RANKS, count);
  SignalParams p = {};
  p.count = count;
  p.value = value;
  for (int r = 0; r < count; ++r) {
    if (flags[r] != nullptr && (reinterpret_cast<uintptr_t>(flags[r]) & 3u) != 0)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_signal: flag %d is not 4-byte aligned", r);
    p.flag[r] = flags[r];
  }
  tp_signal_kernel<<<1, 32, 0, stream>>>(p);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_signal launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

int launch_tp_wait(const int32_t* flags, int count, int32_t value, int32_t* status, cudaStream_t stream) {
  if (flags == nullptr || status == nullptr || count < 1 || count > XCH_MAX_RANKS)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_wait: flags / status missing or count outside [1, %d]", XCH_MAX_RANKS);
  tp_wait_kernel<<<1, 32, 0, stream>>>(flags, count, value, status);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_wait launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

template <int TP>
static int launch_exchange_variant(ExchangeParams p, int grid, int sum_grid, bool single_kernel, size_t smem,
                                   cudaStream_t stream) {
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(tp_exchange_kernel<TP>, 200 * 1024, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_exchange attribute: %s", cudaGetErrorString(e));
  if (!single_kernel) {
    tp_sum_kernel<TP><<<sum_grid, 256, 0, stream>>>(p);
    e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_sum launch: %s", cudaGetErrorString(e));
    if (!p.quantize) return SKYRL_OK;
    p.from_out = 1;          // the same stream orders the two phases
    p.wait_flags = nullptr;  // the first phase has waited
  }
  tp_exchange_kernel<TP><<<grid, QUANT_THREADS, smem, stream>>>(p);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_exchange launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

int launch_tp_exchange(const TpExchangeLaunch& a, cudaStream_t stream) {
  if (a.tp < 1 || a.tp > XCH_MAX_RANKS) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: 1 to %d ranks, got %d", XCH_MAX_RANKS, a.tp);
  if (a.row_count <= 0 || a.row_begin < 0 || a.hidden <= 0 || a.hidden % 16 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: bad row range or hidden size (a multiple of 16 wanted)");
  if (a.residual == nullptr || a.out == nullptr || a.status == nullptr || !aligned16(a.residual) || !aligned16(a.out))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: residual / out / status missing or not 16-byte aligned");
  const size_t smem = static_cast<size_t>(a.hidden) * 2;
  if (smem > 200 * 1024) return fail(SKYRL_ERR_UNSUPPORTED, "tp_exchange: hidden=%d exceeds the staged-row limit", a.hidden);
  ExchangeParams p = {};
  p.tp = a.tp;
  for (int s = 0; s < a.tp; ++s) {
    if (a.partial[s] == nullptr || !aligned16(a.partial[s]))
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: partial-sum buffer %d is null or not 16-byte aligned", s);
    p.partial[s] = a.partial[s];
    p.xq_dst[s] = a.xq_dst[s];
    p.sx_dst[s] = a.sx_dst[s];
    if (a.quantize && ((a.xq_dst[s] == nullptr) != (a.sx_dst[s] == nullptr) || (a.xq_dst[s] != nullptr && !aligned16(a.xq_dst[s]))))
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: code / scale destination %d is inconsistent or misaligned", s);
  }
  p.row_begin = a.row_begin;
  p.row_count = a.row_count;
  p.hidden = a.hidden;
  p.perm = a.perm;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.out_sorted = a.out_sorted ? 1 : 0;
  p.quantize = a.quantize ? 1 : 0;
  p.delta = static_cast<const __nv_bfloat16*>(a.delta);
  p.eps = a.eps;
  p.xn = static_cast<__nv_bfloat16*>(a.xn);
  p.wait_flags = a.wait_flags;
  p.wait_value = a.wait_value;
  p.status = a.status;
  p.from_out = 0;
  int grid = a.grid_ctas > 0 ? a.grid_ctas : 48;
  // The row-wise kernel keeps up to eight CTAs per SM busy; the streaming kernel wants every thread slot of the SMs
  // it gets (eight 256-thread CTAs per SM as well), so both use the same grid unless rows are few.
  int sum_grid = grid;
  const int64_t vec_ctas = (static_cast<int64_t>(a.row_count) * (a.hidden >> 3) + 255) / 256;
  if (sum_grid > vec_ctas) sum_grid = static_cast<int>(vec_ctas);
  if (grid > a.row_count) grid = a.row_count;
  const bool single = a.single_kernel;
  switch (a.tp) {
    case 1: return launch_exchange_variant<1>(p, grid, sum_grid, single, smem, stream);
    case 2: return launch_exchange_variant<2>(p, grid, sum_grid, single, smem, stream);
    case 3: return launch_exchange_variant<3>(p, grid, sum_grid, single, smem, stream);
    case 4: return launch_exchange_variant<4>(p, grid, sum_grid, single, smem, stream);
    case 5: return launch_exchange_variant<5>(p, grid, sum_grid, single, smem, stream);
    case 6: return launch_exchange_variant<6>(p, grid, sum_grid, single, smem, stream);
    case 7: return launch_exchange_variant<7>(p, grid, sum_grid, single, smem, stream);
    default: return launch_exchange_variant<8>(p, grid, sum_grid, single, smem, stream);
  }
}

}  // namespace skyrl
