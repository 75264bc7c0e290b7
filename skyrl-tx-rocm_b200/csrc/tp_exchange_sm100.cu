// Tensor-parallel exchange between two MLP blocks: flag words and three kernels per rank and row chunk.
//
// The reference shards gate_up by output features and down by input features and lets GSPMD add one
// all-reduce behind down_proj (skyrl/tx/models/qwen3_5.py:633,644).  Every stage between the down GEMM of
// block l and the gate_up GEMM of block l + 1 is row-wise, so a rank owns 1/tp of a chunk's adapter-sorted
// rows there, and for those rows this file does:
//
//   sum      the fp32 partial sums of the row from EVERY rank, added in ascending rank order (the fp32 group sum of
//            skyrl/tx/kernels/quantized_lora.py:253): from slabs in this rank's memory that the ranks' copy engines
//            filled, from the ranks' own buffers with plain peer loads, or as one multimem.ld_reduce per 16 bytes
//            from the multicast address of a symmetric buffer (the sum formed inside NVSwitch, in its order)
//   finalize bf16(sum) + residual in bf16 (quantized_lora.py:304, qwen3_5.py:784) -> the block's output row
//   prepare  the next block's RMSNorm(1 + delta), per-token absmax, int8 codes (qwen3_5.py:274-278,
//            quantized_lora.py:199-212), bit for bit what rms_quant_kernel produces
//   push     the codes and the scale of the row into EVERY rank's workspace (plain peer stores), the
//            normalised bf16 row into this rank's, for the LoRA-A projection that follows
//
// as two launches (tp_sum_kernel: sum + finalize, a streaming pass; tp_quant_rows_kernel: prepare + push, one warp
// per row) or as one row-per-CTA kernel (tp_exchange_kernel).  Ordering between ranks is by flag words in each
// rank's memory, never by a collective: a rank raises "partial sums of (block, chunk) in place" on every peer, and
// "prepared rows of (block + 1, chunk) delivered" after its pushes.  Flag values only grow (one sequence number
// per block and chunk), so nothing is ever reset.  Every wait is bounded: when the limit runs out the kernel
// records STATUS_TIMEOUT_PEER in the caller's status word and carries on (its rows are then wrong, the context is
// intact, and no GPU is left waiting).  No TMA touches peer memory anywhere.
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
  int profile;                          // 1: CTA 0 adds to status[1..3] what it spent, in units of 1.024 us: waiting for
                                        // the flags, in the streaming sum, in the row-wise quantiser
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

// Sum over all ranks formed inside NVSwitch: one load from the multicast address of a symmetric buffer returns
// the fp32 sum of every rank's copy (order of the additions not specified), so a row crosses this GPU's links
// once instead of tp - 1 times and no rank pushes anything.
__device__ __forceinline__ float4 ld_reduce_mc16(const float4* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// Where the exchange kernels run.  They share the GPU with the GEMMs of the other row chunk, whose persistent
// CTAs leave `reserve` SMs free.  A kernel of small CTAs does not stay on those SMs: a CTA without shared memory
// fits BESIDE a GEMM CTA and fights it for issue slots, and small CTAs that start before the GEMM spread one per
// SM and keep GEMM CTAs out.  Both exchange kernels are therefore launched as `grid` FAT CTAs (512 or 1024
// threads and a shared-memory request above half an SM's): exactly one per SM, never beside a GEMM CTA, `grid`
// SMs in all whichever kernel arrives first.
constexpr int XCH_FAT_SMEM = 120 * 1024;

// First phase of the two-kernel form: out = bf16(sum over ranks, ascending) + residual for this rank's rows,
// as a pure streaming pass.  Nothing here is row-wide, so every thread keeps its loads in flight all the time
// (the fused kernel above alternates between a load phase and the quantiser's reductions); the quantiser then
// runs as a second pass over the bf16 rows, an eighth to a sixteenth of the bytes.
template <int TP, bool MC>
__global__ void __launch_bounds__((MC || TP <= 4) ? 1024 : 512) tp_sum_kernel(const __grid_constant__ ExchangeParams p) {
  const bool prof = p.profile != 0 && blockIdx.x == 0 && threadIdx.x == 0;
  const unsigned long long t_begin = prof ? global_timer_ns() : 0ull;
  if (threadIdx.x == 0 && p.wait_flags != nullptr) wait_flags_reach(p.wait_flags, TP, p.wait_value, p.status);
  __syncthreads();
  const unsigned long long t_ready = prof ? global_timer_ns() : 0ull;
  const int nvec = p.hidden >> 3;
  const int64_t total = static_cast<int64_t>(p.row_count) * nvec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  constexpr int U = MC ? 4 : 1;  // vectors per thread and pass: 8 (in-switch sum) or 2 TP (peer loads) 16-byte loads in flight
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += U * stride) {
    float4 a[U], b[U];
    uint4 rv[U];
    int ovec[U];  // 16-byte vector of `out` this result goes to (-1: past the end)
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      const bool live = i < total;
      const int r = live ? static_cast<int>(i / nvec) : 0;
      const int v = live ? static_cast<int>(i - static_cast<int64_t>(r) * nvec) : 0;
      const int64_t srow = p.row_begin + r;
      const int64_t trow = p.perm != nullptr ? p.perm[srow] : srow;
      ovec[u] = live ? static_cast<int>((p.out_sorted ? srow : trow) * nvec + v) : -1;
      if (MC) {
        const float4* src = reinterpret_cast<const float4*>(p.partial[0] + srow * p.hidden) + 2 * v;  // multicast address
        a[u] = ld_reduce_mc16(src);
        b[u] = ld_reduce_mc16(src + 1);
      } else {
        float4 lo[TP], hi[TP];
#pragma unroll
        for (int s = 0; s < TP; ++s) {
          const float4* src = reinterpret_cast<const float4*>(p.partial[s] + srow * p.hidden) + 2 * v;
          lo[s] = ld_peer16(src);
          hi[s] = ld_peer16(src + 1);
        }
        a[u] = lo[0];
        b[u] = hi[0];
#pragma unroll
        for (int s = 1; s < TP; ++s) {  // ascending rank order, one fp32 addition per rank
          a[u].x = __fadd_rn(a[u].x, lo[s].x); a[u].y = __fadd_rn(a[u].y, lo[s].y);
          a[u].z = __fadd_rn(a[u].z, lo[s].z); a[u].w = __fadd_rn(a[u].w, lo[s].w);
          b[u].x = __fadd_rn(b[u].x, hi[s].x); b[u].y = __fadd_rn(b[u].y, hi[s].y);
          b[u].z = __fadd_rn(b[u].z, hi[s].z); b[u].w = __fadd_rn(b[u].w, hi[s].w);
        }
      }
      rv[u] = __ldg(reinterpret_cast<const uint4*>(p.residual + trow * p.hidden) + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ovec[u] < 0) continue;
      const float f[8] = {a[u].x, a[u].y, a[u].z, a[u].w, b[u].x, b[u].y, b[u].z, b[u].w};
      const uint32_t rw[4] = {rv[u].x, rv[u].y, rv[u].z, rv[u].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2(__fadd_rn(round_bf16(f[2 * j]), bf16_lo(rw[j])), __fadd_rn(round_bf16(f[2 * j + 1]), bf16_hi(rw[j])));
      reinterpret_cast<uint4*>(p.out)[ovec[u]] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (prof) {
    atomicAdd(p.status + 1, static_cast<int>((t_ready - t_begin) >> 10));
    atomicAdd(p.status + 2, static_cast<int>((global_timer_ns() - t_ready) >> 10));
  }
}

// Second phase: the next block's RMSNorm + int8 quantiser over the finalized bf16 rows, ONE WARP PER ROW.
// A row-per-CTA kernel spends most of its time in block-wide barriers with a single row in flight; a fat CTA of
// 32 warps keeps 32 rows in flight per SM and needs no barrier and no shared memory at all: the three passes
// re-read the row from L2 (it was written a moment ago) and the normalised row makes its round trip through
// the `xn` buffer the LoRA-A projection wants anyway (each lane reads back only what it wrote itself).
// Arithmetic and ORDER are those of quant_row_from_smem with 256 threads, so the bits are the same: lane l plays
// the threads l, l + 32, ..., l + 224 (one per warp w of that kernel), keeps their eight partial sums of squares
// apart, reduces each across the lanes with the same xor butterfly and adds the eight results in ascending w.
constexpr int XQ_VIRTUAL_WARPS = QUANT_THREADS / 32;
__global__ void __launch_bounds__(1024) tp_quant_rows_kernel(const __grid_constant__ ExchangeParams p) {
  const bool prof = p.profile != 0 && blockIdx.x == 0 && threadIdx.x == 0;
  const unsigned long long t_begin = prof ? global_timer_ns() : 0ull;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int nvec = p.hidden >> 3;
  const bool norm = p.delta != nullptr;
  const uint4* dvec = reinterpret_cast<const uint4*>(p.delta);
  for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < p.row_count; r += gridDim.x * warps_per_cta) {
    const int64_t srow = p.row_begin + r;
    const int64_t trow = p.perm != nullptr ? p.perm[srow] : srow;
    const uint4* src = reinterpret_cast<const uint4*>(p.out + (p.out_sorted ? srow : trow) * p.hidden);
    uint4* xn_row = reinterpret_cast<uint4*>(p.xn + srow * p.hidden);
    float amax = 0.f;
    constexpr int B = 4;  // vectors a lane requests before it uses the first: the passes are bound by load latency
    if (norm) {
      // pass 1: sums of squares, one per thread of the 256-thread kernel this lane plays; thread l + 32 w owns
      // vectors l + 32 w + 256 i and adds them in ascending i
      float ssw[XQ_VIRTUAL_WARPS];
#pragma unroll
      for (int w = 0; w < XQ_VIRTUAL_WARPS; ++w) ssw[w] = 0.f;
      for (int i = 0; i * QUANT_THREADS < nvec; ++i) {
        uint4 u[XQ_VIRTUAL_WARPS];
#pragma unroll
        for (int w = 0; w < XQ_VIRTUAL_WARPS; ++w) {
          const int v = lane + 32 * w + QUANT_THREADS * i;
          u[w] = v < nvec ? ld_stream16(src + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int w = 0; w < XQ_VIRTUAL_WARPS; ++w) {
          if (lane + 32 * w + QUANT_THREADS * i < nvec) {  // (a zero vector would add +0 and change nothing, but keep the order explicit)
            const uint32_t o[4] = {u[w].x, u[w].y, u[w].z, u[w].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x0 = bf16_lo(o[j]), x1 = bf16_hi(o[j]);
              ssw[w] = fmaf(x0, x0, ssw[w]);
              ssw[w] = fmaf(x1, x1, ssw[w]);
            }
          }
        }
      }
#pragma unroll
      for (int w = 0; w < XQ_VIRTUAL_WARPS; ++w)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssw[w] = ssw[w] + __shfl_xor_sync(0xffffffffu, ssw[w], o);
      float total = ssw[0];
#pragma unroll
      for (int w = 1; w < XQ_VIRTUAL_WARPS; ++w) total = total + ssw[w];
      const float var = __fdiv_rn(total, static_cast<float>(p.hidden));
      const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, p.eps)));
      // pass 2: normalise, round to bf16, absmax; the normalised row goes to xn
      for (int v0 = lane; v0 < nvec; v0 += 32 * B) {
        uint4 u[B], d[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const int v = v0 + 32 * b;
          u[b] = v < nvec ? ld_stream16(src + v) : make_uint4(0u, 0u, 0u, 0u);
          d[b] = v < nvec ? __ldg(dvec + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const int v = v0 + 32 * b;
          if (v >= nvec) continue;
          const uint32_t w4[4] = {u[b].x, u[b].y, u[b].z, u[b].w};
          const uint32_t dw[4] = {d[b].x, d[b].y, d[b].z, d[b].w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = __fmul_rn(__fmul_rn(bf16_lo(w4[j]), rinv), __fadd_rn(1.0f, bf16_lo(dw[j])));
            const float c = __fmul_rn(__fmul_rn(bf16_hi(w4[j]), rinv), __fadd_rn(1.0f, bf16_hi(dw[j])));
            o[j] = pack_bf16x2(a, c);
            amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(o[j])), fabsf(bf16_hi(o[j]))));
          }
          xn_row[v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    } else {
      for (int v0 = lane; v0 < nvec; v0 += 32 * B) {
        uint4 u[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const int v = v0 + 32 * b;
          u[b] = v < nvec ? ld_stream16(src + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const int v = v0 + 32 * b;
          if (v >= nvec) continue;
          const uint32_t o[4] = {u[b].x, u[b].y, u[b].z, u[b].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(o[j])), fabsf(bf16_hi(o[j]))));
          xn_row[v] = u[b];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float rcp = quant_rcp(scale);
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < XCH_MAX_RANKS; ++s)
        if (s < p.tp && p.sx_dst[s] != nullptr) p.sx_dst[s][srow] = scale;
    }
    // pass 3: codes of the normalised row (each lane reads back its own stores, in program order)
    for (int v0 = lane; v0 < nvec; v0 += 32 * B) {
      uint4 u[B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int v = v0 + 32 * b;
        u[b] = v < nvec ? ld_stream16(xn_row + v) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int v = v0 + 32 * b;
        if (v >= nvec) continue;
        const uint32_t w4[4] = {u[b].x, u[b].y, u[b].z, u[b].w};
        int q[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q[2 * j] = quant_code(bf16_lo(w4[j]), scale, rcp);
          q[2 * j + 1] = quant_code(bf16_hi(w4[j]), scale, rcp);
        }
        const uint2 packed = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
#pragma unroll
        for (int s = 0; s < XCH_MAX_RANKS; ++s)
          if (s < p.tp && p.xq_dst[s] != nullptr) reinterpret_cast<uint2*>(p.xq_dst[s] + srow * p.hidden)[v] = packed;
      }
    }
  }
  __threadfence_system();  // this thread's peer stores are performed before the kernel counts as finished
  if (prof) atomicAdd(p.status + 3, static_cast<int>((global_timer_ns() - t_begin) >> 10));
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
static int launch_exchange_variant(ExchangeParams p, int grid, int fat_grid, bool single_kernel, bool multimem, bool wide,
                                   size_t smem, cudaStream_t stream) {
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(tp_exchange_kernel<TP>, 200 * 1024, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_exchange attribute: %s", cudaGetErrorString(e));
  if (!single_kernel) {
    static bool sum_attr[MAX_DEVICES] = {}, sum_mc_attr[MAX_DEVICES] = {}, quant_attr[MAX_DEVICES] = {};
    // wide: many 256-thread CTAs without shared memory, which run on every SM beside the GEMM CTAs (they finish
    // sooner and slow the GEMM a little); otherwise fat CTAs confined to the SMs the GEMM leaves free
    const size_t fat_smem = wide ? 0 : XCH_FAT_SMEM;
    const int sum_threads = wide ? 256 : ((multimem || TP <= 4) ? 1024 : 512);
    if (multimem) {
      e = ensure_dynamic_smem(tp_sum_kernel<TP, true>, XCH_FAT_SMEM, sum_mc_attr);
      if (e == cudaSuccess) tp_sum_kernel<TP, true><<<fat_grid, sum_threads, fat_smem, stream>>>(p);
    } else {
      e = ensure_dynamic_smem(tp_sum_kernel<TP, false>, XCH_FAT_SMEM, sum_attr);
      if (e == cudaSuccess) tp_sum_kernel<TP, false><<<fat_grid, sum_threads, fat_smem, stream>>>(p);
    }
    if (e == cudaSuccess) e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_sum launch: %s", cudaGetErrorString(e));
    if (!p.quantize) return SKYRL_OK;
    p.wait_flags = nullptr;  // the first phase has waited; the stream orders the two phases
    if (p.xn != nullptr) {
      e = ensure_dynamic_smem(tp_quant_rows_kernel, XCH_FAT_SMEM, quant_attr);
      if (e == cudaSuccess) tp_quant_rows_kernel<<<fat_grid, wide ? 256 : 1024, fat_smem, stream>>>(p);
      if (e == cudaSuccess) e = cudaPeekAtLastError();
      if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_quant_rows launch: %s", cudaGetErrorString(e));
      return SKYRL_OK;
    }
    p.from_out = 1;  // no buffer for the normalised rows: the row-per-CTA kernel stages them in shared memory
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
    if ((s == 0 || !a.multimem) && (a.partial[s] == nullptr || !aligned16(a.partial[s])))
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
  p.profile = a.profile ? 1 : 0;
  p.from_out = 0;
  int grid = a.grid_ctas > 0 ? a.grid_ctas : 48;
  // two-launch form: grid_ctas fat CTAs, one per SM (see XCH_FAT_SMEM)
  int fat_grid = grid;
  const int64_t fat_need = (static_cast<int64_t>(a.row_count) * (a.hidden >> 3) + 1023) / 1024;
  if (fat_grid > fat_need) fat_grid = static_cast<int>(fat_need);
  if (!a.wide && fat_grid > sm_count()) fat_grid = sm_count();
  if (grid > a.row_count) grid = a.row_count;
  const bool single = a.single_kernel;
  const bool mc = a.multimem;
  if (mc && single) return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_exchange: the in-switch sum needs the two-launch form");
  switch (a.tp) {
    case 1: return launch_exchange_variant<1>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 2: return launch_exchange_variant<2>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 3: return launch_exchange_variant<3>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 4: return launch_exchange_variant<4>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 5: return launch_exchange_variant<5>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 6: return launch_exchange_variant<6>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    case 7: return launch_exchange_variant<7>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
    default: return launch_exchange_variant<8>(p, grid, fat_grid, single, mc, a.wide, smem, stream);
  }
}

}  // namespace skyrl
