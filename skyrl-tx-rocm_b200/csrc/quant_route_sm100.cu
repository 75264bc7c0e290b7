// HBM-bound front-end kernels of the W8A8 multi-LoRA path:
//   * route_kernel ....... stable counting sort of token rows by adapter id and
//                          the list of 128-row M tiles (at most two adapters per tile)
//   * rms_quant_kernel ... optional RMSNorm(1 + delta), per-token absmax, int8 codes
//   * pack kernels ....... one-time layout changes of weights and LoRA tables
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "quant_row.cuh"

namespace skyrl {

// ----------------------------------------------------------------------------
// Routing.  One CTA; the histogram is parallel, the stable scatter is done by a
// single warp with match_any so that rows of an adapter keep their order
// (the reference's argsort is used the same way: skyrl/tx/layers/util.py:82-87).
// ----------------------------------------------------------------------------
constexpr int ROUTE_THREADS = 1024;
constexpr int ROUTE_MAX_ADAPTERS = 4096;

// Tile lists.  With chunk_rows == 0 there is one list at `tiles` and its length at num_tiles[0].
// With chunk_rows > 0 (a multiple of 128) the sorted row space is cut at multiples of chunk_rows and
// chunk c gets its own list at tiles + 4 * c * chunk_cap with its length at num_tiles[c]; no tile
// crosses a chunk boundary, so the chunks of a block can be computed and reduced independently.
__global__ void __launch_bounds__(ROUTE_THREADS)
route_kernel(const int32_t* __restrict__ ids, int m, int num_adapters, int32_t* __restrict__ perm,
             int32_t* __restrict__ tiles, int32_t* __restrict__ num_tiles, int max_tiles, int chunk_rows,
             int chunk_cap, int32_t* status, int32_t* __restrict__ zero_words, int zero_count) {
  __shared__ int counts[ROUTE_MAX_ADAPTERS];
  __shared__ int cursor[ROUTE_MAX_ADAPTERS];
  const int tid = threadIdx.x;
  if (zero_words != nullptr && tid < zero_count) zero_words[tid] = 0;
  const int num_chunks = chunk_rows > 0 ? (m + chunk_rows - 1) / chunk_rows : 1;
  const int cap = chunk_rows > 0 ? chunk_cap : max_tiles;
  const int span = chunk_rows > 0 ? chunk_rows : m;

  if (ids == nullptr) {
    for (int i = tid; i < m; i += ROUTE_THREADS) perm[i] = i;
    const int per_chunk = (span + SKYRL_TILE_ROWS - 1) / SKYRL_TILE_ROWS;
    if (per_chunk > cap) {
      if (tid == 0) atomicCAS(status, 0, STATUS_TILE_OVERFLOW);
      for (int c = tid; c < num_chunks; c += ROUTE_THREADS) num_tiles[c] = 0;
      return;
    }
    const int nt = (m + SKYRL_TILE_ROWS - 1) / SKYRL_TILE_ROWS;
    for (int t = tid; t < nt; t += ROUTE_THREADS) {
      const int r0 = t * SKYRL_TILE_ROWS;
      const int c = r0 / span;  // chunk_rows is a multiple of the tile height, so tiles never straddle
      const int slot = c * cap + (r0 - c * span) / SKYRL_TILE_ROWS;
      reinterpret_cast<int4*>(tiles)[slot] = make_int4(r0, min(SKYRL_TILE_ROWS, m - r0), 0, 0);
    }
    for (int c = tid; c < num_chunks; c += ROUTE_THREADS) {
      const int rows = min(span, m - c * span);
      num_tiles[c] = (rows + SKYRL_TILE_ROWS - 1) / SKYRL_TILE_ROWS;
    }
    return;
  }

  for (int a = tid; a < num_adapters; a += ROUTE_THREADS) counts[a] = 0;
  __syncthreads();
  for (int i = tid; i < m; i += ROUTE_THREADS) {
    int a = ids[i];
    if (a < 0 || a >= num_adapters) {
      atomicCAS(status, 0, STATUS_BAD_ADAPTER_ID);
      a = min(max(a, 0), num_adapters - 1);
    }
    atomicAdd(&counts[a], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int start = 0;
    for (int a = 0; a < num_adapters; ++a) {
      cursor[a] = start;
      start += counts[a];
    }
    // Greedy packing of the sorted rows into tiles of up to 128 rows and at most two adapters: where an
    // adapter's run ends inside a tile, the tile is filled up with rows of the next adapter.
    int chunk = 0, in_chunk = 0, pos = 0, a = 0;
    bool overflow = false;
    while (a < num_adapters && counts[a] == 0) ++a;
    while (pos < m && a < num_adapters) {
      while (pos >= (chunk + 1) * span) {  // close the chunks this row has passed
        num_tiles[chunk] = in_chunk;
        ++chunk;
        in_chunk = 0;
      }
      const int cend = min(m, (chunk + 1) * span);
      const int aend = cursor[a] + counts[a];
      const int take = min(SKYRL_TILE_ROWS, min(aend, cend) - pos);
      int rows = take, second = 0;
      if (take < SKYRL_TILE_ROWS && pos + take == aend && pos + take < cend) {
        int b = a + 1;
        while (b < num_adapters && counts[b] == 0) ++b;
        if (b < num_adapters) {
          const int bend = cursor[b] + counts[b];
          rows = take + min(SKYRL_TILE_ROWS - take, min(bend, cend) - (pos + take));
          second = (b + 1) | (take << 16);
        }
      }
      if (in_chunk < cap) {
        reinterpret_cast<int4*>(tiles)[chunk * cap + in_chunk] = make_int4(pos, rows, a, second);
      } else {
        overflow = true;
      }
      ++in_chunk;
      pos += rows;
      while (a < num_adapters && pos >= cursor[a] + counts[a]) ++a;  // the adapter that owns row `pos`
    }
    num_tiles[chunk] = in_chunk;
    for (int c = chunk + 1; c < num_chunks; ++c) num_tiles[c] = 0;
    if (overflow) {
      atomicCAS(status, 0, STATUS_TILE_OVERFLOW);
      for (int c = 0; c < num_chunks; ++c) num_tiles[c] = 0;
    }
  }
  __syncthreads();
  if (tid < 32) {
    const unsigned lt_mask = (1u << tid) - 1u;
    for (int base = 0; base < m; base += 32) {
      const int i = base + tid;
      const bool active = i < m;
      int a = active ? ids[i] : -1;
      if (active) a = min(max(a, 0), num_adapters - 1);
      const unsigned peers = __match_any_sync(0xffffffffu, a);
      const int rank = __popc(peers & lt_mask);
      if (active) perm[cursor[a] + rank] = i;
      __syncwarp();
      if (active && rank == 0) cursor[a] += __popc(peers);
      __syncwarp();
    }
  }
}

int launch_route(const int32_t* ids, int m, int num_adapters, int32_t* perm, int32_t* tiles, int32_t* num_tiles,
                 int max_tiles, int32_t* status, cudaStream_t stream, int chunk_rows, int chunk_cap, int32_t* zero_words,
                 int zero_count) {
  if (m <= 0 || perm == nullptr || tiles == nullptr || num_tiles == nullptr || status == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: m must be positive and perm/tiles/num_tiles/status non-null");
  if (ids != nullptr && (num_adapters <= 0 || num_adapters > ROUTE_MAX_ADAPTERS))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: num_adapters must be in [1, %d], got %d", ROUTE_MAX_ADAPTERS,
                num_adapters);
  if (max_tiles <= 0 || !aligned16(tiles))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: tiles must be 16-byte aligned with max_tiles > 0");
  if (chunk_rows < 0 || chunk_rows % SKYRL_TILE_ROWS != 0 || (chunk_rows > 0 && chunk_cap <= 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: chunk_rows must be a multiple of %d", SKYRL_TILE_ROWS);
  if (chunk_rows > 0 && static_cast<int64_t>((m + chunk_rows - 1) / chunk_rows) * chunk_cap > max_tiles)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: chunk lists do not fit in max_tiles");
  if (zero_count < 0 || zero_count > ROUTE_THREADS)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "route: at most %d words can be cleared", ROUTE_THREADS);
  route_kernel<<<1, ROUTE_THREADS, 0, stream>>>(ids, m, num_adapters, perm, tiles, num_tiles, max_tiles, chunk_rows,
                                                chunk_cap, status, zero_words, zero_count);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "route launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// ----------------------------------------------------------------------------
// RMSNorm + per-token int8 quantisation.  One CTA per output row; the row is
// staged in shared memory so HBM is read once.  Arithmetic follows the
// reference exactly: fp32 mean of squares, (x * rinv) * (1 + delta) rounded to
// bf16 (skyrl/tx/models/qwen3_5.py:274-278), then amax / 127 and
// rint(x / scale) with IEEE division (skyrl/tx/kernels/quantized_lora.py:207-211).
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(QUANT_THREADS)
rms_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, const __nv_bfloat16* __restrict__ delta,
                 float eps, const int32_t* __restrict__ row_map, int k, int8_t* __restrict__ xq,
                 float* __restrict__ sx, __nv_bfloat16* __restrict__ xn) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* row = reinterpret_cast<uint4*>(smem_raw);  // k / 8 vectors of 8 bf16
  __shared__ float red[QUANT_THREADS / 32];

  const int out_row = blockIdx.x;
  const int64_t src_row = row_map != nullptr ? row_map[out_row] : out_row;
  const uint4* src = reinterpret_cast<const uint4*>(x + src_row * x_row_stride);
  const int nvec = k >> 3;
  const bool norm = delta != nullptr;

  float ss = 0.f, amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
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
  QuantDests dst;
  dst.count = 1;
  dst.xq[0] = xq + static_cast<int64_t>(out_row) * k;
  dst.sx[0] = sx + out_row;
  quant_row_from_smem(row, k, delta, eps, ss, amax, red, dst,
                      xn != nullptr ? reinterpret_cast<uint4*>(xn + static_cast<int64_t>(out_row) * k) : nullptr);
}

int launch_rms_quant(const void* x, int64_t x_row_stride, const void* rms_delta, float eps, const int32_t* row_map,
                     int m, int k, void* xq, float* sx, void* xn, cudaStream_t stream) {
  if (x == nullptr || xq == nullptr || sx == nullptr || m <= 0 || k <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant: null buffer or non-positive shape");
  if (k % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant: K must be a multiple of 16, got %d", k);
  if (x_row_stride < k || x_row_stride % 8 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant: row stride must be >= K and a multiple of 8 elements");
  if (!aligned16(x) || !aligned16(xq) || (xn != nullptr && !aligned16(xn)) ||
      (rms_delta != nullptr && !aligned16(rms_delta)))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant: buffers must be 16-byte aligned");
  if (x == xq || x == xn) return fail(SKYRL_ERR_INVALID_ARGUMENT, "rms_quant: inputs and outputs must not alias");
  const size_t smem = static_cast<size_t>(k) * 2;
  if (smem > 200 * 1024) return fail(SKYRL_ERR_UNSUPPORTED, "rms_quant: K=%d exceeds the staged-row limit", k);
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(rms_quant_kernel, 200 * 1024, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "rms_quant attribute: %s", cudaGetErrorString(e));
  rms_quant_kernel<<<m, QUANT_THREADS, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), x_row_stride, static_cast<const __nv_bfloat16*>(rms_delta), eps, row_map,
      k, static_cast<int8_t*>(xq), sx, static_cast<__nv_bfloat16*>(xn));
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "rms_quant launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// Per-token int8 quantisation of rows whose absmax is already known (the GEMM that produced the rows
// collected it in its epilogue): nothing is row-wide any more, so every thread streams two 8-element
// vectors, HBM in -> codes out, with no shared memory and no barrier.  Same arithmetic as
// rms_quant_kernel (scale = amax / 127 or 1, exact rint(x / scale)).
__global__ void __launch_bounds__(256)
quant_stream_kernel(const uint4* __restrict__ x, const float* __restrict__ row_amax, int nvec, int64_t total_vecs,
                    uint2* __restrict__ xq, float* __restrict__ sx) {
  const int64_t v0 = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) * 2;
  if (v0 >= total_vecs) return;
  const bool two = v0 + 1 < total_vecs;
  const uint4 u0 = __ldg(x + v0);
  const uint4 u1 = two ? __ldg(x + v0 + 1) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (i == 1 && !two) break;
    const int64_t v = v0 + i;
    const int64_t row = v / nvec;
    const float amax = __ldg(row_amax + row);
    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float rcp = quant_rcp(scale);
    if (v - row * nvec == 0) sx[row] = scale;
    const uint4 u = i == 0 ? u0 : u1;
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    int q[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      q[2 * j] = quant_code(bf16_lo(w[j]), scale, rcp);
      q[2 * j + 1] = quant_code(bf16_hi(w[j]), scale, rcp);
    }
    xq[v] = make_uint2(pack_codes4(q[0], q[1], q[2], q[3]), pack_codes4(q[4], q[5], q[6], q[7]));
  }
}

int launch_quant_stream(const void* x, const float* row_amax, int m, int k, void* xq, float* sx, cudaStream_t stream) {
  if (x == nullptr || row_amax == nullptr || xq == nullptr || sx == nullptr || m <= 0 || k <= 0 || k % 16 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "quant_stream: null buffer or bad shape");
  if (!aligned16(x) || !aligned16(xq) || x == xq)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "quant_stream: buffers must be distinct and 16-byte aligned");
  const int nvec = k >> 3;
  const int64_t total = static_cast<int64_t>(m) * nvec;
  const int64_t ctas = (total + 511) / 512;
  if (ctas > 0x7fffffffll) return fail(SKYRL_ERR_UNSUPPORTED, "quant_stream: too many rows");
  quant_stream_kernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(static_cast<const uint4*>(x), row_amax, nvec, total,
                                                                      static_cast<uint2*>(xq), sx);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "quant_stream launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// ----------------------------------------------------------------------------
// Row-parallel finalize: out[perm[i]] = bf16(bf16(sum[i]) + residual[perm[i]]).
// The two roundings are the reference's: the projection is cast to bf16 once
// (quantized_lora.py:304) and the residual add is a bf16 add (qwen3_5.py:784).
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
tp_finalize_kernel(const float* __restrict__ reduced, const int32_t* __restrict__ perm,
                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int hidden,
                   int row_begin, int out_sorted) {
  const int64_t srow = row_begin + blockIdx.x;
  const int64_t orow = perm != nullptr ? perm[srow] : srow;
  const float4* src = reinterpret_cast<const float4*>(reduced + srow * hidden);
  const uint4* res = reinterpret_cast<const uint4*>(residual + orow * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (out_sorted ? srow : orow) * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    const float4 a = __ldg(src + 2 * v), b = __ldg(src + 2 * v + 1);
    const uint4 r = __ldg(res + v);
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(__fadd_rn(round_bf16(f[2 * j]), bf16_lo(rw[j])),
                         __fadd_rn(round_bf16(f[2 * j + 1]), bf16_hi(rw[j])));
    dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int launch_tp_finalize(const float* reduced, const int32_t* perm, const void* residual, void* out, int hidden,
                       int row_begin, int row_count, cudaStream_t stream, bool out_sorted) {
  if (residual == nullptr || !aligned16(reduced) || !aligned16(residual) || !aligned16(out))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize: residual missing or buffers not 16-byte aligned");
  tp_finalize_kernel<<<row_count, 256, 0, stream>>>(reduced, perm, static_cast<const __nv_bfloat16*>(residual),
                                                    static_cast<__nv_bfloat16*>(out), hidden, row_begin,
                                                    out_sorted ? 1 : 0);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_finalize launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// The same with the ranks' partial sums still apart: slab s holds rank s's fp32 partial sums of the rows
// [row_begin, row_begin + gridDim.x), each rank having stored them into this GPU's memory from its down
// GEMM epilogue.  Added in ascending rank order in fp32 (quantized_lora.py:253), then as above.
struct SlabList {
  const float* slab[8];
  int count;
};

__global__ void __launch_bounds__(256)
tp_finalize_slabs_kernel(const SlabList slabs, const int32_t* __restrict__ perm,
                         const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int hidden,
                         int row_begin, int out_sorted) {
  const int64_t srow = row_begin + blockIdx.x;
  const int64_t orow = perm != nullptr ? perm[srow] : srow;
  const int64_t off = static_cast<int64_t>(blockIdx.x) * hidden;
  const uint4* res = reinterpret_cast<const uint4*>(residual + orow * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (out_sorted ? srow : orow) * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    const float4* src = reinterpret_cast<const float4*>(slabs.slab[0] + off);
    float4 a = __ldg(src + 2 * v), b = __ldg(src + 2 * v + 1);
    for (int s = 1; s < slabs.count; ++s) {
      src = reinterpret_cast<const float4*>(slabs.slab[s] + off);
      const float4 c = __ldg(src + 2 * v), d = __ldg(src + 2 * v + 1);
      a.x = __fadd_rn(a.x, c.x); a.y = __fadd_rn(a.y, c.y); a.z = __fadd_rn(a.z, c.z); a.w = __fadd_rn(a.w, c.w);
      b.x = __fadd_rn(b.x, d.x); b.y = __fadd_rn(b.y, d.y); b.z = __fadd_rn(b.z, d.z); b.w = __fadd_rn(b.w, d.w);
    }
    const uint4 r = __ldg(res + v);
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(__fadd_rn(round_bf16(f[2 * j]), bf16_lo(rw[j])),
                         __fadd_rn(round_bf16(f[2 * j + 1]), bf16_hi(rw[j])));
    dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int launch_tp_finalize_slabs(const float* const* slabs, int num_slabs, const int32_t* perm, const void* residual,
                             void* out, int hidden, int row_begin, int row_count, cudaStream_t stream, bool out_sorted) {
  if (slabs == nullptr || num_slabs < 1 || num_slabs > 8)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: 1 to 8 slabs wanted, got %d", num_slabs);
  SlabList list = {};
  list.count = num_slabs;
  for (int s = 0; s < num_slabs; ++s) {
    if (slabs[s] == nullptr || !aligned16(slabs[s]))
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: slab %d is null or not 16-byte aligned", s);
    list.slab[s] = slabs[s];
  }
  if (residual == nullptr || !aligned16(residual) || !aligned16(out))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "tp_finalize_slabs: residual missing or buffers not 16-byte aligned");
  tp_finalize_slabs_kernel<<<row_count, 256, 0, stream>>>(list, perm, static_cast<const __nv_bfloat16*>(residual),
                                                          static_cast<__nv_bfloat16*>(out), hidden, row_begin,
                                                          out_sorted ? 1 : 0);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "tp_finalize_slabs launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// Self-test of the bounded wait every kernel of this library uses: one CTA waits on an mbarrier that
// nothing ever arrives at, for `limit_ns`.  The wait gives up, writes its code into the status word and
// the kernel returns normally; the context stays usable.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int32_t* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  mbar_wait(&bar, 0u, &abort_flag, status, STATUS_SELFTEST_TIMEOUT, limit_ns);
}

int launch_bounded_wait_selftest(int32_t* status, unsigned long long limit_ns, cudaStream_t stream) {
  if (status == nullptr || limit_ns == 0 || limit_ns > WAIT_LIMIT_NS)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "selftest: status must be non-null and the limit within (0, 2 s]");
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "selftest launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// Rows of a bf16 [m, hidden] matrix in adapter-sorted order back to token order: out[perm[i]] = in[i].
__global__ void __launch_bounds__(256)
unsort_rows_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ perm, uint4* __restrict__ out, int vecs) {
  const int64_t srow = blockIdx.x;
  const int64_t orow = perm != nullptr ? perm[srow] : srow;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) out[orow * vecs + v] = __ldg(in + srow * vecs + v);
}

int launch_unsort_rows(const void* sorted_rows, const int32_t* perm, void* out, int m, int hidden, cudaStream_t stream) {
  if (sorted_rows == nullptr || out == nullptr || sorted_rows == out || !aligned16(sorted_rows) || !aligned16(out) ||
      hidden % 8 != 0 || m <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "unsort_rows: distinct 16-byte aligned buffers and hidden % 8 == 0 wanted");
  unsort_rows_kernel<<<m, 256, 0, stream>>>(static_cast<const uint4*>(sorted_rows), perm, static_cast<uint4*>(out),
                                            hidden / 8);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "unsort_rows launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

// ----------------------------------------------------------------------------
// Grouped weights (group_size < K, the reference's native format): the caller
// runs one single-group GEMM per K group into fp32 slabs (f32(acc) * sx_g) * sw_g;
// this kernel adds the slabs in ascending group order, as the reference's
// `sum(scaled, axis=1)` does (skyrl/tx/kernels/quantized_lora.py:248-253), casts
// once to bf16 and scatters rows back to token order.
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
group_sum_cast_kernel(const float* __restrict__ slabs, int groups, int64_t slab_stride, int n,
                      const int32_t* __restrict__ row_map, __nv_bfloat16* __restrict__ out, int64_t out_stride) {
  const int64_t srow = blockIdx.x;
  const int64_t orow = row_map != nullptr ? row_map[srow] : srow;
  for (int c = threadIdx.x * 2; c < n; c += 2 * blockDim.x) {
    float2 acc = *reinterpret_cast<const float2*>(slabs + srow * n + c);
    for (int g = 1; g < groups; ++g) {
      const float2 t = *reinterpret_cast<const float2*>(slabs + g * slab_stride + srow * n + c);
      acc.x = __fadd_rn(acc.x, t.x);
      acc.y = __fadd_rn(acc.y, t.y);
    }
    *reinterpret_cast<uint32_t*>(out + orow * out_stride + c) = pack_bf16x2(acc.x, acc.y);
  }
}

// ----------------------------------------------------------------------------
// Pack kernels (load time).  Tiled transposes through shared memory.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols,
                                 int64_t in_batch, int64_t out_batch, int out_pitch) {
  // in [B, rows, cols] -> out [B, cols, out_pitch] with out[b, c, r] = in[b, r, c]; out is pre-zeroed.
  __shared__ T tile[32][33];
  const T* ib = in + blockIdx.z * in_batch;
  T* ob = out + blockIdx.z * out_batch;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = ib[static_cast<int64_t>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) ob[static_cast<int64_t>(c) * out_pitch + r] = tile[threadIdx.x][j];
  }
}

// Weight codes in the K-block-major device layout [ceil(K / 128), N, 128]: for one 128-byte block of K
// the rows of all output channels lie back to back, so the TMA box of ANY run of output channels is
// one contiguous piece of HBM (K zero-padded to the block).
__global__ void pack_weight_kn_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int k, int n) {
  // in [K, N] (reference layout) -> out[kb][n][kk] = in[kb * 128 + kk][n]
  __shared__ int8_t tile[32][33];
  const int kb = blockIdx.z;
  const int n0 = blockIdx.x * 32, kk0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int kg = kb * SKYRL_WEIGHT_KBLOCK + kk0 + j, nn = n0 + threadIdx.x;
    tile[j][threadIdx.x] = (kg < k && nn < n) ? in[static_cast<int64_t>(kg) * n + nn] : int8_t(0);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int nn = n0 + j, kk = kk0 + threadIdx.x;
    if (nn < n) out[(static_cast<int64_t>(kb) * n + nn) * SKYRL_WEIGHT_KBLOCK + kk] = tile[threadIdx.x][j];
  }
}

__global__ void pack_weight_nk_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int n, int k,
                                      int64_t vecs) {
  // in [N, K] (K contiguous) -> out[kb][n][kk]; 16-byte vectors
  const int vpb = SKYRL_WEIGHT_KBLOCK / 16;
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < vecs;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int q = static_cast<int>(v % vpb);
    const int64_t row = v / vpb;  // kb * n + nn
    const int nn = static_cast<int>(row % n);
    const int kb = static_cast<int>(row / n);
    const int kg = kb * SKYRL_WEIGHT_KBLOCK + q * 16;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (kg < k) val = __ldg(reinterpret_cast<const uint4*>(in + static_cast<int64_t>(nn) * k + kg));
    reinterpret_cast<uint4*>(out)[v] = val;
  }
}

template <typename T>
static int run_transpose(const T* in, T* out, int batch, int rows, int cols, int64_t out_batch, int out_pitch,
                         size_t out_bytes, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(out, 0, out_bytes, stream);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "pack memset: %s", cudaGetErrorString(e));
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
  if (grid.y > 65535 || grid.z > 65535) return fail(SKYRL_ERR_UNSUPPORTED, "pack: shape exceeds the launch grid");
  transpose_kernel<T><<<grid, block, 0, stream>>>(in, out, rows, cols, static_cast<int64_t>(rows) * cols, out_batch,
                                                   out_pitch);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "pack launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

}  // namespace skyrl

using namespace skyrl;

extern "C" int skyrl_pack_weight_kn_sm100_v1(const void* codes_kn, int32_t k, int32_t n, void* wq_blocked,
                                             skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (codes_kn == nullptr || wq_blocked == nullptr || k <= 0 || n <= 0 || codes_kn == wq_blocked)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_weight_kn: null/aliased buffer or non-positive shape");
  const int kb = (k + SKYRL_WEIGHT_KBLOCK - 1) / SKYRL_WEIGHT_KBLOCK;
  cudaError_t e = cudaMemsetAsync(wq_blocked, 0, static_cast<size_t>(kb) * n * SKYRL_WEIGHT_KBLOCK, stream);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "pack memset: %s", cudaGetErrorString(e));
  dim3 grid((n + 31) / 32, SKYRL_WEIGHT_KBLOCK / 32, kb), block(32, 8);
  if (grid.z > 65535) return fail(SKYRL_ERR_UNSUPPORTED, "pack_weight_kn: K exceeds the launch grid");
  pack_weight_kn_kernel<<<grid, block, 0, stream>>>(static_cast<const int8_t*>(codes_kn), static_cast<int8_t*>(wq_blocked),
                                                     k, n);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "pack_weight_kn launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

extern "C" int skyrl_pack_weight_nk_sm100_v1(const void* codes_nk, int32_t n, int32_t k, void* wq_blocked,
                                             skyrl_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (codes_nk == nullptr || wq_blocked == nullptr || k <= 0 || n <= 0 || codes_nk == wq_blocked)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_weight_nk: null/aliased buffer or non-positive shape");
  if (k % 16 != 0 || !aligned16(codes_nk) || !aligned16(wq_blocked))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_weight_nk: K must be a multiple of 16 and buffers 16-byte aligned");
  const int kb = (k + SKYRL_WEIGHT_KBLOCK - 1) / SKYRL_WEIGHT_KBLOCK;
  const int64_t vecs = static_cast<int64_t>(kb) * n * (SKYRL_WEIGHT_KBLOCK / 16);
  const int blocks = static_cast<int>((vecs + 255) / 256 < 148 * 32 ? (vecs + 255) / 256 : 148 * 32);
  pack_weight_nk_kernel<<<blocks, 256, 0, stream>>>(static_cast<const int8_t*>(codes_nk),
                                                    static_cast<int8_t*>(wq_blocked), n, k, vecs);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "pack_weight_nk launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

extern "C" int skyrl_pack_lora_a_sm100_v1(const void* a_akr, int32_t num_adapters, int32_t k, int32_t rank,
                                          void* a_packed, skyrl_stream_t stream) {
  if (a_akr == nullptr || a_packed == nullptr || num_adapters <= 0 || k <= 0 || rank <= 0 || a_akr == a_packed)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_lora_a: null/aliased buffer or non-positive shape");
  if (rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "pack_lora_a: rank %d exceeds %d", rank, SKYRL_LORA_RANK_PAD);
  // per adapter: in [K, r] -> out [64, K] (rows >= r stay zero)
  return run_transpose<uint16_t>(static_cast<const uint16_t*>(a_akr), static_cast<uint16_t*>(a_packed), num_adapters,
                                 k, rank, static_cast<int64_t>(SKYRL_LORA_RANK_PAD) * k, k,
                                 static_cast<size_t>(num_adapters) * SKYRL_LORA_RANK_PAD * k * 2,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_pack_lora_b_sm100_v1(const void* b_arn, int32_t num_adapters, int32_t rank, int32_t n,
                                          void* b_packed, skyrl_stream_t stream) {
  if (b_arn == nullptr || b_packed == nullptr || num_adapters <= 0 || n <= 0 || rank <= 0 || b_arn == b_packed)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_lora_b: null/aliased buffer or non-positive shape");
  if (rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "pack_lora_b: rank %d exceeds %d", rank, SKYRL_LORA_RANK_PAD);
  // per adapter: in [r, N] -> out [N, 64] (columns >= r stay zero)
  return run_transpose<uint16_t>(static_cast<const uint16_t*>(b_arn), static_cast<uint16_t*>(b_packed), num_adapters,
                                 rank, n, static_cast<int64_t>(n) * SKYRL_LORA_RANK_PAD, SKYRL_LORA_RANK_PAD,
                                 static_cast<size_t>(num_adapters) * n * SKYRL_LORA_RANK_PAD * 2,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_pack_lora_b_rows_sm100_v1(const void* b_arn, int32_t num_adapters, int32_t rank, int32_t n,
                                               void* b_rows, skyrl_stream_t stream) {
  if (b_arn == nullptr || b_rows == nullptr || num_adapters <= 0 || n <= 0 || rank <= 0 || b_arn == b_rows)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "pack_lora_b_rows: null/aliased buffer or non-positive shape");
  if (rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "pack_lora_b_rows: rank %d exceeds %d", rank, SKYRL_LORA_RANK_PAD);
  const int rr = (rank + 7) / 8 * 8;
  return run_transpose<uint16_t>(static_cast<const uint16_t*>(b_arn), static_cast<uint16_t*>(b_rows), num_adapters,
                                 rank, n, static_cast<int64_t>(n) * rr, rr,
                                 static_cast<size_t>(num_adapters) * n * rr * 2, static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_group_sum_cast_sm100_v1(const float* slabs, int32_t groups, int32_t m, int32_t n,
                                             const int32_t* row_map, void* out, int64_t out_row_stride,
                                             skyrl_stream_t stream) {
  if (slabs == nullptr || out == nullptr || groups <= 0 || m <= 0 || n <= 0 || n % 2 != 0 || out_row_stride < n)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "group_sum_cast: null buffer or bad shape");
  group_sum_cast_kernel<<<m, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      slabs, groups, static_cast<int64_t>(m) * n, n, row_map, static_cast<__nv_bfloat16*>(out), out_row_stride);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "group_sum_cast launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

extern "C" int skyrl_w8a8_bounded_wait_selftest_sm100_v1(int32_t* status, uint64_t limit_ns, skyrl_stream_t stream) {
  return skyrl::launch_bounded_wait_selftest(status, limit_ns, static_cast<cudaStream_t>(stream));
}

extern "C" int skyrl_lora_route_sm100_v1(const int32_t* adapter_ids, int32_t m, int32_t num_adapters, int32_t* perm,
                                         int32_t* tiles, int32_t* num_tiles, int32_t max_tiles, int32_t* status,
                                         skyrl_stream_t stream) {
  return launch_route(adapter_ids, m, num_adapters, perm, tiles, num_tiles, max_tiles, status,
                      static_cast<cudaStream_t>(stream), 0, 0, nullptr, 0);
}

extern "C" int skyrl_rms_quant_sm100_v1(const void* x, int64_t x_row_stride, const void* rms_delta, float eps,
                                        const int32_t* row_map, int32_t m, int32_t k, void* xq, float* sx, void* xn,
                                        skyrl_stream_t stream) {
  return launch_rms_quant(x, x_row_stride, rms_delta, eps, row_map, m, k, xq, sx, xn,
                          static_cast<cudaStream_t>(stream));
}
