// Persistent, warp-specialised W8A8 GEMM with fused dequant / LoRA-B / SwiGLU /
// residual epilogue for sm_100a.
//
//   acc[m, n]  = sum_k xq[m, k] * wq[n, k]                (tcgen05.mma kind::i8, int32 in TMEM)
//   v[m, n]    = (f32(acc) * sx[m]) * sw[n]               (skyrl/tx/kernels/quantized_lora.py:248-252)
//   v[m, n]   += sum_j z[m, j] * B[a(m)][n, j]            (tcgen05.mma kind::f16 onto the SAME TMEM
//                                                          columns, z = three bf16 planes, quantized_lora.py:301-304)
//   out        = epilogue(v)                              (one bf16 cast, then SwiGLU / residual)
//
// Roles (320 threads): warps 0-3 and 6-9 drain TMEM (warp w owns TMEM lanes
// 32 (w % 4) .. +31; the two warps of a lane quadrant split the tile's columns,
// and two warps per scheduler hide each other's latencies in the SwiGLU math),
// warp 4 is the TMA producer, warp 5 issues the MMAs and owns the TMEM
// allocation.  Two accumulator stages of BN columns let the epilogue of tile t
// overlap the main loop of tile t+1.  The LoRA term does not get accumulator
// columns of its own (2 x 256 int32 columns already fill the 512-column TMEM):
// the epilogue rewrites the int32 accumulator in place as dequantised fp32,
// the MMA warp then issues the rank-r bf16 MMAs that accumulate z @ B^T onto
// it, and the tile is read back a second time for the final cast.  The LoRA
// operands (three z planes, one B tile) have no shared memory of their own
// either: they travel through two slots of the same TMA pipeline, injected
// into the stream of the NEXT tile's K blocks, so the whole buffer serves
// pipeline depth (the main loop is bound by bytes in flight per SM).
//
// Rows live in the adapter-sorted space: every 128-row M tile comes from the
// tile list and holds rows of at most two adapters (each row's z is zero in the
// slot of the adapter that is not its own); rows past the tile's count are
// computed but never stored.  Every wait is bounded (see ptx_sm100.cuh).
#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace skyrl {

constexpr int BM = 128;       // rows per tile == TMEM lanes
constexpr int BK = 128;       // int8 elements (bytes) of K per pipeline stage: one 128-byte swizzled row
constexpr int UMMA_K_I8 = 32; // K of one kind::i8 instruction
constexpr int GEMM_THREADS = 320;  // warps 0-3 and 6-9 epilogue, warp 4 TMA producer, warp 5 MMA issuer
constexpr int EPI_THREADS = 256;
constexpr int LORA_ROW_BYTES = SKYRL_LORA_RANK_PAD * 2;  // 128-byte rows of z and packed B

constexpr int STAGE_AREA_BYTES = 224 * 1024;  // shared memory given to the TMA pipeline stages
constexpr int EPI_STAGE_PITCH = 80;           // bytes per row of an epilogue warp's bf16 store-staging tile (64 + pad)
constexpr int EPI_STAGE_BYTES = 32 * 128;     // the fp32 form holds 32 rows x 128 bytes, swizzled instead of padded
// the single-tile kernel carves eight such tiles out of the top of the stage area
constexpr int SINGLE_STAGE_AREA = STAGE_AREA_BYTES - 8 * EPI_STAGE_BYTES;
constexpr int MAX_STAGES = 12;
constexpr int Z_PLANE_BYTES = BM * LORA_ROW_BYTES;  // one bf16 plane of z for a tile: 128 rows x 128 bytes
constexpr int LORA_INJECT_AFTER = 8;  // K blocks of the next tile issued before the previous tile's LoRA operands

template <int BN>
struct GemmCfg {
  static constexpr int BAR_OFF = STAGE_AREA_BYTES;
  static constexpr int NUM_BARS = 2 * MAX_STAGES + 4 + 2;
  static constexpr int SMEM_BYTES = BAR_OFF + NUM_BARS * 8 + 16 + 128 + 1024;  // + tmem ptr/abort, tile ring, alignment slack
  static constexpr int TMEM_COLS = 2 * BN;
};

struct GemmParams {
  CUtensorMap tm_xq;   // int8 [M, K], box 128 x 128
  CUtensorMap tm_w;    // int8 [K / 128, N, 128], box 128 x bn_eff x 1
  CUtensorMap tm_z;    // bf16 [M, 6, 64], box 64 x 1 x 128 (one part of one adapter slot of one tile's rows)
  CUtensorMap tm_b;    // bf16 [A, N, 64], box 64 x BN x 1
  const float* sx;
  const float* sw;
  const int4* tiles;
  const int32_t* num_tiles;
  const int32_t* out_row_map;
  const __nv_bfloat16* residual;
  void* out;
  int64_t out_stride;
  int64_t res_stride;
  int32_t* status;
  int m, n, k;
  int rank_blocks;  // ceil(rank / 16) MMAs per z plane
  int band;         // M tiles per raster band
  int bn_eff;       // columns per N tile actually used (multiple of 16, <= BN): MMA N, TMA box rows
  int num_stages;   // pipeline depth and byte pitch of one stage (A tile + bn_eff weight rows)
  int stage_bytes;
  int k_splits;     // > 1: each tile covers kb_per_split K blocks and writes its int32 partial sums to slab (t % k_splits)
  int kb_per_split;
  int64_t slab_stride;  // elements between slabs of the int32 output
  int a_rows;       // rows of the activation TMA box (64 when the batch has at most 64 rows, else 128)
  int* sched;       // {tile claim counter, finished-CTA counter} of this launch, both zero on entry
  int direct_stores;  // tuning aid: 1 = bf16 epilogues store from registers instead of through the staging tile
  // Row scatter of the fp32 partial sums (tensor-parallel reduce-scatter folded into the epilogue): row i of
  // the sorted order belongs to owner o = (i - scatter_row0) / scatter_rows and is written to
  // scatter_base[o] + (i - scatter_row0 - o * scatter_rows) * out_stride, which may be another GPU's memory
  // (plain stores over NVLink).  scatter_rows == 0: rows go to `out`.
  float* scatter_base[8];
  int scatter_row0;
  int scatter_rows;
  // SwiGLU epilogue: absmax of every output row, collected with atomicMax on the bit pattern (the values
  // are >= 0) so that the quantiser of the next projection needs no pass of its own to find it.
  // Indexed by sorted row; the caller zeroes it before the launch.  NULL: not collected.
  float* row_amax;
  // Small-batch LoRA (ROWS kernels, at most 128 rows in token order, every row with its own adapter): the
  // epilogue warps evaluate l[m, n] = sum_j z[m, j] * B[a(m)][n, j] on the CUDA cores into a shared-memory
  // tile WHILE the main loop streams the weights, and the epilogue proper adds it to the dequantised
  // accumulator before the single cast.  z comes from rms_quant_rows_kernel (fp32 [m, 64], already scaled),
  // B from the dense table [A, n, lora_rank_vecs * 8].
  const float* z_rows;
  const int32_t* row_ids;      // adapter id per row, NULL = adapter 0
  const __nv_bfloat16* b_rows;
  int64_t b_adapter_stride;    // elements between adapters of b_rows
  int b_row_stride;            // elements between output channels of b_rows
  int lora_rank_vecs;          // 8-element vectors of the rank that are used, 0 = no LoRA term
  int num_adapters;
  int profile;                 // 1: the MMA issuer of CTA 0 adds the cycles it spent waiting to status[1..3]
  int lterm_off;               // byte offset of the l tile inside the stage area
  int lterm_pitch;             // floats per row of the l tile (odd, so that a column is conflict-free)
  const unsigned char* prefetch;  // bytes another kernel will stream soon: requested into L2 once the own loads are out
  long long prefetch_bytes;
};

// The producer's last act: this CTA's share of the prefetch range, in pieces interleaved over the grid so
// that the range arrives roughly front to back (the order its consumer reads it in).
__device__ __forceinline__ void prefetch_share_to_l2(const GemmParams& p) {
  constexpr long long PIECE = 16384;
  const long long pieces = (p.prefetch_bytes + PIECE - 1) / PIECE;
  for (long long i = blockIdx.x; i < pieces; i += gridDim.x) {
    const long long off = i * PIECE;
    const uint32_t bytes = static_cast<uint32_t>(min(PIECE, p.prefetch_bytes - off));
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.prefetch + off), "r"(bytes) : "memory");
  }
}

// NULL (and status STATUS_BAD_SCATTER) for a row that has no owner: the caller skips the store.
__device__ __forceinline__ float* partial_row_ptr(const GemmParams& p, int64_t orow) {
  if (p.scatter_rows > 0) {
    const int rel = static_cast<int>(orow) - p.scatter_row0;
    const int o = rel >= 0 ? rel / p.scatter_rows : 8;
    float* base = o < 8 ? p.scatter_base[o] : nullptr;
    if (base == nullptr) {
      atomicCAS(p.status, 0, STATUS_BAD_SCATTER);
      return nullptr;
    }
    return base + static_cast<int64_t>(rel - o * p.scatter_rows) * p.out_stride;
  }
  return static_cast<float*>(p.out) + orow * p.out_stride;
}

// ---- dynamic tile scheduler --------------------------------------------------------------------------
// Tiles are claimed from a global counter instead of a fixed stride, so a CTA that starts late (its SM
// was held by another stream's kernel, e.g. a collective) simply takes fewer tiles.  The producer thread
// claims tile numbers and hands them to the MMA and epilogue roles through a 4-slot ring in shared memory.
constexpr int SCHED_SLOTS = 4;
struct TileRing {
  uint64_t full[SCHED_SLOTS];
  uint64_t empty[SCHED_SLOTS];
  int tile[SCHED_SLOTS];
};
__device__ __forceinline__ int sched_claim(TileRing* ring, uint32_t it, int* counter, int total,
                                           volatile int* abort_flag, int* status, bool& ok) {
  const uint32_t slot = it & (SCHED_SLOTS - 1);
  ok = mbar_wait(&ring->empty[slot], ((it / SCHED_SLOTS) & 1u) ^ 1u, abort_flag, status, STATUS_TIMEOUT_PRODUCER);
  if (!ok) return -1;
  int t = atomicAdd(counter, 1);
  if (t >= total) t = -1;
  ring->tile[slot] = t;
  mbar_arrive(&ring->full[slot]);  // release: the tile number is visible to whoever observes the phase
  return t;
}
__device__ __forceinline__ int sched_read(TileRing* ring, uint32_t it, volatile int* abort_flag, int* status,
                                          int code, bool& ok) {
  const uint32_t slot = it & (SCHED_SLOTS - 1);
  ok = mbar_wait(&ring->full[slot], (it / SCHED_SLOTS) & 1u, abort_flag, status, code);
  return ok ? ring->tile[slot] : -1;
}
__device__ __forceinline__ void sched_release(TileRing* ring, uint32_t it) {
  mbar_arrive(&ring->empty[it & (SCHED_SLOTS - 1)]);
}
// The last CTA of a launch puts the claim counter back to zero for the slot's next user.
__device__ __forceinline__ void sched_finish(int* sched) {
  if (atomicAdd(sched + 1, 1) == static_cast<int>(gridDim.x) - 1) {
    sched[0] = 0;
    sched[1] = 0;
    __threadfence();
  }
}

// Where the MMA issuer's time goes (diagnostic, CTA 0 only): cycles waiting for operands in shared memory,
// for a free accumulator stage, and for the epilogue's rewrite of the accumulator in front of the LoRA MMAs.
struct IssuerProfile {
  long long operands = 0, accumulator = 0, rewrite = 0;
};
__device__ __forceinline__ bool timed_wait(bool on, long long& acc, uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           int* status, int code) {
  if (!on) return mbar_wait(bar, parity, abort_flag, status, code);
  const long long t0 = clock64();
  const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
  acc += clock64() - t0;
  return ok;
}
__device__ __forceinline__ void store_profile(const IssuerProfile& pr, int* status, long long total) {
  // in units of 1024 cycles, so that a long launch fits an int32 word; the caller's status word [0] is untouched
  atomicAdd(status + 1, static_cast<int>(pr.operands >> 10));
  atomicAdd(status + 2, static_cast<int>((pr.accumulator + pr.rewrite) >> 10));
  atomicAdd(status + 3, static_cast<int>(total >> 10));
}

struct TileCoord {
  int m_idx, n_idx;
};
// Raster order: bands of `band` M tiles; inside a band the M index runs fastest,
// so CTAs running at the same time share few distinct weight tiles and the
// activation band stays L2-resident while the weights stream past once.
__device__ __forceinline__ TileCoord tile_coord(int t, int tm, int tn, int band) {
  const int per_band = band * tn;
  const int b = t / per_band;
  const int rem = t - b * per_band;
  const int rows = min(band, tm - b * band);
  TileCoord c;
  c.n_idx = rem / rows;
  c.m_idx = b * band + (rem - c.n_idx * rows);
  return c;
}

__device__ __forceinline__ float silu_f32(float t) { return __fdiv_rn(t, 1.0f + expf(-t)); }


// ---- epilogue building blocks (one 32-column chunk of one TMEM lane quadrant) ------------------------
// pass 1 of the LoRA path: int32 accumulator -> (f32(acc) * sx[m]) * sw[n], written back in place
__device__ __forceinline__ void epi_convert_chunk(uint32_t taddr, int nc, int n_end, float sxr,
                                                  const float* __restrict__ sw) {
  uint32_t v[32];
  __syncwarp();
  tmem_ld32(taddr, v);
  tmem_wait_ld();
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (nc + g * 4 < n_end) w = __ldg(reinterpret_cast<const float4*>(sw + nc) + g);
    v[4 * g + 0] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 0])), sxr), w.x));
    v[4 * g + 1] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 1])), sxr), w.y));
    v[4 * g + 2] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 2])), sxr), w.z));
    v[4 * g + 3] = __float_as_uint(__fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 3])), sxr), w.w));
  }
  tmem_st32(taddr, v);
}

// Row r of an epilogue warp's chunk is held by lane r, so a register store instruction touches 32 rows
// with 16 bytes each: half sectors, scattered.  With a staging tile the warp transposes the chunk and
// every store instruction writes whole 32- or 64-byte runs of 8 or 16 rows (and reads the residual the
// same way).  `stage` == nullptr keeps the direct form.
__device__ __forceinline__ void epi_staged_store(unsigned char* stage, int lane, const uint32_t* packed, int words,
                                                 bool row_valid, int64_t orow, __nv_bfloat16* out, int64_t out_stride,
                                                 int col0, int cols_valid, const __nv_bfloat16* residual,
                                                 int64_t res_stride) {
  // `words` 32-bit words (2 bf16 each) per row: 16 (64 bytes) or 8 (32 bytes)
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * EPI_STAGE_PITCH);
  for (int q = 0; q < words / 4; ++q) mine[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
  __syncwarp();
  const int pieces = words / 4;            // 16-byte pieces per row: 4 or 2
  const int rows_per_round = 32 / pieces;  // 8 or 16
  const int piece = lane % pieces, sub = lane / pieces;
  const int orow_lo = static_cast<int>(orow & 0xffffffffll), orow_hi = static_cast<int>(orow >> 32);
  for (int round = 0; round < pieces; ++round) {
    const int r = sub + round * rows_per_round;
    const bool valid = __shfl_sync(0xffffffffu, row_valid ? 1 : 0, r) != 0;
    const int lo = __shfl_sync(0xffffffffu, orow_lo, r), hi = __shfl_sync(0xffffffffu, orow_hi, r);
    if (valid && piece * 8 < cols_valid) {
      const int64_t row = (static_cast<int64_t>(hi) << 32) | static_cast<uint32_t>(lo);
      uint4 v = *reinterpret_cast<const uint4*>(stage + r * EPI_STAGE_PITCH + piece * 16);
      if (residual != nullptr) {
        const uint4 rv = __ldg(reinterpret_cast<const uint4*>(residual + row * res_stride + col0 + piece * 8));
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
        uint32_t o[4];
#pragma unroll
        for (int j2 = 0; j2 < 4; ++j2)
          o[j2] = pack_bf16x2(__fadd_rn(bf16_lo(vw[j2]), bf16_lo(rw[j2])), __fadd_rn(bf16_hi(vw[j2]), bf16_hi(rw[j2])));
        v = make_uint4(o[0], o[1], o[2], o[3]);
      }
      *reinterpret_cast<uint4*>(out + row * out_stride + col0 + piece * 8) = v;
    }
  }
  __syncwarp();
}

// pass 2: final values of one chunk -> global memory (single bf16 cast, SwiGLU / residual / raw forms)
template <int EPI, bool HAS_LORA>
__device__ __forceinline__ void epi_store_chunk(const GemmParams& p, uint32_t taddr, int nc, int n_end, float sxr,
                                                bool row_valid, int64_t orow, int64_t slab_off,
                                                unsigned char* stage = nullptr, int lane = 0,
                                                float* amax_acc = nullptr, const float* lrow = nullptr) {
  uint32_t v[32];
  __syncwarp();
  tmem_ld32(taddr, v);
  tmem_wait_ld();
  if (EPI == SKYRL_EPI_ACC_I32) {
    if (row_valid) {
      // split K: every split owns one [M, N] slab; the consumer adds the slabs (exact in int32)
      int4* dst = reinterpret_cast<int4*>(static_cast<int32_t*>(p.out) + slab_off + orow * p.out_stride + nc);
#pragma unroll
      for (int g = 0; g < 8; ++g)
        if (nc + g * 4 < n_end) dst[g] = make_int4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    }
    return;
  }
  float f[32];
  if (HAS_LORA) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
      if (nc + g * 4 < n_end) w = __ldg(reinterpret_cast<const float4*>(p.sw + nc) + g);
      f[4 * g + 0] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 0])), sxr), w.x);
      f[4 * g + 1] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 1])), sxr), w.y);
      f[4 * g + 2] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 2])), sxr), w.z);
      f[4 * g + 3] = __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int>(v[4 * g + 3])), sxr), w.w);
    }
    if (lrow != nullptr) {  // small-batch LoRA term of this row (this chunk's 32 columns), added before the cast
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __fadd_rn(f[i], lrow[i]);
    }
  }
  if (EPI == SKYRL_EPI_PARTIAL_F32) {
    if (stage != nullptr) {
      // transposed through the staging tile (16-byte pieces XOR-swizzled by row): eight lanes then write the
      // 128 contiguous bytes of one row, whole lines for local memory and for NVLink alike
      float4* tile = reinterpret_cast<float4*>(stage);
#pragma unroll
      for (int g = 0; g < 8; ++g)
        tile[lane * 8 + (g ^ (lane & 7))] = make_float4(f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3]);
      __syncwarp();
      const int piece = lane & 7, sub = lane >> 3;
      const int orow_lo = static_cast<int>(orow & 0xffffffffll), orow_hi = static_cast<int>(orow >> 32);
#pragma unroll
      for (int round = 0; round < 8; ++round) {
        const int r = sub + round * 4;
        const bool valid = __shfl_sync(0xffffffffu, row_valid ? 1 : 0, r) != 0;
        const int lo = __shfl_sync(0xffffffffu, orow_lo, r), hi = __shfl_sync(0xffffffffu, orow_hi, r);
        if (valid && nc + piece * 4 < n_end) {
          const int64_t row = (static_cast<int64_t>(hi) << 32) | static_cast<uint32_t>(lo);
          float* rowp = partial_row_ptr(p, row);
          if (rowp != nullptr) *reinterpret_cast<float4*>(rowp + nc + piece * 4) = tile[r * 8 + (piece ^ (r & 7))];
        }
      }
      __syncwarp();
      return;
    }
    if (!row_valid) return;
    float* rowp = partial_row_ptr(p, orow);
    if (rowp == nullptr) return;
    float4* dst = reinterpret_cast<float4*>(rowp + nc);
#pragma unroll
    for (int g = 0; g < 8; ++g)
      if (nc + g * 4 < n_end) dst[g] = make_float4(f[4 * g], f[4 * g + 1], f[4 * g + 2], f[4 * g + 3]);
    return;
  }
  if (stage != nullptr) {
    // staged form: every lane takes part (shuffles), invalid rows are masked at the store
    uint32_t o[16];
    if (EPI == SKYRL_EPI_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float h0 = __fmul_rn(silu_f32(round_bf16(f[4 * j])), round_bf16(f[4 * j + 1]));
        const float h1 = __fmul_rn(silu_f32(round_bf16(f[4 * j + 2])), round_bf16(f[4 * j + 3]));
        o[j] = pack_bf16x2(h0, h1);
        if (amax_acc != nullptr) {  // columns past the tile's end hold whatever TMEM held: leave them out
          if (nc + 4 * j < n_end) *amax_acc = fmaxf(*amax_acc, fabsf(h0));
          if (nc + 4 * j + 2 < n_end) *amax_acc = fmaxf(*amax_acc, fabsf(h1));
        }
      }
      epi_staged_store(stage, lane, o, 8, row_valid, orow, static_cast<__nv_bfloat16*>(p.out), p.out_stride, nc >> 1,
                       (n_end - nc) >> 1, nullptr, 0);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) o[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
      epi_staged_store(stage, lane, o, 16, row_valid, orow, static_cast<__nv_bfloat16*>(p.out), p.out_stride, nc,
                       n_end - nc, EPI == SKYRL_EPI_RESIDUAL ? p.residual : nullptr, p.res_stride);
    }
    return;
  }
  if (!row_valid) return;
  if (EPI == SKYRL_EPI_LINEAR) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + orow * p.out_stride + nc);
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (nc + g * 8 < n_end)
        dst[g] = make_uint4(pack_bf16x2(f[8 * g], f[8 * g + 1]), pack_bf16x2(f[8 * g + 2], f[8 * g + 3]),
                            pack_bf16x2(f[8 * g + 4], f[8 * g + 5]), pack_bf16x2(f[8 * g + 6], f[8 * g + 7]));
  } else if (EPI == SKYRL_EPI_RESIDUAL) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + orow * p.out_stride + nc);
    const uint4* res = reinterpret_cast<const uint4*>(p.residual + orow * p.res_stride + nc);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (nc + g * 8 < n_end) {
        const uint4 rv = __ldg(res + g);
        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = __fadd_rn(round_bf16(f[8 * g + 2 * j]), bf16_lo(rw[j]));
          const float b = __fadd_rn(round_bf16(f[8 * g + 2 * j + 1]), bf16_hi(rw[j]));
          o[j] = pack_bf16x2(a, b);
        }
        dst[g] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else if (EPI == SKYRL_EPI_SWIGLU) {
    // columns (2i, 2i+1) = (gate_i, up_i); 32 physical columns -> 16 outputs
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + orow * p.out_stride + (nc >> 1));
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      if (nc + g * 16 < n_end) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i0 = 16 * g + 4 * j;
          const float h0 = __fmul_rn(silu_f32(round_bf16(f[i0])), round_bf16(f[i0 + 1]));
          const float h1 = __fmul_rn(silu_f32(round_bf16(f[i0 + 2])), round_bf16(f[i0 + 3]));
          o[j] = pack_bf16x2(h0, h1);
          if (amax_acc != nullptr) {
            if (nc + i0 < n_end) *amax_acc = fmaxf(*amax_acc, fabsf(h0));
            if (nc + i0 + 2 < n_end) *amax_acc = fmaxf(*amax_acc, fabsf(h1));
          }
        }
        dst[g] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// l tile of the small-batch LoRA path for one output tile: l[r, c] = sum_j z[r, j] * B[a(r)][n0 + c, j] for
// rows [0, rows) x columns [n0, n_end), written by the eight epilogue warps while the main loop runs.
//
// Everything here is bound by memory latency (every row reads its own adapter's table), so the work is laid
// out for loads in flight, not for arithmetic: first the tile's adapter ids and z rows are staged in shared
// memory with one round of loads; then warp `ew` takes rows ew, ew + 8, ..., its lanes take consecutive
// columns (a warp-wide load is one contiguous run of one adapter's table), and the (rank vector q, row,
// column) items of a warp are processed in batches of ROWS_LORA_BATCH independent 16-byte loads per lane
// before any of them is used.  Per element the fmaf order is rank vector q ascending, then the eight ranks of
// the vector: the order of finalize_rows_kernel, so both give the same bits.
constexpr int ROWS_LORA_BATCH = 24;

__device__ __forceinline__ void rows_lora_tile(const GemmParams& p, float* lterm, int rows, int n0, int n_end, int ew,
                                               int lane, int epi_tid) {
  const int cols = n_end - n0;
  const int rank_floats = p.lora_rank_vecs * 8;
  const int rows_pad = p.a_rows;                                    // rows of the l tile (64 or 128)
  float* zs = lterm + rows_pad * p.lterm_pitch;                     // [rows_pad][rank_floats]
  int* ids_s = reinterpret_cast<int*>(zs + rows_pad * rank_floats);  // [rows_pad]
  // stage ids (clamped, reported) and z
  for (int r = epi_tid; r < rows; r += EPI_THREADS) {
    int adapter = p.row_ids != nullptr ? __ldg(p.row_ids + r) : 0;
    if (adapter < 0 || adapter >= p.num_adapters) {  // never used as an index
      atomicCAS(p.status, 0, STATUS_BAD_ADAPTER_ID);
      adapter = min(max(adapter, 0), p.num_adapters - 1);
    }
    ids_s[r] = adapter;
  }
  const int zvecs = rows * (rank_floats >> 2);
  for (int v = epi_tid; v < zvecs; v += EPI_THREADS) {
    const int r = v / (rank_floats >> 2), j = v - r * (rank_floats >> 2);
    // plain loads: z was written by the kernel just before this one
    reinterpret_cast<float4*>(zs)[v] = *reinterpret_cast<const float4*>(p.z_rows + static_cast<int64_t>(r) * SKYRL_LORA_RANK_PAD + 4 * j);
  }
  named_bar_sync(1, EPI_THREADS);

  const int nr = rows > ew ? (rows - ew + EPI_THREADS / 32 - 1) / (EPI_THREADS / 32) : 0;  // rows of this warp
  const int cpl = (cols + 31) / 32;                                                        // columns per lane
  const int items = p.lora_rank_vecs * nr * cpl;                                           // (q, row, column) per lane
  // item -> (q, row, column) without integer division (cpl <= 8, nr <= 16, items <= 1024: the float quotients of
  // (i + 0.5) are never within 0.03 of an integer, so truncation is exact)
  const float inv_cpl = 1.0f / static_cast<float>(max(cpl, 1)), inv_nr = 1.0f / static_cast<float>(max(nr, 1));
  for (int base = 0; base < items; base += ROWS_LORA_BATCH) {
    uint4 u[ROWS_LORA_BATCH];
#pragma unroll
    for (int i = 0; i < ROWS_LORA_BATCH; ++i) {
      const int item = base + i;
      u[i] = make_uint4(0u, 0u, 0u, 0u);
      if (item < items) {
        const int qr = __float2int_rz((item + 0.5f) * inv_cpl), c = item - qr * cpl;
        const int q = __float2int_rz((qr + 0.5f) * inv_nr), ri = qr - q * nr;
        const int r = ew + ri * (EPI_THREADS / 32), col = lane + 32 * c;
        if (col < cols)
          u[i] = __ldg(reinterpret_cast<const uint4*>(p.b_rows + ids_s[r] * p.b_adapter_stride +
                                                       static_cast<int64_t>(n0 + col) * p.b_row_stride) + q);
      }
    }
#pragma unroll
    for (int i = 0; i < ROWS_LORA_BATCH; ++i) {
      const int item = base + i;
      if (item < items) {
        const int qr = __float2int_rz((item + 0.5f) * inv_cpl), c = item - qr * cpl;
        const int q = __float2int_rz((qr + 0.5f) * inv_nr), ri = qr - q * nr;
        const int r = ew + ri * (EPI_THREADS / 32), col = lane + 32 * c;
        if (col < cols) {
          const float* z = zs + r * rank_floats + 8 * q;
          float* dst = lterm + r * p.lterm_pitch + col;
          float acc = q == 0 ? 0.f : *dst;
          const uint32_t w[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc = fmaf(z[2 * j], bf16_lo(w[j]), acc);
            acc = fmaf(z[2 * j + 1], bf16_hi(w[j]), acc);
          }
          *dst = acc;
        }
      }
    }
  }
}

template <int BN, int EPI, bool HAS_LORA, bool ROWS = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1) w8a8_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + MAX_STAGES;
  uint64_t* tmem_full = bars + 2 * MAX_STAGES;        // [2]
  uint64_t* tmem_empty = tmem_full + 2;               // [2]
  uint64_t* conv_done = tmem_empty + 2;               // 128 epilogue threads rewrote the accumulator
  uint64_t* lora_done = conv_done + 1;                // LoRA MMAs accumulated into TMEM
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  TileRing* ring = reinterpret_cast<TileRing*>(tmem_ptr_smem + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SCHED_SLOTS; ++s) {
      mbar_init(&ring->full[s], 1);
      mbar_init(&ring->empty[s], 1 + EPI_THREADS / 32);  // the MMA thread and one lane of every epilogue warp
    }
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], EPI_THREADS);
    }
    mbar_init(conv_done, EPI_THREADS);
    mbar_init(lora_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_ptr_smem, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&p.tm_xq);
    tma_prefetch_desc(&p.tm_w);
    if (HAS_LORA) {
      tma_prefetch_desc(&p.tm_z);
      tma_prefetch_desc(&p.tm_b);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int tm = *p.num_tiles;
  const int bn_eff = p.bn_eff;
  const int tn = (p.n + bn_eff - 1) / bn_eff;
  const int ksplits = p.k_splits;
  const int total = tm * tn * ksplits;
  const int a_bytes = p.a_rows * BK;  // the MMA still reads 128 rows; rows past a_rows hold stale finite int8
  const uint32_t stage_tx = a_bytes + bn_eff * BK;
  const int nstages = p.num_stages;
  const int stage_bytes = p.stage_bytes;

  const int kblocks = (p.k + BK - 1) / BK;
  const int band = min(p.band, max(tm, 1));

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true, have_prev = false;
      bool dep_ready = false;  // the previous kernel of the stream has finished (programmatic launch)
      int held = 0, held_stage[MAX_STAGES], held_kb[MAX_STAGES];
      int prev_row0 = 0, prev_n0 = 0, prev_adapter = 0, prev_second = 0;
      // LoRA operands of one adapter slot of one tile: pipeline slot 1 = z parts lo and mid, pipeline
      // slot 2 = z part hi and the adapter's B tile
      auto lora_slots_of = [&](int row0, int n0, int adapter, int zslot) -> bool {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
        unsigned char* sa = smem + stage * stage_bytes;
        mbar_expect_tx(&full_bar[stage], 2 * Z_PLANE_BYTES);
        tma_load_3d(sa, &p.tm_z, 0, 3 * zslot + 2, row0, &full_bar[stage]);
        tma_load_3d(sa + Z_PLANE_BYTES, &p.tm_z, 0, 3 * zslot + 1, row0, &full_bar[stage]);
        if (++stage == nstages) {
          stage = 0;
          phase ^= 1u;
        }
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
        sa = smem + stage * stage_bytes;
        mbar_expect_tx(&full_bar[stage], Z_PLANE_BYTES + bn_eff * LORA_ROW_BYTES);
        tma_load_3d(sa, &p.tm_z, 0, 3 * zslot, row0, &full_bar[stage]);
        tma_load_3d(sa + Z_PLANE_BYTES, &p.tm_b, 0, n0, adapter, &full_bar[stage]);
        if (++stage == nstages) {
          stage = 0;
          phase ^= 1u;
        }
        return true;
      };
      // a tile of two adapters (second != 0) brings both slots: z(slot 0) with the first adapter's B,
      // z(slot 1) with the second's; each row is zero in the slot that is not its own
      auto lora_slots = [&](int row0, int n0, int adapter, int second) -> bool {
        if (!lora_slots_of(row0, n0, adapter, 0)) return false;
        return second == 0 || lora_slots_of(row0, n0, (second & 0xffff) - 1, 1);
      };
      for (uint32_t it = 0; ok; ++it) {
        const int t = sched_claim(ring, it, p.sched, total, abort_flag, p.status, ok);
        if (t < 0) break;
        const TileCoord c = tile_coord(t / ksplits, tm, tn, band);
        const int4 tile = __ldg(p.tiles + c.m_idx);
        const int n0 = c.n_idx * bn_eff;
        const int kb0 = (t % ksplits) * p.kb_per_split;
        const int kb1 = min(kblocks, kb0 + p.kb_per_split);
        const int inject_at = min(LORA_INJECT_AFTER, kb1 - kb0);
        int issued = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER);
          if (!ok) break;
          unsigned char* sa = smem + stage * stage_bytes;
          mbar_expect_tx(&full_bar[stage], stage_tx);
          if (!dep_ready) {
            // The weights never depend on the kernel before this one, the activations do: until the
            // pipeline is full only the weight half of each stage is requested, then the producer waits
            // for the previous kernel and requests the activation halves.
            tma_load_3d(sa + a_bytes, &p.tm_w, 0, n0, kb, &full_bar[stage]);
            held_stage[held] = stage;
            held_kb[held] = kb;
            ++held;
            if (held == nstages || kb + 1 == kb1) {
              pdl_wait();
              pdl_trigger();
              dep_ready = true;
              for (int hq = 0; hq < held; ++hq)
                tma_load_2d(smem + held_stage[hq] * stage_bytes, &p.tm_xq, held_kb[hq] * BK, tile.x,
                            &full_bar[held_stage[hq]]);
            }
          } else {
            tma_load_2d(sa, &p.tm_xq, kb * BK, tile.x, &full_bar[stage]);
            tma_load_3d(sa + a_bytes, &p.tm_w, 0, n0, kb, &full_bar[stage]);
          }
          if (++stage == nstages) {
            stage = 0;
            phase ^= 1u;
          }
          if (HAS_LORA && have_prev && ++issued == inject_at) {
            ok = lora_slots(prev_row0, prev_n0, prev_adapter, prev_second);
            if (!ok) break;
          }
        }
        prev_row0 = tile.x;
        prev_n0 = n0;
        prev_adapter = tile.z;
        prev_second = tile.w;
        have_prev = true;
      }
      if (HAS_LORA && have_prev && ok) lora_slots(prev_row0, prev_n0, prev_adapter, prev_second);
      if (ok && p.prefetch_bytes > 0) prefetch_share_to_l2(p);
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(IDESC_D_S32, IDESC_S8, IDESC_S8, BM, bn_eff);
      const uint32_t idesc_lora = make_idesc(IDESC_D_F32, IDESC_BF16, IDESC_BF16, BM, bn_eff);
      int stage = 0;
      uint32_t phase = 0, it = 0, lora_rounds = 0;
      bool ok = true, have_prev = false;
      uint32_t prev_s = 0;
      int prev_second = 0;
      const bool prof = p.profile != 0 && blockIdx.x == 0;
      IssuerProfile pr;
      const long long prof_t0 = clock64();
      // rank-r bf16 MMAs of one adapter slot of one tile, accumulated onto the accumulator the epilogue
      // rewrote as fp32; `first` waits for that rewrite, `last` hands the accumulator back to the epilogue
      auto lora_mma_of = [&](uint32_t acc_stage, bool first, bool last) -> bool {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        const int st1 = stage;
        if (++stage == nstages) {
          stage = 0;
          phase ^= 1u;
        }
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        const int st2 = stage;
        if (++stage == nstages) {
          stage = 0;
          phase ^= 1u;
        }
        if (first && !timed_wait(prof, pr.rewrite, conv_done, lora_rounds & 1u, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        tc_fence_after_sync();
        const uint32_t e1 = smem_u32(smem + st1 * stage_bytes), e2 = smem_u32(smem + st2 * stage_bytes);
        const uint64_t bd = make_desc_sw128(e2 + Z_PLANE_BYTES);
        const uint64_t zd[3] = {make_desc_sw128(e1), make_desc_sw128(e1 + Z_PLANE_BYTES), make_desc_sw128(e2)};
        const uint32_t d = tmem_base + acc_stage * BN;
        // smallest plane first, so the low-order terms are not absorbed early
        for (int plane = 0; plane < 3; ++plane)
          for (int kk = 0; kk < p.rank_blocks; ++kk) mma_bf16(d, zd[plane] + 2 * kk, bd + 2 * kk, idesc_lora, 1u);
        mma_commit(&empty_bar[st1]);
        mma_commit(&empty_bar[st2]);
        if (last) {
          mma_commit(lora_done);
          ++lora_rounds;
        }
        return true;
      };
      auto lora_mma = [&](uint32_t acc_stage, int second) -> bool {
        if (!lora_mma_of(acc_stage, true, second == 0)) return false;
        return second == 0 || lora_mma_of(acc_stage, false, true);
      };
      for (; ok; ++it) {
        const int t = sched_read(ring, it, abort_flag, p.status, STATUS_TIMEOUT_MMA, ok);
        if (ok) sched_release(ring, it);
        if (t < 0) break;
        const uint32_t s = it & 1u, aphase = (it >> 1) & 1u;
        ok = timed_wait(prof, pr.accumulator, &tmem_empty[s], aphase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + s * BN;
        const int kb0 = (t % ksplits) * p.kb_per_split;
        const int kb1 = min(kblocks, kb0 + p.kb_per_split);
        const int inject_at = min(LORA_INJECT_AFTER, kb1 - kb0);
        const int second = HAS_LORA ? __ldg(p.tiles + tile_coord(t / ksplits, tm, tn, band).m_idx).w : 0;
        int issued = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = timed_wait(prof, pr.operands, &full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint64_t adesc = make_desc_sw128(sa);
          const uint64_t bdesc = make_desc_sw128(sa + a_bytes);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K_I8; ++j) {
            mma_i8(d, adesc + 2 * j, bdesc + 2 * j, idesc, (kb != kb0 || j != 0) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);
          if (++stage == nstages) {
            stage = 0;
            phase ^= 1u;
          }
          if (HAS_LORA && have_prev && ++issued == inject_at) {
            ok = lora_mma(prev_s, prev_second);
            if (!ok) break;
          }
        }
        if (ok) mma_commit(&tmem_full[s]);
        prev_s = s;
        prev_second = second;
        have_prev = true;
      }
      if (HAS_LORA && have_prev && ok) lora_mma(prev_s, prev_second);
      if (prof) store_profile(pr, p.status, clock64() - prof_t0);
    }
  } else {
    // ------------------------------ epilogue warps 0-3, 6-9 --------------------
    const int nchunks = (bn_eff + 31) / 32;
    const int quad = warp & 3;                        // TMEM lane quadrant this warp may access
    const int c_begin = warp < 4 ? 0 : (nchunks + 1) / 2;  // column chunks [c_begin, c_end) of the tile
    const int c_end = warp < 4 ? (nchunks + 1) / 2 : nchunks;
    const int r = quad * 32 + lane;  // row of the tile == TMEM lane
    unsigned char* store_stage =
        p.direct_stores ? nullptr : smem + SINGLE_STAGE_AREA + (warp < 4 ? warp : warp - 2) * EPI_STAGE_BYTES;
    float* lterm = reinterpret_cast<float*>(smem + p.lterm_off);
    const bool rows_lora = ROWS && p.lora_rank_vecs > 0;
    const int ew = warp < 4 ? warp : warp - 2;  // 0 ... 7 among the epilogue warps
    uint32_t it = 0, lora_it = 0;
    bool ok = true;
    if (ROWS) pdl_wait();  // scales, z and the residual may come from the kernel just before this one
    for (; ok; ++it) {
      const int t = sched_read(ring, it, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE, ok);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) sched_release(ring, it);  // every lane has read the slot (warp-wide vote above)
      if (t < 0) break;
      const TileCoord c = tile_coord(t / ksplits, tm, tn, band);
      const int4 tile = __ldg(p.tiles + c.m_idx);
      const int n0 = c.n_idx * bn_eff;
      const int n_end = min(p.n, n0 + bn_eff);  // first column this tile does not own
      const uint32_t s = it & 1u, aphase = (it >> 1) & 1u;
      const bool row_valid = r < tile.y;
      const int srow = tile.x + r;
      float sxr = 0.f;
      if (row_valid) sxr = ROWS ? *(p.sx + srow) : __ldg(p.sx + srow);
      const int64_t orow = row_valid ? (p.out_row_map != nullptr ? __ldg(p.out_row_map + srow) : srow) : 0;
      if (rows_lora) {
        // the LoRA term of this tile, computed while the tensor cores still work on it
        rows_lora_tile(p, lterm, tile.y, n0, n_end, ew, lane, ew * 32 + lane);
        named_bar_sync(1, EPI_THREADS);
      }

      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[s], aphase, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tbase = tmem_base + s * BN + (static_cast<uint32_t>(quad * 32) << 16);

      if (HAS_LORA) {
        // pass 1: int32 accumulator -> dequantised fp32, in place
#pragma unroll 1
        for (int cc = c_begin; cc < c_end; ++cc)
          epi_convert_chunk(tbase + cc * 32, n0 + cc * 32, n_end, sxr, p.sw);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(conv_done);
        __syncwarp();
        ok = __all_sync(0xffffffffu, mbar_wait(lora_done, lora_it & 1u, abort_flag, p.status, STATUS_TIMEOUT_LORA));
        if (!ok) break;
        tc_fence_after_sync();
        ++lora_it;
      }

      // pass 2: final values -> global memory
      float tile_amax = 0.f;
      float* amax_acc = (EPI == SKYRL_EPI_SWIGLU && p.row_amax != nullptr) ? &tile_amax : nullptr;
#pragma unroll 1
      for (int cc = c_begin; cc < c_end; ++cc)
        epi_store_chunk<EPI, HAS_LORA>(p, tbase + cc * 32, n0 + cc * 32, n_end, sxr, row_valid, orow,
                                       (t % ksplits) * p.slab_stride, store_stage, lane, amax_acc,
                                       (rows_lora && row_valid) ? lterm + r * p.lterm_pitch + cc * 32 : nullptr);
      // rounding to bf16 is monotonic, so the absmax of the stored values is the rounded absmax
      if (amax_acc != nullptr && row_valid && tile_amax > 0.f)
        atomicMax(reinterpret_cast<int*>(p.row_amax) + srow, __float_as_int(round_bf16(tile_amax)));
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[s]);
      if (rows_lora) named_bar_sync(1, EPI_THREADS);  // the l tile is rewritten for the next tile
    }
  }

  // ------------------------------ teardown -------------------------------------
  __syncwarp();
  if (*abort_flag) {
    // give copies still in flight time to land before shared memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0) sched_finish(p.sched);
}


// ---------------------------------------------------------------------------------------------------
// Paired-tile variant for large problems.  One CTA computes TWO 128-row M tiles against the same
// 256-column weight tile: a K stage holds both activation tiles (2 x 16 KB) and one weight tile (32 KB)
// and feeds two MMAs per K step, so the bytes a CTA must pull per unit of tensor-core work drop by a
// third (64 KB per 1024 MMA cycles instead of 48 KB per 512) and three stages cover the TMA latency
// that four 48 KB stages of the single-tile kernel do not.  The two accumulators fill TMEM
// (2 x 256 columns), so the epilogue of a pair is not overlapped with the next pair's main loop; it is
// kept short instead by sixteen epilogue warps (two tiles x four lane quadrants x two column halves).
// The two tiles of a pair are neighbours in the tile list and may belong to different adapters: each
// gets its own LoRA operands (two pipeline slots per tile, issued right after the pair's K loop).
// ---------------------------------------------------------------------------------------------------
constexpr int PAIR_THREADS = 576;      // warps 0-15 epilogue, warp 16 TMA producer, warp 17 MMA issuer
constexpr int PAIR_EPI_THREADS = 512;
constexpr int PAIR_BN = 256;
constexpr int PAIR_A_BYTES = 2 * BM * BK;
constexpr int PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_BN * BK;  // 64 KB
constexpr int PAIR_STAGES = STAGE_AREA_BYTES / PAIR_STAGE_BYTES;  // 3
constexpr int PAIR_SMEM_BYTES = STAGE_AREA_BYTES + (2 * PAIR_STAGES + 4) * 8 + 16 + 128 + 1024;

template <int EPI, bool HAS_LORA>
__global__ void __launch_bounds__(PAIR_THREADS, 1) w8a8_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGE_AREA_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + PAIR_STAGES;
  uint64_t* tmem_full = bars + 2 * PAIR_STAGES;
  uint64_t* tmem_empty = tmem_full + 1;
  uint64_t* conv_done = tmem_empty + 1;
  uint64_t* lora_done = conv_done + 1;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(lora_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  TileRing* ring = reinterpret_cast<TileRing*>(tmem_ptr_smem + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SCHED_SLOTS; ++s) {
      mbar_init(&ring->full[s], 1);
      mbar_init(&ring->empty[s], 1 + PAIR_EPI_THREADS / 32);
    }
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, PAIR_EPI_THREADS);
    mbar_init(conv_done, PAIR_EPI_THREADS);
    mbar_init(lora_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 17) {
    tmem_alloc(tmem_ptr_smem, 512);
    tmem_relinquish();
  }
  if (warp == 16 && lane == 0) {
    tma_prefetch_desc(&p.tm_xq);
    tma_prefetch_desc(&p.tm_w);
    if (HAS_LORA) {
      tma_prefetch_desc(&p.tm_z);
      tma_prefetch_desc(&p.tm_b);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int tm = *p.num_tiles;
  const int tp = (tm + 1) / 2;  // tile pairs
  const int tn = (p.n + PAIR_BN - 1) / PAIR_BN;
  const int total = tp * tn;
  const int kblocks = (p.k + BK - 1) / BK;
  const int band = min(max(p.band / 2, 1), max(tp, 1));

  if (warp == 16) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto lora_slots_of = [&](int row0, int n0, int adapter, int zslot) -> bool {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
        unsigned char* sa = smem + stage * PAIR_STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], 2 * Z_PLANE_BYTES);
        tma_load_3d(sa, &p.tm_z, 0, 3 * zslot + 2, row0, &full_bar[stage]);
        tma_load_3d(sa + Z_PLANE_BYTES, &p.tm_z, 0, 3 * zslot + 1, row0, &full_bar[stage]);
        if (++stage == PAIR_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
        sa = smem + stage * PAIR_STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], Z_PLANE_BYTES + PAIR_BN * LORA_ROW_BYTES);
        tma_load_3d(sa, &p.tm_z, 0, 3 * zslot, row0, &full_bar[stage]);
        tma_load_3d(sa + Z_PLANE_BYTES, &p.tm_b, 0, n0, adapter, &full_bar[stage]);
        if (++stage == PAIR_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        return true;
      };
      auto lora_slots = [&](const int4& tile, int n0) -> bool {  // both adapter slots of a two-adapter tile
        if (!lora_slots_of(tile.x, n0, tile.z, 0)) return false;
        return tile.w == 0 || lora_slots_of(tile.x, n0, (tile.w & 0xffff) - 1, 1);
      };
      for (uint32_t it = 0; ok; ++it) {
        const int t = sched_claim(ring, it, p.sched, total, abort_flag, p.status, ok);
        if (t < 0) break;
        const TileCoord c = tile_coord(t, tp, tn, band);
        const int4 tile_a = __ldg(p.tiles + 2 * c.m_idx);
        const bool has_b = 2 * c.m_idx + 1 < tm;
        const int4 tile_b = has_b ? __ldg(p.tiles + 2 * c.m_idx + 1) : tile_a;
        const int n0 = c.n_idx * PAIR_BN;
        const uint32_t tx = (has_b ? 2 : 1) * BM * BK + PAIR_BN * BK;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER);
          if (!ok) break;
          unsigned char* sa = smem + stage * PAIR_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], tx);
          tma_load_2d(sa, &p.tm_xq, kb * BK, tile_a.x, &full_bar[stage]);
          if (has_b) tma_load_2d(sa + BM * BK, &p.tm_xq, kb * BK, tile_b.x, &full_bar[stage]);
          tma_load_3d(sa + PAIR_A_BYTES, &p.tm_w, 0, n0, kb, &full_bar[stage]);
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (HAS_LORA && ok) {
          ok = lora_slots(tile_a, n0);
          if (ok && has_b) ok = lora_slots(tile_b, n0);
        }
      }
    }
  } else if (warp == 17) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(IDESC_D_S32, IDESC_S8, IDESC_S8, BM, PAIR_BN);
      const uint32_t idesc_lora = make_idesc(IDESC_D_F32, IDESC_BF16, IDESC_BF16, BM, PAIR_BN);
      int stage = 0;
      uint32_t phase = 0, it = 0;
      bool ok = true;
      auto lora_mma = [&](uint32_t d, bool wait_conv, uint32_t conv_parity) -> bool {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        const int st1 = stage;
        if (++stage == PAIR_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        const int st2 = stage;
        if (++stage == PAIR_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        if (wait_conv && !mbar_wait(conv_done, conv_parity, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
        tc_fence_after_sync();
        const uint32_t e1 = smem_u32(smem + st1 * PAIR_STAGE_BYTES), e2 = smem_u32(smem + st2 * PAIR_STAGE_BYTES);
        const uint64_t bd = make_desc_sw128(e2 + Z_PLANE_BYTES);
        const uint64_t zd[3] = {make_desc_sw128(e1), make_desc_sw128(e1 + Z_PLANE_BYTES), make_desc_sw128(e2)};
        for (int plane = 0; plane < 3; ++plane)
          for (int kk = 0; kk < p.rank_blocks; ++kk) mma_bf16(d, zd[plane] + 2 * kk, bd + 2 * kk, idesc_lora, 1u);
        mma_commit(&empty_bar[st1]);
        mma_commit(&empty_bar[st2]);
        return true;
      };
      for (; ok; ++it) {
        const int t = sched_read(ring, it, abort_flag, p.status, STATUS_TIMEOUT_MMA, ok);
        if (ok) sched_release(ring, it);
        if (t < 0) break;
        const TileCoord c = tile_coord(t, tp, tn, band);
        const bool has_b = 2 * c.m_idx + 1 < tm;
        ok = mbar_wait(tmem_empty, (it & 1u) ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * PAIR_STAGE_BYTES);
          const uint64_t a0 = make_desc_sw128(sa), a1 = make_desc_sw128(sa + BM * BK);
          const uint64_t bdesc = make_desc_sw128(sa + PAIR_A_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K_I8; ++j) {
            const uint32_t accumulate = (kb != 0 || j != 0) ? 1u : 0u;
            mma_i8(tmem_base, a0 + 2 * j, bdesc + 2 * j, idesc, accumulate);
            if (has_b) mma_i8(tmem_base + PAIR_BN, a1 + 2 * j, bdesc + 2 * j, idesc, accumulate);
          }
          mma_commit(&empty_bar[stage]);
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        mma_commit(tmem_full);
        if (HAS_LORA) {
          const int second_a = __ldg(p.tiles + 2 * c.m_idx).w;
          const int second_b = has_b ? __ldg(p.tiles + 2 * c.m_idx + 1).w : 0;
          ok = lora_mma(tmem_base, true, it & 1u);
          if (ok && second_a != 0) ok = lora_mma(tmem_base, false, 0u);
          if (ok && has_b) ok = lora_mma(tmem_base + PAIR_BN, false, 0u);
          if (ok && second_b != 0) ok = lora_mma(tmem_base + PAIR_BN, false, 0u);
          if (ok) mma_commit(lora_done);
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps 0-15 -----------------------
    const int which = warp >> 3;            // 0: first tile of the pair, 1: second
    const int quad = warp & 3;              // TMEM lane quadrant this warp may access
    const int c_begin = ((warp >> 2) & 1) * 4, c_end = c_begin + 4;  // column chunks of 32
    const int r = quad * 32 + lane;
    uint32_t it = 0;
    bool ok = true;
    for (; ok; ++it) {
      const int t = sched_read(ring, it, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE, ok);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) sched_release(ring, it);
      if (t < 0) break;
      const TileCoord c = tile_coord(t, tp, tn, band);
      const int tidx = 2 * c.m_idx + which;
      const bool present = tidx < tm;
      const int4 tile = present ? __ldg(p.tiles + tidx) : make_int4(0, 0, 0, 0);
      const int n0 = c.n_idx * PAIR_BN;
      const int n_end = min(p.n, n0 + PAIR_BN);
      const bool row_valid = r < tile.y;
      const int srow = tile.x + r;
      const float sxr = row_valid ? __ldg(p.sx + srow) : 0.f;
      const int64_t orow = row_valid ? (p.out_row_map != nullptr ? __ldg(p.out_row_map + srow) : srow) : 0;

      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full, it & 1u, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tbase = tmem_base + which * PAIR_BN + (static_cast<uint32_t>(quad * 32) << 16);
      if (HAS_LORA) {
        if (present) {
#pragma unroll 1
          for (int cc = c_begin; cc < c_end; ++cc)
            epi_convert_chunk(tbase + cc * 32, n0 + cc * 32, n_end, sxr, p.sw);
          tmem_wait_st();
        }
        tc_fence_before_sync();
        mbar_arrive(conv_done);
        __syncwarp();
        ok = __all_sync(0xffffffffu, mbar_wait(lora_done, it & 1u, abort_flag, p.status, STATUS_TIMEOUT_LORA));
        if (!ok) break;
        tc_fence_after_sync();
      }
      if (present) {
        float tile_amax = 0.f;
        float* amax_acc = (EPI == SKYRL_EPI_SWIGLU && p.row_amax != nullptr) ? &tile_amax : nullptr;
#pragma unroll 1
        for (int cc = c_begin; cc < c_end; ++cc)
          epi_store_chunk<EPI, HAS_LORA>(p, tbase + cc * 32, n0 + cc * 32, n_end, sxr, row_valid, orow, 0, nullptr, 0,
                                         amax_acc);
        if (amax_acc != nullptr && row_valid && tile_amax > 0.f)
          atomicMax(reinterpret_cast<int*>(p.row_amax) + srow, __float_as_int(round_bf16(tile_amax)));
      }
      tc_fence_before_sync();
      mbar_arrive(tmem_empty);
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0) sched_finish(p.sched);
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2) for large problems with a short K loop.  Two CTAs of a cluster
// compute a 256-row x 256-column output tile: each stages ITS 128-row activation tile and ITS 128 output
// channels of the weight tile (32 KB per K stage and CTA instead of 48 KB), the leader issues one 256-row MMA
// per K step that reads both CTAs' shared memory, and each CTA receives its 128 rows of the accumulator in
// its own tensor memory (256 columns, two stages: the epilogue of a pair's tile overlaps the next main loop).
// Per unit of tensor-core work a CTA pulls a third fewer bytes from L2, which is what bounds the single-tile
// kernel (bytes in flight per SM).  The two M tiles of a pair are neighbours in the tile list.
//
// LoRA: one MMA spans both tiles and has ONE B operand, while the two tiles may hold rows of up to four
// adapters.  For every distinct adapter of the pair the leader issues the rank-r MMAs once, with each CTA
// staging, at the same offset, the z planes of the slot that adapter has in ITS tile or, if it has none, a
// box that lies outside the tensor and is therefore filled with zeros; every row receives exactly its own
// adapter's term.
//
// Static schedule (pair i takes tiles i, i + pairs, ...).  Barriers: TMA loads of both CTAs report to the
// leader's full barrier; commits arrive on both CTAs' barriers; the epilogue warps of both CTAs release an
// accumulator stage (and announce the rewritten accumulator) on the leader's barriers.  All waits bounded.
// ---------------------------------------------------------------------------------------------------
constexpr int PAIR2_STAGE_BYTES = BM * BK + 128 * BK;                      // 32 KB: A tile + half of the weight tile
constexpr int PAIR2_BN = 256;
// Sixteen epilogue warps per CTA (four per tensor-memory lane quadrant, 64 columns each): with eight the
// epilogue of a 128 x 256 tile (two passes over tensor memory with LoRA, SwiGLU math, staged stores) takes
// longer than the tile's main loop and bounds the kernel; warp 16 is the TMA producer, warp 17 issues the MMAs.
constexpr int PAIR2_EPI_WARPS = 16;
constexpr int PAIR2_THREADS = (PAIR2_EPI_WARPS + 2) * 32;
constexpr int PAIR2_STAGE_AREA = STAGE_AREA_BYTES - PAIR2_EPI_WARPS * EPI_STAGE_BYTES;   // store-staging tiles on top
constexpr int PAIR2_STAGES = PAIR2_STAGE_AREA / PAIR2_STAGE_BYTES;                        // 5

struct PairAdapters {
  int count;       // distinct adapters of the pair, <= 4
  int adapter[4];
  int slot[4];     // z slot of that adapter in THIS CTA's tile (0 / 1) or -1 (none: zero planes)
};
// `first` / `second` of the two tiles of a pair (second == 0: none); `mine` selects this CTA's tile
__device__ __forceinline__ PairAdapters pair_adapters(const int4& t0, bool has1, const int4& t1, int mine) {
  PairAdapters pa;
  pa.count = 0;
  const int cand[4] = {t0.z, t0.w != 0 ? (t0.w & 0xffff) - 1 : -1, has1 ? t1.z : -1, (has1 && t1.w != 0) ? (t1.w & 0xffff) - 1 : -1};
  const int4& me = mine == 0 ? t0 : t1;
  const bool have_me = mine == 0 || has1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (cand[i] < 0) continue;
    bool seen = false;
    for (int j = 0; j < pa.count; ++j) seen = seen || pa.adapter[j] == cand[i];
    if (seen) continue;
    int slot = -1;
    if (have_me && me.z == cand[i]) slot = 0;
    else if (have_me && me.w != 0 && (me.w & 0xffff) - 1 == cand[i]) slot = 1;
    pa.adapter[pa.count] = cand[i];
    pa.slot[pa.count] = slot;
    ++pa.count;
  }
  return pa;
}

template <int EPI, bool HAS_LORA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR2_THREADS, 1)
w8a8_gemm_pair2_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<PAIR2_BN>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* full_bar = bars;                          // the leader's are used
  uint64_t* empty_bar = bars + MAX_STAGES;            // each CTA's own, released by the leader's commits
  uint64_t* tmem_full = bars + 2 * MAX_STAGES;        // [2], each CTA's own
  uint64_t* tmem_empty = tmem_full + 2;               // [2], the leader's: one arrival per epilogue warp of both CTAs
  uint64_t* conv_done = tmem_empty + 2;               // the leader's: accumulators of both CTAs rewritten
  uint64_t* lora_done = conv_done + 1;                // each CTA's own
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 2 * PAIR2_EPI_WARPS);
    }
    mbar_init(conv_done, 2 * PAIR2_EPI_WARPS);
    mbar_init(lora_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == PAIR2_EPI_WARPS + 1) {
    tmem_alloc_pair(tmem_ptr_smem, 512);
    tmem_relinquish_pair();
  }
  if (warp == PAIR2_EPI_WARPS && lane == 0) {
    tma_prefetch_desc(&p.tm_xq);
    tma_prefetch_desc(&p.tm_w);
    if (HAS_LORA) {
      tma_prefetch_desc(&p.tm_z);
      tma_prefetch_desc(&p.tm_b);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything of this CTA signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int tm = *p.num_tiles;
  const int tpairs = (tm + 1) / 2;
  const int tn = (p.n + PAIR2_BN - 1) / PAIR2_BN;
  const int total = tpairs * tn;
  const int kblocks = (p.k + BK - 1) / BK;
  const int band = min(max(p.band / 2, 1), max(tpairs, 1));
  const int pair_id = static_cast<int>(blockIdx.x >> 1), num_pairs = static_cast<int>(gridDim.x >> 1);
  const int oob_row = p.m;   // a box that starts here lies outside the tensor: filled with zeros

  if (warp == PAIR2_EPI_WARPS) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true, have_prev = false;
      int4 prev0 = make_int4(0, 0, 0, 0), prev1 = prev0;
      bool prev_has1 = false;
      int prev_n0 = 0;
      auto next_stage = [&]() {
        if (++stage == PAIR2_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      };
      // LoRA operands of the pair's previous tile: per distinct adapter two pipeline slots
      // (slot A: z parts lo and mid; slot B: z part hi and this CTA's half of the adapter's B tile)
      auto lora_slots = [&]() -> bool {
        const PairAdapters pa = pair_adapters(prev0, prev_has1, prev1, static_cast<int>(rank));
        const int4& me = rank == 0 ? prev0 : prev1;
        for (int g = 0; g < pa.count; ++g) {
          const int zrow = pa.slot[g] >= 0 ? me.x : oob_row;
          const int zs = pa.slot[g] >= 0 ? pa.slot[g] : 0;
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
          unsigned char* sa = smem + stage * PAIR2_STAGE_BYTES;
          uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * 2 * Z_PLANE_BYTES);
          tma_load_3d_pair(sa, &p.tm_z, 0, 3 * zs + 2, zrow, fb);
          tma_load_3d_pair(sa + Z_PLANE_BYTES, &p.tm_z, 0, 3 * zs + 1, zrow, fb);
          next_stage();
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) return false;
          sa = smem + stage * PAIR2_STAGE_BYTES;
          fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * (Z_PLANE_BYTES + 128 * LORA_ROW_BYTES));
          tma_load_3d_pair(sa, &p.tm_z, 0, 3 * zs, zrow, fb);
          tma_load_3d_pair(sa + Z_PLANE_BYTES, &p.tm_b, 0, prev_n0 + static_cast<int>(rank) * 128, pa.adapter[g], fb);
          next_stage();
        }
        return true;
      };
      for (int t = pair_id; t < total && ok; t += num_pairs) {
        const TileCoord c = tile_coord(t, tpairs, tn, band);
        const int4 t0 = __ldg(p.tiles + 2 * c.m_idx);
        const bool has1 = 2 * c.m_idx + 1 < tm;
        const int4 t1 = has1 ? __ldg(p.tiles + 2 * c.m_idx + 1) : make_int4(oob_row, 0, 0, 0);
        const int row0 = rank == 0 ? t0.x : (has1 ? t1.x : oob_row);
        const int n0 = c.n_idx * PAIR2_BN;
        const int inject_at = min(LORA_INJECT_AFTER, kblocks);
        int issued = 0;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER);
          if (!ok) break;
          unsigned char* sa = smem + stage * PAIR2_STAGE_BYTES;
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * PAIR2_STAGE_BYTES);
          tma_load_2d_pair(sa, &p.tm_xq, kb * BK, row0, fb);
          tma_load_3d_pair(sa + BM * BK, &p.tm_w, 0, n0 + static_cast<int>(rank) * 128, kb, fb);
          next_stage();
          if (HAS_LORA && have_prev && ++issued == inject_at) {
            ok = lora_slots();
            if (!ok) break;
          }
        }
        prev0 = t0;
        prev1 = t1;
        prev_has1 = has1;
        prev_n0 = n0;
        have_prev = true;
      }
      if (HAS_LORA && have_prev && ok) lora_slots();
    }
  } else if (warp == PAIR2_EPI_WARPS + 1) {
    // ------------------------------ MMA issuer (the leader only) ---------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc(IDESC_D_S32, IDESC_S8, IDESC_S8, 2 * BM, PAIR2_BN);
      const uint32_t idesc_lora = make_idesc(IDESC_D_F32, IDESC_BF16, IDESC_BF16, 2 * BM, PAIR2_BN);
      int stage = 0;
      uint32_t phase = 0, it = 0, lora_rounds = 0;
      bool ok = true, have_prev = false;
      uint32_t prev_s = 0;
      int prev_groups = 0;
      const bool prof = p.profile != 0 && blockIdx.x == 0;
      IssuerProfile pr;
      const long long prof_t0 = clock64();
      auto next_stage = [&]() {
        if (++stage == PAIR2_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      };
      auto lora_mma = [&](uint32_t acc_stage, int groups) -> bool {
        for (int g = 0; g < groups; ++g) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
          const int st1 = stage;
          next_stage();
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
          const int st2 = stage;
          next_stage();
          if (g == 0 && !timed_wait(prof, pr.rewrite, conv_done, lora_rounds & 1u, abort_flag, p.status, STATUS_TIMEOUT_LORA)) return false;
          tc_fence_after_sync();
          const uint32_t e1 = smem_u32(smem + st1 * PAIR2_STAGE_BYTES), e2 = smem_u32(smem + st2 * PAIR2_STAGE_BYTES);
          const uint64_t bd = make_desc_sw128(e2 + Z_PLANE_BYTES);
          const uint64_t zd[3] = {make_desc_sw128(e1), make_desc_sw128(e1 + Z_PLANE_BYTES), make_desc_sw128(e2)};
          const uint32_t d = tmem_base + acc_stage * PAIR2_BN;
          for (int plane = 0; plane < 3; ++plane)   // smallest plane first
            for (int kk = 0; kk < p.rank_blocks; ++kk) mma_bf16_pair(d, zd[plane] + 2 * kk, bd + 2 * kk, idesc_lora, 1u);
          mma_commit_pair(&empty_bar[st1]);
          mma_commit_pair(&empty_bar[st2]);
        }
        mma_commit_pair(lora_done);
        ++lora_rounds;
        return true;
      };
      for (int t = pair_id; t < total && ok; t += num_pairs, ++it) {
        const uint32_t s = it & 1u, aphase = (it >> 1) & 1u;
        ok = timed_wait(prof, pr.accumulator, &tmem_empty[s], aphase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + s * PAIR2_BN;
        int groups = 0;
        if (HAS_LORA) {
          const TileCoord c = tile_coord(t, tpairs, tn, band);
          const int4 t0 = __ldg(p.tiles + 2 * c.m_idx);
          const bool has1 = 2 * c.m_idx + 1 < tm;
          const int4 t1 = has1 ? __ldg(p.tiles + 2 * c.m_idx + 1) : make_int4(0, 0, 0, 0);
          groups = pair_adapters(t0, has1, t1, 0).count;
        }
        const int inject_at = min(LORA_INJECT_AFTER, kblocks);
        int issued = 0;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = timed_wait(prof, pr.operands, &full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * PAIR2_STAGE_BYTES);
          const uint64_t adesc = make_desc_sw128(sa);
          const uint64_t bdesc = make_desc_sw128(sa + BM * BK);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K_I8; ++j)
            mma_i8_pair(d, adesc + 2 * j, bdesc + 2 * j, idesc, (kb != 0 || j != 0) ? 1u : 0u);
          mma_commit_pair(&empty_bar[stage]);
          next_stage();
          if (HAS_LORA && have_prev && ++issued == inject_at) {
            ok = lora_mma(prev_s, prev_groups);
            if (!ok) break;
          }
        }
        if (ok) mma_commit_pair(&tmem_full[s]);
        prev_s = s;
        prev_groups = groups;
        have_prev = true;
      }
      if (HAS_LORA && have_prev && ok) lora_mma(prev_s, prev_groups);
      if (prof) store_profile(pr, p.status, clock64() - prof_t0);
    }
  } else {
    // ------------------------------ epilogue warps 0-15 (both CTAs, own tile) ---------------
    const int quad = warp & 3;                                          // tensor-memory lane quadrant of this warp
    const int c_begin = (warp >> 2) * 2, c_end = c_begin + 2;           // two 32-column chunks of the 256 columns
    const int r = quad * 32 + lane;
    unsigned char* store_stage = smem + PAIR2_STAGE_AREA + warp * EPI_STAGE_BYTES;
    const uint32_t conv_remote = map_to_cta(smem_u32(conv_done), 0);
    uint32_t it = 0, lora_it = 0;
    bool ok = true;
    for (int t = pair_id; t < total && ok; t += num_pairs, ++it) {
      const TileCoord c = tile_coord(t, tpairs, tn, band);
      const int tidx = 2 * c.m_idx + static_cast<int>(rank);
      const bool present = tidx < tm;
      const int4 tile = present ? __ldg(p.tiles + tidx) : make_int4(0, 0, 0, 0);
      const int n0 = c.n_idx * PAIR2_BN;
      const int n_end = min(p.n, n0 + PAIR2_BN);
      const uint32_t s = it & 1u, aphase = (it >> 1) & 1u;
      const bool row_valid = r < tile.y;
      const int srow = tile.x + r;
      const float sxr = row_valid ? __ldg(p.sx + srow) : 0.f;
      const int64_t orow = row_valid ? (p.out_row_map != nullptr ? __ldg(p.out_row_map + srow) : srow) : 0;

      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[s], aphase, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tbase = tmem_base + s * PAIR2_BN + (static_cast<uint32_t>(quad * 32) << 16);
      if (HAS_LORA) {
#pragma unroll 1
        for (int cc = c_begin; cc < c_end; ++cc)
          epi_convert_chunk(tbase + cc * 32, n0 + cc * 32, n_end, sxr, p.sw);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(conv_remote);
        ok = __all_sync(0xffffffffu, mbar_wait(lora_done, lora_it & 1u, abort_flag, p.status, STATUS_TIMEOUT_LORA));
        if (!ok) break;
        tc_fence_after_sync();
        ++lora_it;
      }
      float tile_amax = 0.f;
      float* amax_acc = (EPI == SKYRL_EPI_SWIGLU && p.row_amax != nullptr) ? &tile_amax : nullptr;
#pragma unroll 1
      for (int cc = c_begin; cc < c_end; ++cc)
        epi_store_chunk<EPI, HAS_LORA>(p, tbase + cc * 32, n0 + cc * 32, n_end, sxr, row_valid, orow, 0, store_stage, lane,
                                       amax_acc);
      if (amax_acc != nullptr && row_valid && tile_amax > 0.f)
        atomicMax(reinterpret_cast<int*>(p.row_amax) + srow, __float_as_int(round_bf16(tile_amax)));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[s]), 0));
    }
  }

  // ------------------------------ teardown -------------------------------------
  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers or read its shared memory
  if (warp == PAIR2_EPI_WARPS + 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int EPI, bool HAS_LORA>
static int launch_pair2_variant(const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<PAIR2_BN>;
  auto kernel = w8a8_gemm_pair2_kernel<EPI, HAS_LORA>;
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(kernel, Cfg::SMEM_BYTES, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm attribute: %s", cudaGetErrorString(e));
  kernel<<<grid, PAIR2_THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

static int launch_pair2(const GemmParams& p, int epi, bool lora, int grid, cudaStream_t stream) {
  switch (epi) {
    case SKYRL_EPI_LINEAR:
      return lora ? launch_pair2_variant<SKYRL_EPI_LINEAR, true>(p, grid, stream)
                  : launch_pair2_variant<SKYRL_EPI_LINEAR, false>(p, grid, stream);
    case SKYRL_EPI_SWIGLU:
      return lora ? launch_pair2_variant<SKYRL_EPI_SWIGLU, true>(p, grid, stream)
                  : launch_pair2_variant<SKYRL_EPI_SWIGLU, false>(p, grid, stream);
    case SKYRL_EPI_RESIDUAL:
      return lora ? launch_pair2_variant<SKYRL_EPI_RESIDUAL, true>(p, grid, stream)
                  : launch_pair2_variant<SKYRL_EPI_RESIDUAL, false>(p, grid, stream);
    case SKYRL_EPI_PARTIAL_F32:
      return lora ? launch_pair2_variant<SKYRL_EPI_PARTIAL_F32, true>(p, grid, stream)
                  : launch_pair2_variant<SKYRL_EPI_PARTIAL_F32, false>(p, grid, stream);
    case SKYRL_EPI_ACC_I32:
      return launch_pair2_variant<SKYRL_EPI_ACC_I32, false>(p, grid, stream);
    default:
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: unknown epilogue %d", epi);
  }
}

template <int EPI, bool HAS_LORA>
static int launch_pair_variant(const GemmParams& p, int grid, cudaStream_t stream) {
  auto kernel = w8a8_gemm_pair_kernel<EPI, HAS_LORA>;
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(kernel, PAIR_SMEM_BYTES, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm attribute: %s", cudaGetErrorString(e));
  kernel<<<grid, PAIR_THREADS, PAIR_SMEM_BYTES, stream>>>(p);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

static int launch_pair(const GemmParams& p, int epi, bool lora, int grid, cudaStream_t stream) {
  switch (epi) {
    case SKYRL_EPI_LINEAR:
      return lora ? launch_pair_variant<SKYRL_EPI_LINEAR, true>(p, grid, stream)
                  : launch_pair_variant<SKYRL_EPI_LINEAR, false>(p, grid, stream);
    case SKYRL_EPI_SWIGLU:
      return lora ? launch_pair_variant<SKYRL_EPI_SWIGLU, true>(p, grid, stream)
                  : launch_pair_variant<SKYRL_EPI_SWIGLU, false>(p, grid, stream);
    case SKYRL_EPI_RESIDUAL:
      return lora ? launch_pair_variant<SKYRL_EPI_RESIDUAL, true>(p, grid, stream)
                  : launch_pair_variant<SKYRL_EPI_RESIDUAL, false>(p, grid, stream);
    case SKYRL_EPI_PARTIAL_F32:
      return lora ? launch_pair_variant<SKYRL_EPI_PARTIAL_F32, true>(p, grid, stream)
                  : launch_pair_variant<SKYRL_EPI_PARTIAL_F32, false>(p, grid, stream);
    case SKYRL_EPI_ACC_I32:
      return launch_pair_variant<SKYRL_EPI_ACC_I32, false>(p, grid, stream);
    default:
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: unknown epilogue %d", epi);
  }
}

template <int BN, int EPI, bool HAS_LORA, bool ROWS = false>
static int launch_variant(const GemmParams& p, int grid, cudaStream_t stream, bool programmatic) {
  using Cfg = GemmCfg<BN>;
  auto kernel = w8a8_gemm_kernel<BN, EPI, HAS_LORA, ROWS>;
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(kernel, Cfg::SMEM_BYTES, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm attribute: %s", cudaGetErrorString(e));
  e = launch_kernel(kernel, dim3(grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, programmatic, p);
  if (e == cudaSuccess) e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "gemm launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

template <int BN>
static int launch_bn(const GemmParams& p, int epi, bool lora, int grid, cudaStream_t stream, bool programmatic) {
  switch (epi) {
    case SKYRL_EPI_LINEAR:
      return lora ? launch_variant<BN, SKYRL_EPI_LINEAR, true>(p, grid, stream, programmatic)
                  : launch_variant<BN, SKYRL_EPI_LINEAR, false>(p, grid, stream, programmatic);
    case SKYRL_EPI_SWIGLU:
      return lora ? launch_variant<BN, SKYRL_EPI_SWIGLU, true>(p, grid, stream, programmatic)
                  : launch_variant<BN, SKYRL_EPI_SWIGLU, false>(p, grid, stream, programmatic);
    case SKYRL_EPI_RESIDUAL:
      return lora ? launch_variant<BN, SKYRL_EPI_RESIDUAL, true>(p, grid, stream, programmatic)
                  : launch_variant<BN, SKYRL_EPI_RESIDUAL, false>(p, grid, stream, programmatic);
    case SKYRL_EPI_PARTIAL_F32:
      return lora ? launch_variant<BN, SKYRL_EPI_PARTIAL_F32, true>(p, grid, stream, programmatic)
                  : launch_variant<BN, SKYRL_EPI_PARTIAL_F32, false>(p, grid, stream, programmatic);
    case SKYRL_EPI_ACC_I32:
      return launch_variant<BN, SKYRL_EPI_ACC_I32, false>(p, grid, stream, programmatic);
    default:
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: unknown epilogue %d", epi);
  }
}

// small-batch variants: token order, per-row LoRA term on the CUDA cores (see GemmParams::z_rows)
template <int BN>
static int launch_rows_bn(const GemmParams& p, int epi, int grid, cudaStream_t stream, bool programmatic) {
  switch (epi) {
    case SKYRL_EPI_LINEAR: return launch_variant<BN, SKYRL_EPI_LINEAR, false, true>(p, grid, stream, programmatic);
    case SKYRL_EPI_SWIGLU: return launch_variant<BN, SKYRL_EPI_SWIGLU, false, true>(p, grid, stream, programmatic);
    case SKYRL_EPI_RESIDUAL: return launch_variant<BN, SKYRL_EPI_RESIDUAL, false, true>(p, grid, stream, programmatic);
    case SKYRL_EPI_PARTIAL_F32: return launch_variant<BN, SKYRL_EPI_PARTIAL_F32, false, true>(p, grid, stream, programmatic);
    default: return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: the small-batch LoRA epilogue does not combine with epilogue %d", epi);
  }
}

static inline int kblocks_of(int k) { return (k + BK - 1) / BK; }

// Claim counters of the dynamic tile scheduler: one {claimed, finished} pair per launch, handed out round
// robin.  A launch leaves its pair at zero (sched_finish), so a pair is ready again long before the ring
// of SCHED_COUNTER_SLOTS launches comes back to it.
constexpr int SCHED_COUNTER_SLOTS = 1024;
static __device__ int g_sched_counters[SCHED_COUNTER_SLOTS][2];

static int* next_sched_counter() {
  static std::mutex mu;
  static int* base[64] = {nullptr};
  static unsigned seq = 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sched_counters) != cudaSuccess) return nullptr;
    base[dev] = static_cast<int*>(ptr);
  }
  return base[dev] + 2 * (seq++ % SCHED_COUNTER_SLOTS);
}

GemmPlan plan_gemm(int m, int n, int k, int epilogue, int max_slabs) {
  GemmPlan pl;
  int sms = sm_count();
  if (sms <= 0) sms = 148;  // planning without a device (workspace queries): the B200 count
  const int mt_est = (m + BM - 1) / BM;
  const int kblocks = (k + BK - 1) / BK;
  const int64_t tiles256 = static_cast<int64_t>(mt_est) * ((n + 255) / 256);
  pl.bn_eff = 256;
  pl.k_splits = 1;
  pl.kb_per_split = kblocks;
  // 256-wide N tiles when they fill the GPU; otherwise one wave of narrower tiles sized so that every SM
  // streams an equal share of the weight (the decode shapes are HBM-bound) ...
  if (tiles256 < sms) {
    const int per_mtile = sms / mt_est > 0 ? sms / mt_est : 1;
    int bn = ((n + per_mtile - 1) / per_mtile + 15) / 16 * 16;
    if (bn < 16) bn = 16;
    if (bn > 256) bn = 256;
    pl.bn_eff = bn;
    if (bn < 96 && epilogue == SKYRL_EPI_ACC_I32 && max_slabs > 1) {
      // ... unless that makes the tiles so narrow that every CTA re-reads the same activation codes for
      // little weight data: then keep wide tiles and split K over slabs of the int32 output instead.
      pl.bn_eff = n >= 256 ? 256 : (n + 15) / 16 * 16;
      const int tn = (n + pl.bn_eff - 1) / pl.bn_eff;
      int want = sms / (mt_est * tn);
      if (want > max_slabs) want = max_slabs;
      if (want < 1) want = 1;
      if (want > kblocks) want = kblocks;
      pl.kb_per_split = (kblocks + want - 1) / want;
      pl.k_splits = (kblocks + pl.kb_per_split - 1) / pl.kb_per_split;
    }
  }
  return pl;
}

int launch_gemm(const SkyrlW8A8GemmArgs& a, cudaStream_t stream, bool programmatic) {
  if (a.struct_size != sizeof(SkyrlW8A8GemmArgs))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: struct_size %u does not match ABI v%d (%zu)", a.struct_size,
                SKYRL_W8A8_ABI_VERSION, sizeof(SkyrlW8A8GemmArgs));
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: non-positive shape");
  if (a.k % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: K must be a multiple of 16, got %d", a.k);
  if (a.n % 16 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: N must be a multiple of 16, got %d", a.n);
  if (a.xq == nullptr || a.sx == nullptr || a.wq == nullptr || a.sw == nullptr || a.out == nullptr ||
      a.tiles == nullptr || a.num_tiles == nullptr || a.status == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: null buffer");
  if (!aligned16(a.xq) || !aligned16(a.wq) || !aligned16(a.sw) || !aligned16(a.out) || !aligned16(a.tiles))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: buffers must be 16-byte aligned");
  if (a.rank < 0 || a.rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "gemm: LoRA rank must be in [0, %d], got %d", SKYRL_LORA_RANK_PAD, a.rank);
  const bool rows = a.z_rows != nullptr;  // small-batch LoRA: token order, per-row adapter, CUDA-core LoRA term
  if (rows) {
    if (a.m > SKYRL_TILE_ROWS)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: the small-batch LoRA epilogue takes at most %d rows, got %d", SKYRL_TILE_ROWS, a.m);
    if (a.rank <= 0 || a.lora_b_rows == nullptr || !aligned16(a.lora_b_rows) || !aligned16(a.z_rows) ||
        a.lora_b_rows_rank < a.rank || a.lora_b_rows_rank % 8 != 0 || a.num_adapters <= 0)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: small-batch LoRA operands missing, misaligned or of the wrong rank");
    if (a.out_row_map != nullptr || a.split_k_slabs > 1 || a.scatter_rows > 0 || a.row_amax != nullptr)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: the small-batch LoRA epilogue keeps token order and does not split K");
  }
  const bool lora = a.rank > 0 && !rows;
  if (lora && (a.z_parts == nullptr || !aligned16(a.z_parts) || a.lora_b_packed == nullptr || a.num_adapters <= 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: LoRA buffers missing");
  if (lora && a.epilogue == SKYRL_EPI_ACC_I32)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: the int32 accumulator output excludes the LoRA term");
  if (a.epilogue == SKYRL_EPI_RESIDUAL && (a.residual == nullptr || !aligned16(a.residual) ||
                                           a.residual_row_stride < a.n || a.residual_row_stride % 8 != 0))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: residual missing, misaligned or with a bad stride");
  const int64_t out_cols = a.epilogue == SKYRL_EPI_SWIGLU ? a.n / 2 : a.n;
  if (a.epilogue == SKYRL_EPI_SWIGLU && a.n % 32 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: SwiGLU needs N (2*I) to be a multiple of 32, got %d", a.n);
  if (a.out_row_stride < out_cols || a.out_row_stride % 8 != 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: output stride must be >= the row length and a multiple of 8");
  if (a.out == a.xq || a.out == a.wq || a.out == a.z_parts)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: output aliases an input");
  if (a.max_tiles <= 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: max_tiles must be positive");

  const int sms = sm_count();
  if (sms <= 0) return fail(SKYRL_ERR_LAUNCH, "gemm: no CUDA device");
  const GemmPlan pl = plan_gemm(a.m, a.n, a.k, a.epilogue, a.split_k_slabs);
  const int mt_est = (a.m + BM - 1) / BM;
  int bn_eff = pl.bn_eff;
  if (rows && a.m > 64 && bn_eff > 128) bn_eff = 128;  // the l tile (rows x columns fp32) must leave room for the pipeline
  const int k_splits = pl.k_splits, kb_per_split = pl.kb_per_split;
  const int bn = bn_eff > 128 ? 256 : 128;
  // Kernel variant for large problems (all give the same bits).
  //   long K loop (>= 64 blocks of 128): a CTA pair per 256 x 256 tile (tcgen05 cta_group::2): each CTA stages its
  //     128 rows and half of the weight tile, a third fewer bytes per unit of tensor-core work, two accumulator
  //     stages, sixteen epilogue warps.  Measured on B200: down projection of the Qwen3-32B-shaped block (K = 25600)
  //     1.57 ms against 1.61 ms for the two-tiles-per-CTA kernel, the Qwen3-8B-shaped one (K = 12288) 0.555 against
  //     0.607 ms.  With a CTA cap (a concurrent stream wants SMs) the two-tile kernel, whose tile claims are dynamic.
  //   shorter K loop: one 128 x 256 tile per CTA.  There the MMA-issuing thread is blocked on the tensor pipe ~89 %
  //     of the time whatever the variant (SKYRL_GEMM_VARIANT_PROFILE), the CTA pair brings nothing (K = 5120:
  //     3.61 ms against 3.50 ms), and the single tile keeps dynamic tile claims.
  // Neither pair form with a row scatter (their epilogues' tile order is static / their stores are 16 bytes per
  // row from registers, which NVLink carries poorly).
  const bool big = !rows && bn_eff == 256 && k_splits == 1 && a.scatter_rows == 0 &&
                   static_cast<int64_t>(mt_est) * ((a.n + 255) / 256) >= 4 * sms;
  bool pair2 = big && kblocks_of(a.k) >= 64 && a.cta_limit <= 0;
  bool paired = big && kblocks_of(a.k) >= 64 && !pair2;
  const int forced = a.variant & 3;
  if (forced == SKYRL_GEMM_VARIANT_SINGLE) paired = pair2 = false;
  if (forced == SKYRL_GEMM_VARIANT_TWO_TILES) paired = big, pair2 = false;
  if (forced == SKYRL_GEMM_VARIANT_CTA_PAIR) pair2 = big && a.cta_limit <= 0, paired = paired && !pair2;
  const int w_box_rows = pair2 ? 128 : bn_eff;   // a CTA of a pair stages half of the weight (and LoRA-B) tile

  GemmParams p;
  int rc;
  if ((rc = encode_tmap_2d(&p.tm_xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, a.k, a.m, a.k, BK,
                           (!lora && a.m <= 64) ? 64 : BM)))
    return rc;
  if ((rc = encode_tmap_3d(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.wq, BK, a.n, (a.k + BK - 1) / BK, BK,
                           static_cast<uint64_t>(a.n) * BK, BK, w_box_rows)))
    return rc;
  if (lora) {
    if ((rc = encode_tmap_3d(&p.tm_z, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.z_parts, SKYRL_LORA_RANK_PAD, SKYRL_Z_PARTS,
                             a.m, LORA_ROW_BYTES, SKYRL_Z_PARTS * LORA_ROW_BYTES, SKYRL_LORA_RANK_PAD, 1, BM)))
      return rc;
    if ((rc = encode_tmap_3d(&p.tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.lora_b_packed, SKYRL_LORA_RANK_PAD, a.n,
                             a.num_adapters, LORA_ROW_BYTES, static_cast<uint64_t>(a.n) * LORA_ROW_BYTES,
                             SKYRL_LORA_RANK_PAD, w_box_rows)))
      return rc;
  } else {
    p.tm_z = p.tm_xq;
    p.tm_b = p.tm_xq;
  }
  p.sx = a.sx;
  p.sw = a.sw;
  p.tiles = reinterpret_cast<const int4*>(a.tiles);
  p.num_tiles = a.num_tiles;
  p.out_row_map = a.out_row_map;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual);
  p.out = a.out;
  p.out_stride = a.out_row_stride;
  p.res_stride = a.residual_row_stride;
  p.status = a.status;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.rank_blocks = (a.rank + 15) / 16;
#ifndef SKYRL_RASTER_BAND
#define SKYRL_RASTER_BAND 32  // M tiles per raster band; c5 step on one B200: 51.1 / 49.4 / 48.7 / 49.9 ms for 8 / 16 / 32 / 64
#endif
  p.band = SKYRL_RASTER_BAND;
  p.bn_eff = bn_eff;
  // The whole stage area is pipeline depth: the main loop is bound by bytes in flight per SM.
  p.a_rows = (!lora && a.m <= 64) ? 64 : BM;
  p.stage_bytes = p.a_rows * BK + (bn_eff * BK + 1023) / 1024 * 1024;
  if (lora && p.stage_bytes < 2 * Z_PLANE_BYTES) p.stage_bytes = 2 * Z_PLANE_BYTES;  // a slot also carries two z planes
  p.num_stages = SINGLE_STAGE_AREA / p.stage_bytes;
  p.z_rows = nullptr;
  p.row_ids = nullptr;
  p.b_rows = nullptr;
  p.b_adapter_stride = 0;
  p.b_row_stride = 0;
  p.lora_rank_vecs = 0;
  p.num_adapters = a.num_adapters;
  p.lterm_off = 0;
  p.lterm_pitch = 0;
  p.profile = (a.variant & SKYRL_GEMM_VARIANT_PROFILE) != 0;
  if (rows) {
    p.z_rows = a.z_rows;
    p.row_ids = a.row_adapter_ids;
    p.b_rows = static_cast<const __nv_bfloat16*>(a.lora_b_rows);
    p.b_row_stride = a.lora_b_rows_rank;
    p.b_adapter_stride = static_cast<int64_t>(a.n) * a.lora_b_rows_rank;
    p.lora_rank_vecs = (a.rank + 7) / 8;
    p.lterm_pitch = (bn_eff + 31) / 32 * 32 + 1;
    // l tile [rows][pitch] fp32 + staged z [rows][rank] fp32 + adapter ids [rows]
    const int lrows = a.m <= 64 ? 64 : BM;
    const int lterm_bytes = (lrows * (p.lterm_pitch + p.lora_rank_vecs * 8 + 1) * 4 + 1023) / 1024 * 1024;
    p.num_stages = (SINGLE_STAGE_AREA - lterm_bytes) / p.stage_bytes;
    if (p.num_stages < 2) return fail(SKYRL_ERR_UNSUPPORTED, "gemm: no room for the small-batch LoRA tile");
    if (p.num_stages > MAX_STAGES) p.num_stages = MAX_STAGES;
    p.lterm_off = p.num_stages * p.stage_bytes;
  }
  p.scatter_rows = 0;
  p.scatter_row0 = 0;
  for (int o = 0; o < 8; ++o) p.scatter_base[o] = nullptr;
  if (a.scatter_rows > 0) {
    if (a.epilogue != SKYRL_EPI_PARTIAL_F32 || a.scatter_row0 < 0)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: a row scatter needs SKYRL_EPI_PARTIAL_F32 and scatter_row0 >= 0");
    // owners are the leading non-null bases; a row whose owner has none is skipped and flagged in `status`
    if (a.scatter_bases[0] == nullptr) return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: scatter base 0 is null");
    for (int o = 0; o < 8; ++o) {
      if (!aligned16(a.scatter_bases[o]))
        return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: scatter base %d is not 16-byte aligned", o);
      p.scatter_base[o] = static_cast<float*>(a.scatter_bases[o]);
    }
    p.scatter_rows = a.scatter_rows;
    p.scatter_row0 = a.scatter_row0;
  }
  p.row_amax = nullptr;
  if (a.row_amax != nullptr) {
    if (a.epilogue != SKYRL_EPI_SWIGLU || a.out_row_map != nullptr)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: row_amax needs the SwiGLU epilogue and rows left in sorted order");
    p.row_amax = a.row_amax;
  }
  p.direct_stores = 0;
  if (p.num_stages > MAX_STAGES) p.num_stages = MAX_STAGES;
  p.sched = a.sched != nullptr ? a.sched : next_sched_counter();
  if (p.sched == nullptr) return fail(SKYRL_ERR_LAUNCH, "gemm: scheduler counters unavailable");
  p.prefetch = nullptr;
  p.prefetch_bytes = 0;
  if (a.prefetch != nullptr && a.prefetch_bytes > 0) {
    if (!aligned16(a.prefetch) || a.prefetch_bytes % 16 != 0)
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: the prefetch range must be 16-byte aligned in address and size");
    p.prefetch = static_cast<const unsigned char*>(a.prefetch);
    p.prefetch_bytes = a.prefetch_bytes;
  }
  p.k_splits = k_splits;
  p.kb_per_split = kb_per_split;
  p.slab_stride = static_cast<int64_t>(a.m) * a.out_row_stride;
  const int64_t max_total = static_cast<int64_t>(a.max_tiles) * ((a.n + bn_eff - 1) / bn_eff) * k_splits;
  int grid = static_cast<int>(max_total < sms ? max_total : sms);
  if (a.cta_limit > 0 && grid > a.cta_limit) grid = a.cta_limit;  // leave SMs to a concurrent collective
  if (pair2) {
    const int64_t pair_total = static_cast<int64_t>((a.max_tiles + 1) / 2) * ((a.n + 255) / 256);
    const int pairs = static_cast<int>(pair_total < sms / 2 ? pair_total : sms / 2);
    return launch_pair2(p, a.epilogue, lora, 2 * pairs, stream);
  }
  if (paired) {
    const int64_t pair_total = static_cast<int64_t>((a.max_tiles + 1) / 2) * ((a.n + 255) / 256);
    int pgrid = static_cast<int>(pair_total < sms ? pair_total : sms);
    if (a.cta_limit > 0 && pgrid > a.cta_limit) pgrid = a.cta_limit;
    return launch_pair(p, a.epilogue, lora, pgrid, stream);
  }
  if (rows)
    return bn == 256 ? launch_rows_bn<256>(p, a.epilogue, grid, stream, programmatic)
                     : launch_rows_bn<128>(p, a.epilogue, grid, stream, programmatic);
  return bn == 256 ? launch_bn<256>(p, a.epilogue, lora, grid, stream, programmatic)
                   : launch_bn<128>(p, a.epilogue, lora, grid, stream, programmatic);
}

}  // namespace skyrl

extern "C" int skyrl_w8a8_gemm_sm100_v1(const SkyrlW8A8GemmArgs* args, skyrl_stream_t stream) {
  if (args == nullptr) return skyrl::fail(SKYRL_ERR_INVALID_ARGUMENT, "gemm: args is null");
  return skyrl::launch_gemm(*args, static_cast<cudaStream_t>(stream), false);
}

extern "C" int skyrl_w8a8_gemm_k_splits(int32_t m, int32_t n, int32_t k, int32_t split_k_slabs) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  return skyrl::plan_gemm(m, n, k, SKYRL_EPI_ACC_I32, split_k_slabs).k_splits;
}
