// LoRA-A projection on the tensor cores: for every 128-row tile of the
// adapter-sorted row space, z = s[a] * (x_tile @ A[a]) with a bf16 tcgen05 MMA
// (fp32 accumulator in TMEM, products of bf16 inputs are exact), written out as
// three bf16 parts (hi, mid, lo) that sum to the fp32 value exactly, so that the
// rank-r contraction of the GEMM epilogue sees z at full fp32 precision.  The parts of a row sit side by
// side, z_parts[row][part][64], so that a range of rows is one contiguous block (a rank of a
// tensor-parallel group computes a range and gathers the rest).  HBM-bound: x is streamed once through a
// 6-stage TMA pipeline, one CTA per tile.  A row window [row_lo, row_hi) limits the rows written: tiles
// outside it are skipped, tiles that straddle its edge compute all their rows (rows of an MMA are
// independent, so whatever the unowned rows of x hold cannot reach an owned row) and store the owned ones.
//
// Reference arithmetic: `x.astype(f32) @ lora_a.astype(f32)`
// (skyrl/tx/kernels/quantized_lora.py:301) and the first ragged_dot of
// skyrl/tx/layers/lora.py:150; the per-adapter scaling of lora.py:155-156 is
// folded in here.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace skyrl {

constexpr int PROJ_BM = 128;
constexpr int PROJ_BK = 64;  // bf16 elements per stage row (128 bytes)
constexpr int PROJ_N = SKYRL_LORA_RANK_PAD;  // columns of one adapter; a tile of two adapters uses 2 * PROJ_N
constexpr int PROJ_STAGES = 6;
constexpr int PROJ_A_BYTES = PROJ_BM * 128;
constexpr int PROJ_B1_BYTES = PROJ_N * 128;   // one adapter's slice of A for one K block
constexpr int PROJ_B_BYTES = 2 * PROJ_B1_BYTES;
constexpr int PROJ_STAGE_BYTES = PROJ_A_BYTES + PROJ_B_BYTES;
constexpr int PROJ_BAR_OFF = PROJ_STAGES * PROJ_STAGE_BYTES;
constexpr int PROJ_SMEM_BYTES = PROJ_BAR_OFF + (2 * PROJ_STAGES + 1) * 8 + 16 + 1024;
constexpr int PROJ_THREADS = 192;
constexpr int PROJ_TMEM_COLS = 128;
constexpr int PROJ_Z_ROW = SKYRL_Z_PARTS * PROJ_N;  // bf16 elements of one row of z_parts

struct ProjParams {
  CUtensorMap tm_x;  // bf16 [M, K], box 64 x 128
  CUtensorMap tm_a;  // bf16 [A, 64, K], box 64 x 64 x 1
  const float* scaling;
  const int4* tiles;
  const int32_t* num_tiles;
  __nv_bfloat16* z_parts[8];  // [m, 6, 64]: adapter slot 0 parts (hi, mid, lo), adapter slot 1 parts; the same rows
  int z_count;                // are written to every one of the z_count destinations (a tensor-parallel rank hands
                              // its rows to every peer's workspace with plain stores; one destination otherwise)
  int row_lo, row_hi;      // rows written
  int tile_base;           // CTA b looks at tile tile_base + b (a row window needs only the tiles that can overlap it)
  int32_t* status;
  int k;
};

__global__ void __launch_bounds__(PROJ_THREADS, 1) lora_a_proj_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + PROJ_BAR_OFF);
  uint64_t* empty_bar = full_bar + PROJ_STAGES;
  uint64_t* acc_full = empty_bar + PROJ_STAGES;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_index = static_cast<int>(blockIdx.x) + p.tile_base;
  if (tile_index >= *p.num_tiles) return;  // uniform for the CTA
  const int4 tile = __ldg(p.tiles + tile_index);
  if (tile.x >= p.row_hi || tile.x + tile.y <= p.row_lo) return;  // outside the row window, also uniform

  if (threadIdx.x == 0) {
    for (int s = 0; s < PROJ_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_ptr_smem, PROJ_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int kblocks = (p.k + PROJ_BK - 1) / PROJ_BK;
  // a tile of two adapters: rows [0, split) belong to tile.z, the rest to `second`; both projections are
  // computed for all rows in one MMA of twice the width and every row keeps the one of its adapter
  const bool mixed = tile.w != 0;
  const int second = mixed ? (tile.w & 0xffff) - 1 : tile.z;
  const int split = mixed ? (tile.w >> 16) : PROJ_BM;

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&p.tm_x);
      tma_prefetch_desc(&p.tm_a);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, STATUS_TIMEOUT_PRODUCER)) break;
        unsigned char* sa = smem + stage * PROJ_STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], PROJ_A_BYTES + (mixed ? 2 : 1) * PROJ_B1_BYTES);
        tma_load_2d(sa, &p.tm_x, kb * PROJ_BK, tile.x, &full_bar[stage]);
        tma_load_3d(sa + PROJ_A_BYTES, &p.tm_a, kb * PROJ_BK, 0, tile.z, &full_bar[stage]);
        if (mixed) tma_load_3d(sa + PROJ_A_BYTES + PROJ_B1_BYTES, &p.tm_a, kb * PROJ_BK, 0, second, &full_bar[stage]);
        if (++stage == PROJ_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(IDESC_D_F32, IDESC_BF16, IDESC_BF16, PROJ_BM, mixed ? 2 * PROJ_N : PROJ_N);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < kblocks; ++kb) {
        ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * PROJ_STAGE_BYTES);
        const uint64_t adesc = make_desc_sw128(sa);
        const uint64_t bdesc = make_desc_sw128(sa + PROJ_A_BYTES);
#pragma unroll
        for (int j = 0; j < PROJ_BK / 16; ++j) mma_bf16(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | j) != 0);
        mma_commit(&empty_bar[stage]);
        if (++stage == PROJ_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) mma_commit(acc_full);
    }
  } else {
    const int r = warp * 32 + lane;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0u, abort_flag, p.status, STATUS_TIMEOUT_EPILOGUE));
    if (ok) {
      tc_fence_after_sync();
      const int64_t row = tile.x + r;
      const bool row_valid = r < tile.y && row >= p.row_lo && row < p.row_hi;
      const int slot = r >= split ? 1 : 0;  // adapter slot of this row inside its tile
      const float s = __ldg(p.scaling + (slot ? second : tile.z));
      const int nchunks = (mixed ? 2 : 1) * (PROJ_N / 32);
      for (int cc = 0; cc < nchunks; ++cc) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + cc * 32, v);
        tmem_wait_ld();
        if (row_valid) {
          const int dslot = cc / (PROJ_N / 32);      // the slot these 32 columns belong to
          const bool mine = dslot == slot;           // the other slot of a two-adapter tile is zeroed
          uint32_t hi[16], mid[16], lo[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float z0 = mine ? __fmul_rn(__uint_as_float(v[2 * i]), s) : 0.f;
            const float z1 = mine ? __fmul_rn(__uint_as_float(v[2 * i + 1]), s) : 0.f;
            const float h0 = round_bf16(z0), h1 = round_bf16(z1);
            const float r0 = __fsub_rn(z0, h0), r1 = __fsub_rn(z1, h1);  // exact
            const float m0 = round_bf16(r0), m1 = round_bf16(r1);
            hi[i] = pack_bf16x2(h0, h1);
            mid[i] = pack_bf16x2(m0, m1);
            lo[i] = pack_bf16x2(__fsub_rn(r0, m0), __fsub_rn(r1, m1));  // <= 8 bits left: exact in bf16
          }
          const int64_t off = row * PROJ_Z_ROW + dslot * 3 * PROJ_N + (cc % (PROJ_N / 32)) * 32;
          for (int d = 0; d < p.z_count; ++d) {
            __nv_bfloat16* base = p.z_parts[d] + off;
            uint4* dh = reinterpret_cast<uint4*>(base);
            uint4* dm = reinterpret_cast<uint4*>(base + PROJ_N);
            uint4* dl = reinterpret_cast<uint4*>(base + 2 * PROJ_N);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              dh[g] = make_uint4(hi[4 * g], hi[4 * g + 1], hi[4 * g + 2], hi[4 * g + 3]);
              dm[g] = make_uint4(mid[4 * g], mid[4 * g + 1], mid[4 * g + 2], mid[4 * g + 3]);
              dl[g] = make_uint4(lo[4 * g], lo[4 * g + 1], lo[4 * g + 2], lo[4 * g + 3]);
            }
          }
        }
      }
      if (p.z_count > 1) __threadfence_system();  // stores into other GPUs' memory are performed before the kernel ends
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, PROJ_TMEM_COLS);
  }
}

int launch_lora_a_proj(const void* x, int m, int k, const void* a_packed, const float* scaling, int num_adapters,
                       int rank, const int32_t* tiles, const int32_t* num_tiles, int max_tiles, void* z_parts,
                       int32_t* status, cudaStream_t stream, int row_lo, int row_hi, void* const* extra_dests,
                       int extra_count, int list_row0) {
  if (x == nullptr || a_packed == nullptr || scaling == nullptr || tiles == nullptr || num_tiles == nullptr ||
      z_parts == nullptr || status == nullptr)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: null buffer");
  if (m <= 0 || k <= 0 || num_adapters <= 0 || max_tiles <= 0)
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: non-positive shape");
  if (k % 8 != 0) return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: K must be a multiple of 8, got %d", k);
  if (rank <= 0 || rank > SKYRL_LORA_RANK_PAD)
    return fail(SKYRL_ERR_UNSUPPORTED, "lora_a_proj: rank must be in [1, %d], got %d", SKYRL_LORA_RANK_PAD, rank);
  if (!aligned16(x) || !aligned16(a_packed) || !aligned16(z_parts) || !aligned16(tiles))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: buffers must be 16-byte aligned");
  if (x == z_parts) return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: aliased buffers");
  ProjParams p;
  int rc;
  if ((rc = encode_tmap_2d(&p.tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, k, m, static_cast<uint64_t>(k) * 2,
                           PROJ_BK, PROJ_BM)))
    return rc;
  if ((rc = encode_tmap_3d(&p.tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_packed, k, SKYRL_LORA_RANK_PAD,
                           num_adapters, static_cast<uint64_t>(k) * 2,
                           static_cast<uint64_t>(k) * 2 * SKYRL_LORA_RANK_PAD, PROJ_BK, PROJ_N)))
    return rc;
  p.scaling = scaling;
  p.tiles = reinterpret_cast<const int4*>(tiles);
  p.num_tiles = num_tiles;
  if (extra_count < 0 || extra_count > 7 || (extra_count > 0 && extra_dests == nullptr))
    return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: at most 7 extra destinations");
  p.z_parts[0] = static_cast<__nv_bfloat16*>(z_parts);
  p.z_count = 1;
  for (int d = 0; d < extra_count; ++d) {
    if (extra_dests[d] == nullptr || !aligned16(extra_dests[d]))
      return fail(SKYRL_ERR_INVALID_ARGUMENT, "lora_a_proj: extra destination %d is null or not 16-byte aligned", d);
    p.z_parts[p.z_count++] = static_cast<__nv_bfloat16*>(extra_dests[d]);
  }
  p.row_lo = row_lo;
  p.row_hi = row_hi < 0 ? m : row_hi;
  p.status = status;
  p.k = k;
  static bool attr_set[MAX_DEVICES] = {};
  cudaError_t e = ensure_dynamic_smem(lora_a_proj_kernel, PROJ_SMEM_BYTES, attr_set);
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "lora_a_proj attribute: %s", cudaGetErrorString(e));
  // `tiles` lists the tiles of the sorted rows from list_row0 on (a whole block, or one row chunk of it).  A tile
  // holds at most 128 rows and is short only where an adapter's run ends, so the tile that holds row r has an
  // index in [(r - list_row0) / 128, (r - list_row0) / 128 + adapters + 1]: a row window launches only those.
  // (Every CTA asks for most of an SM's shared memory, so CTAs that would only find out that they have nothing to
  // do still queue for an SM; beside a running GEMM that queue is what the projection of a small window costs.)
  int grid = max_tiles;
  p.tile_base = 0;
  if ((p.row_lo > list_row0 || p.row_hi < m) && list_row0 >= 0 && p.row_lo >= list_row0 && p.row_hi > p.row_lo) {
    p.tile_base = (p.row_lo - list_row0) / PROJ_BM;
    const int last = (p.row_hi - 1 - list_row0) / PROJ_BM + num_adapters + 1;
    grid = last - p.tile_base + 1;
    if (grid > max_tiles - p.tile_base) grid = max_tiles - p.tile_base;
    if (grid <= 0) return SKYRL_OK;
  }
  lora_a_proj_kernel<<<grid, PROJ_THREADS, PROJ_SMEM_BYTES, stream>>>(p);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return fail(SKYRL_ERR_LAUNCH, "lora_a_proj launch: %s", cudaGetErrorString(e));
  return SKYRL_OK;
}

}  // namespace skyrl

extern "C" int skyrl_lora_a_proj_sm100_v1(const void* x, int32_t m, int32_t k, const void* lora_a_packed,
                                          const float* lora_scaling, int32_t num_adapters, int32_t rank,
                                          const int32_t* tiles, const int32_t* num_tiles, int32_t max_tiles,
                                          void* z_parts, int32_t* status, skyrl_stream_t stream) {
  return skyrl::launch_lora_a_proj(x, m, k, lora_a_packed, lora_scaling, num_adapters, rank, tiles, num_tiles,
                                   max_tiles, z_parts, status, static_cast<cudaStream_t>(stream));
}
