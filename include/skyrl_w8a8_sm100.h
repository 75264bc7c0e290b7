/*
 * C ABI of the B200 (sm_100a) W8A8 multi-LoRA MLP kernels.
 *
 * Every entry point enqueues work on the caller's CUDA stream and returns
 * without synchronising; buffers are owned by the caller (for XLA: by XLA, as
 * results of the custom call) and must stay alive until the stream reaches the
 * end of the enqueued work.  Entry points return 0 on success or a negative
 * SKYRL_ERR_* code; the message of the last error of the calling thread is
 * available from skyrl_w8a8_last_error().  They never throw and never allocate
 * device memory: scratch comes from the caller-supplied workspace.
 *
 * Naming and versioning follow the reference's native-ABI convention
 * (rocm/compile_probes/down_lora_residual_gfx1100_abi.h:12-85: versioned
 * symbols, explicit device addresses + dimensions, and the layout of every
 * argument block asserted at compile time: the SKYRL_ABI_ASSERT lines behind
 * each struct below, as down_lora_residual_gfx1100_abi.h:77-85 does).
 * Citations are file:line inside the reference project.  The header is plain
 * C (C11) and C++.
 *
 * Device data layouts
 *   activations ........ bf16 [M, K] row-major
 *   packed weight ...... int8 [ceil(K / 128), N, 128]: K-block-major, each row 128
 *                        consecutive K values of one output channel, K zero-padded
 *                        to the block (the reference stores [K, N]:
 *                        skyrl/tx/kernels/quantized_lora.py:20-41; its own design asks
 *                        for a load-time permute to a canonical device weight:
 *                        rocm/QUANTIZED_FFI.md:69-74).  Any run of output channels of
 *                        one K block is then one contiguous piece of HBM.
 *   weight scales ...... fp32 [N] (the exact value of the reference's bf16
 *                        per-output scale, group_size == K)
 *   gate_up ............ N = 2*I physical columns, interleaved
 *                        (gate0, up0, gate1, up1, ...): skyrl/tx/layers/lora.py:338-351
 *   packed LoRA A ...... bf16 [A, 64, K]  (rank padded to 64 rows with zeros; the
 *                        reference stores [A, K, r]: skyrl/tx/layers/lora.py:259-268)
 *   packed LoRA B ...... bf16 [A, N, 64]  (rank padded to 64 columns with zeros;
 *                        reference [A, r, N])
 *   LoRA scaling ....... fp32 [A]
 *   adapter ids ........ int32 [M], one per token row (NULL = every row uses adapter 0)
 */
#ifndef SKYRL_W8A8_SM100_H_
#define SKYRL_W8A8_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SKYRL_API __attribute__((visibility("default")))
#else
#define SKYRL_API
#endif

#define SKYRL_W8A8_ABI_VERSION 1
#define SKYRL_LORA_RANK_PAD 64 /* packed LoRA tables hold 64 rank slots            */
#define SKYRL_TILE_ROWS 128     /* rows of one M tile (rows of at most two adapters) */
#define SKYRL_Z_PARTS 6         /* bf16 parts of a row of the LoRA-A projection: 2 adapter slots x (hi, mid, lo) */
#define SKYRL_WEIGHT_KBLOCK 128 /* K values per block of the packed weight layout    */

#if defined(__cplusplus)
#define SKYRL_ABI_ASSERT(cond, msg) static_assert(cond, msg)
#else
#define SKYRL_ABI_ASSERT(cond, msg) _Static_assert(cond, msg)
#endif

#define SKYRL_OK 0
#define SKYRL_ERR_INVALID_ARGUMENT (-1) /* shape / alignment / null / alias violation    */
#define SKYRL_ERR_LAUNCH (-2)           /* CUDA reported an error at enqueue time        */
#define SKYRL_ERR_UNSUPPORTED (-3)      /* valid request outside the built kernel set    */
#define SKYRL_ERR_WORKSPACE (-4)        /* workspace missing, misaligned or too small    */
#define SKYRL_ERR_DRIVER (-5)           /* CUDA driver entry point unavailable           */

typedef void* skyrl_stream_t; /* cudaStream_t */

/* epilogue selector of the GEMM kernel */
#define SKYRL_EPI_LINEAR 0   /* y[M, N] bf16                                          */
#define SKYRL_EPI_SWIGLU 1   /* h[M, N/2] bf16 = silu(gate) * up on interleaved pairs */
#define SKYRL_EPI_RESIDUAL 2 /* out[M, N] bf16 = bf16(y) + residual                   */
#define SKYRL_EPI_ACC_I32 3  /* raw int32 accumulator [M, N] (parity / debug)         */
#define SKYRL_EPI_PARTIAL_F32 4 /* fp32 [M, N] before the cast (tensor-parallel partial sums) */

SKYRL_API int skyrl_w8a8_abi_version(void);
SKYRL_API const char* skyrl_w8a8_last_error(void);

/* Self-test of failure detection (no counterpart in the reference).  Every wait inside the kernels of
 * this library is bounded: when a limit runs out the kernel writes a code into the caller's device status
 * word, drains and returns, and the CUDA context stays usable.  This entry point launches one CTA that
 * waits, for `limit_ns` (at most 2 s), on a barrier nothing ever arrives at; afterwards *status holds
 * 190 and later launches on the device work as before.  Nothing faults, traps or hangs. */
SKYRL_API int skyrl_w8a8_bounded_wait_selftest_sm100_v1(int32_t* status, uint64_t limit_ns, skyrl_stream_t stream);

/* ------------------------------------------------------------------------- *
 * Stage kernels
 * ------------------------------------------------------------------------- */

/* Batches of at most SKYRL_TILE_ROWS rows (decode shapes) skip the adapter sort:
 * the operators keep token order, use one M tile and evaluate the LoRA term row
 * by row on the CUDA cores (every row carries its own adapter id), so that the
 * weights are streamed from HBM exactly once however many adapters are in use. */

/* Stable sort of token rows by adapter id and the M-tile list over the sorted
 * row space.  Replaces prepare_routing (skyrl/tx/layers/util.py:66-87: argsort,
 * bincount, unsort) and the ragged grouping of skyrl/tx/layers/lora.py:142-157.
 *   perm[i]      original row of sorted position i                 int32 [m]
 *   tiles[4*t..] (first sorted row, row count <= 128, adapter, second)  int32 [4*max_tiles]
 *                A tile holds rows of at most two adapters, so that the end of an adapter's run does
 *                not leave a partly empty tile: second == 0 for one adapter, else
 *                (second adapter + 1) | (rows of the first adapter << 16).
 *   num_tiles    device scalar, number of tiles written
 * adapter_ids == NULL: identity permutation, uniform tiles of adapter 0.
 * status: device int32, set non-zero on a bad id or tile overflow.            */
SKYRL_API int skyrl_lora_route_sm100_v1(const int32_t* adapter_ids, int32_t m, int32_t num_adapters, int32_t* perm,
                              int32_t* tiles, int32_t* num_tiles, int32_t max_tiles, int32_t* status,
                              skyrl_stream_t stream);

/* RMSNorm (optional) + per-token absmax int8 quantisation in one pass.
 * Replaces Qwen3_5RMSNorm.__call__ (skyrl/tx/models/qwen3_5.py:269-278) and
 * _dynamic_group_quantize with group_size == K
 * (skyrl/tx/kernels/quantized_lora.py:199-212).
 *   x          bf16 [*, k], row pitch x_row_stride elements
 *   rms_delta  bf16 [k] or NULL (no normalisation)
 *   row_map    int32 [m] source row of each output row, or NULL (identity)
 *   xq         int8 [m, k] codes;  sx fp32 [m] scales (1.0 for an all-zero row)
 *   xn         bf16 [m, k] normalised (and gathered) activations, or NULL     */
SKYRL_API int skyrl_rms_quant_sm100_v1(const void* x, int64_t x_row_stride, const void* rms_delta, float eps,
                             const int32_t* row_map, int32_t m, int32_t k, void* xq, float* sx, void* xn,
                             skyrl_stream_t stream);

/* Output-cotangent quantiser of the backward pass (input gradient).  The straight-through
 * backward of the W8A8 linear, _quantized_lora_linear_bwd
 * (skyrl/tx/kernels/quantized_lora.py:337-394), needs dx = dy deq(W)^T + R A^T.  This call
 * moves the weight's per-output-channel scale to the cotangent, g = dy * col_scale, and
 * splits each row of g into int8 planes g ~= s1 q1 + s2 q2 (per-row absmax / 127 scales;
 * the second plane quantises the residual of the first), so that the int8 GEMM entry point
 * over the TRANSPOSED packed weight (unit weight scales) computes g wq^T.
 *   dy         bf16 [*, n], row pitch dy_row_stride elements
 *   col_scale  fp32 [n] (the forward weight's sw)
 *   row_map    int32 [m] source row of each output row, or NULL
 *   q1, q2     int8 [m, n];  s1, s2 fp32 [m];  q2 = s2 = NULL gives one plane          */
SKYRL_API int skyrl_w8a8_grad_quant_sm100_v1(const void* dy, int64_t dy_row_stride, const float* col_scale,
                             const int32_t* row_map, int32_t m, int32_t n, void* q1, float* s1, void* q2,
                             float* s2, skyrl_stream_t stream);

/* LoRA-A projection on the tensor cores: z[i, :] = s[a] * (x[i, :] @ A[a]) for
 * the adapter a of row i's tile, written as three bf16 planes
 * (hi, mid, lo) whose sum is the fp32 value of z exactly.  Replaces the first ragged_dot of
 * skyrl/tx/layers/lora.py:150 and `x.f32 @ lora_a.f32` of
 * skyrl/tx/kernels/quantized_lora.py:301.
 *   x bf16 [m, k] in sorted row order; lora_a_packed bf16 [A, 64, k];
 *   z_parts bf16 [m, 6, 64]: per row two adapter slots of three parts each.  A row's value sits in
 *   the slot of its adapter within its tile (0 = the tile's first adapter, 1 = its second) and, in a
 *   tile of two adapters, the other slot holds zeros; the GEMM then adds slot 0 times the first
 *   adapter's B and slot 1 times the second's for all rows of the tile.  Tiles of one adapter
 *   neither write nor read slot 1.                                            */
SKYRL_API int skyrl_lora_a_proj_sm100_v1(const void* x, int32_t m, int32_t k, const void* lora_a_packed,
                               const float* lora_scaling, int32_t num_adapters, int32_t rank, const int32_t* tiles,
                               const int32_t* num_tiles, int32_t max_tiles, void* z_parts, int32_t* status,
                               skyrl_stream_t stream);

/* Grouped weights (group_size < K: GroupQuantizedWeight with several scale rows,
 * skyrl/tx/kernels/quantized_lora.py:20-41; the reference's Pallas prototype uses
 * group 64, skyrl/tx/kernels/rocm/w8a8_lora.py:44).  The caller runs one
 * single-group GEMM per K group with SKYRL_EPI_PARTIAL_F32 into slab g of
 * `slabs` (fp32 [groups, m, n], sorted rows); this adds the slabs in ascending
 * group order (quantized_lora.py:253), casts once to bf16 and writes row i to
 * out[row_map[i]].  A compatibility path: correct for any group size, not tuned. */
SKYRL_API int skyrl_group_sum_cast_sm100_v1(const float* slabs, int32_t groups, int32_t m, int32_t n, const int32_t* row_map,
                                  void* out, int64_t out_row_stride, skyrl_stream_t stream);

/* Arguments of the int8 tensor-core GEMM with fused epilogue.  Computes
 *   acc = xq @ wq^T (int32, exact);  v = (f32(acc) * sx[m]) * sw[n] + z[m,:] @ B[a]^T
 * (skyrl/tx/kernels/quantized_lora.py:242-254, 298-304) and applies `epilogue`. */
typedef struct SkyrlW8A8GemmArgs {
  uint32_t struct_size;     /* sizeof(SkyrlW8A8GemmArgs)                              */
  int32_t epilogue;         /* SKYRL_EPI_*                                             */
  int32_t m, n, k;          /* rows (sorted space), physical out features, in features */
  int32_t rank;             /* LoRA rank (0 = frozen base only), <= 64                 */
  int32_t num_adapters;
  int32_t max_tiles;        /* capacity of `tiles`                                     */
  const void* xq;           /* int8 [m, k]                                             */
  const float* sx;          /* fp32 [m]                                                */
  const void* wq;           /* int8 [ceil(k / 128), n, 128] packed                     */
  const float* sw;          /* fp32 [n]                                                */
  const void* z_parts;      /* bf16 [m, 6, 64] (see skyrl_lora_a_proj_sm100_v1) or NULL when rank == 0 */
  const void* lora_b_packed;/* bf16 [A, n, 64]                                         */
  const int32_t* tiles;     /* int32 [4 * max_tiles] from skyrl_lora_route_sm100_v1    */
  const int32_t* num_tiles; /* device scalar                                           */
  const int32_t* out_row_map; /* int32 [m]: output (and residual) row of sorted row i; NULL = identity */
  const void* residual;     /* bf16 [m, n] for SKYRL_EPI_RESIDUAL                      */
  void* out;                /* see SKYRL_EPI_*                                         */
  int64_t out_row_stride;   /* elements                                                */
  int64_t residual_row_stride;
  int32_t* status;          /* device int32, non-zero after a bounded wait ran out     */
  int32_t split_k_slabs;    /* SKYRL_EPI_ACC_I32 only: `out` holds this many [m, out_row_stride] int32 slabs
                               (<= 1: no split).  The kernel may split K over up to that many CTAs per
                               tile; split s writes its partial sums to slab s and the caller adds the
                               skyrl_w8a8_gemm_k_splits(...) slabs (int32 addition is exact)      */
  int32_t cta_limit;        /* > 0: launch at most this many CTAs (one per SM otherwise), so that a
                               collective running on another stream finds free SMs            */
  void* scatter_bases[8];   /* SKYRL_EPI_PARTIAL_F32 with scatter_rows > 0: the reduce-scatter of a row-    */
  int32_t scatter_row0;     /* parallel projection folded into the epilogue.  Sorted row i belongs to owner */
  int32_t scatter_rows;     /* o = (i - scatter_row0) / scatter_rows and its fp32 partial sums are stored   */
                            /* at scatter_bases[o] + (i - scatter_row0 - o * scatter_rows) * out_row_stride */
                            /* instead of `out`; a base may point into another GPU's memory (peer mapping): */
                            /* the kernel uses plain stores.  Rows below scatter_row0 must not occur in     */
                            /* `tiles`.  XLA inserts a separate collective here                             */
                            /* (skyrl/tx/models/qwen3_5.py:644, ("tp", "fsdp") sharding of down_proj).      */
  float* row_amax;          /* SKYRL_EPI_SWIGLU without out_row_map: fp32 [m], zeroed by the caller; the     */
                            /* epilogue leaves max |out[i, :]| of every row in it (the absmax that           */
                            /* _dynamic_group_quantize, quantized_lora.py:205, takes of the next projection's */
                            /* input), so the quantiser need not read the rows twice.  NULL: not collected.  */
  int32_t* sched;           /* two device words {tiles claimed, CTAs finished} of the kernel's dynamic tile   */
                            /* scheduler: zero when the kernel starts, left at zero when it ends, and not     */
                            /* shared with a launch that may run at the same time.  NULL: the library hands   */
                            /* out a pair from a ring of 1024 per device; that is safe while the GEMM         */
                            /* launches of a process on one device are ordered (one stream, or events), and   */
                            /* NOT safe for a captured graph replayed next to eager launches on another       */
                            /* stream (the graph keeps its pairs).  The operator entry points below keep      */
                            /* their pairs in the caller's workspace and have no such constraint.             */
  const float* z_rows;      /* Small batches (m <= SKYRL_TILE_ROWS rows in token order, every row with its    */
  const int32_t* row_adapter_ids; /* own adapter): non-NULL z_rows selects the small-batch LoRA epilogue.    */
  const void* lora_b_rows;  /* z_rows fp32 [m, 64] = s[a] * (x[i] A[a]) per row, row_adapter_ids int32 [m]    */
  int32_t lora_b_rows_rank; /* (NULL: adapter 0), lora_b_rows the dense table bf16 [A, n, lora_b_rows_rank].  */
  int32_t variant;          /* SKYRL_GEMM_VARIANT_* (0: the library chooses).                                 */
                            /* The epilogue warps evaluate z B[a]^T per row on the CUDA cores while the main  */
                            /* loop runs and add it before the single cast (skyrl/tx/layers/lora.py:142-157   */
                            /* per token); z_parts / lora_b_packed / out_row_map are then unused, K is not    */
                            /* split, and any epilogue but SKYRL_EPI_ACC_I32 is allowed.                      */
  const void* prefetch;     /* Optional: once a CTA has requested its last weight tile it asks the memory     */
  int64_t prefetch_bytes;   /* system to bring its share of [prefetch, prefetch + prefetch_bytes) into L2     */
                            /* (cp.async.bulk.prefetch.L2; 16-byte aligned address and size): the weights of  */
                            /* the NEXT GEMM of a decode step, which HBM can deliver while the short row-wise */
                            /* kernels between two GEMMs run.  No effect on any result.  0 bytes: nothing.    */
} SkyrlW8A8GemmArgs;
SKYRL_ABI_ASSERT(sizeof(SkyrlW8A8GemmArgs) == 288, "SkyrlW8A8GemmArgs layout");
SKYRL_ABI_ASSERT(offsetof(SkyrlW8A8GemmArgs, xq) == 32 && offsetof(SkyrlW8A8GemmArgs, out_row_stride) == 120 &&
                     offsetof(SkyrlW8A8GemmArgs, scatter_bases) == 152 && offsetof(SkyrlW8A8GemmArgs, sched) == 232 &&
                     offsetof(SkyrlW8A8GemmArgs, z_rows) == 240 && offsetof(SkyrlW8A8GemmArgs, lora_b_rows_rank) == 264,
                 "SkyrlW8A8GemmArgs layout");

/* Kernel variants of the GEMM for large problems (all give the same bits; the choice is a matter of speed):
 * one 128 x 256 tile per CTA; two M tiles per CTA against one weight tile; a CTA pair per 256 x 256 tile
 * (tcgen05 cta_group::2).  A forced variant that does not apply to the shape falls back to the single tile. */
#define SKYRL_GEMM_VARIANT_AUTO 0
#define SKYRL_GEMM_VARIANT_SINGLE 1
#define SKYRL_GEMM_VARIANT_TWO_TILES 2
#define SKYRL_GEMM_VARIANT_CTA_PAIR 3
#define SKYRL_GEMM_VARIANT_PROFILE 4 /* or-ed in: the MMA-issuing thread of CTA 0 adds, in units of 1024 cycles, to the
                                        three int32 words BEHIND the status word (status[1..3], which must then exist):
                                        cycles waiting for operands in shared memory; cycles waiting for a free or a
                                        rewritten accumulator; total cycles of its loop.  A diagnostic of what bounds a
                                        launch (operand feed, epilogue, or neither: the tensor pipe itself). */
SKYRL_API int skyrl_w8a8_gemm_sm100_v1(const SkyrlW8A8GemmArgs* args, skyrl_stream_t stream);
/* Number of K splits (slabs written) the GEMM uses for this shape when given `split_k_slabs` slabs. */
SKYRL_API int skyrl_w8a8_gemm_k_splits(int32_t m, int32_t n, int32_t k, int32_t split_k_slabs);

/* ------------------------------------------------------------------------- *
 * Operator entry points (what the reference's custom-call layer binds)
 * ------------------------------------------------------------------------- */

/* One W8A8 LoRA linear, y = bf16(dequant(xq wq^T) + s (x A) B).
 * Typed-FFI handler it stands in for: rocm/QUANTIZED_FFI.md:587-599
 * (x, w8, sw, a, b, scaling -> y on the caller's stream); Python operator:
 * w8a8_lora_linear / w8a8_frozen_linear, skyrl/tx/kernels/rocm/w8a8_lora.py:827-920.
 * Fused front half: bf16_rms_gate_up_lora_swiglu_contiguous,
 * skyrl/tx/kernels/rocm/bf16_rms_gate_up_lora_swiglu_contiguous.py:698-757.
 * Fused back half: bf16_lora_residual, skyrl/tx/kernels/rocm/bf16_lora_residual.py:507-566. */
#define SKYRL_LINEAR_FUSED_ROWS 1u /* batches of at most SKYRL_TILE_ROWS rows: apply scales, the per-row LoRA term, the
                                      cast and the SwiGLU / residual step in the GEMM's own epilogue (its eight epilogue
                                      warps evaluate the LoRA term while the weights stream) instead of leaving the int32
                                      accumulator in the workspace for a second, row-wise kernel.  Same bits.  One launch
                                      fewer per projection, but on B200 the two-step form is faster at decode shapes (the
                                      row-wise work is latency-bound and eight warps per SM hide less of it than a whole
                                      grid does), so it stays the default */
typedef struct SkyrlW8A8LinearArgs {
  uint32_t struct_size;
  int32_t epilogue;          /* SKYRL_EPI_LINEAR / _SWIGLU / _RESIDUAL / _ACC_I32 / _PARTIAL_F32 */
  int32_t m, n, k;
  int32_t rank;              /* 0 = frozen base only */
  int32_t num_adapters;
  uint32_t flags;            /* SKYRL_LINEAR_* */
  const void* x;             /* bf16 [m, k] */
  int64_t x_row_stride;
  const void* rms_delta;     /* bf16 [k] or NULL: RMSNorm(1 + delta) in front of the quantiser */
  float rms_eps;
  int32_t reserved1;
  const void* wq;            /* int8 [ceil(k / 128), n, 128] packed */
  const float* sw;           /* fp32 [n] */
  const void* lora_a_packed; /* bf16 [A, 64, k] */
  const void* lora_b_packed; /* bf16 [A, n, 64] */
  const float* lora_scaling; /* fp32 [A] */
  const int32_t* adapter_ids;/* int32 [m] or NULL */
  const void* residual;      /* bf16 [m, n] (SKYRL_EPI_RESIDUAL) */
  int64_t residual_row_stride;
  void* out;
  int64_t out_row_stride;
  void* workspace;           /* >= skyrl_w8a8_linear_workspace_bytes(m, n, k, num_adapters), 1024-byte aligned */
  size_t workspace_bytes;
  int32_t* status;           /* device int32, zeroed by the caller */
  void* timing_events[2];    /* optional cudaEvent_t recorded before / after the GEMM kernel */
  const void* lora_b_rows;   /* optional dense LoRA-B table bf16 [A, n, lora_b_rows_rank] (rank rounded up to 8)
                                read by the small-batch path instead of the 64-slot table */
  int32_t lora_b_rows_rank;
  int32_t reserved2;
} SkyrlW8A8LinearArgs;
SKYRL_ABI_ASSERT(sizeof(SkyrlW8A8LinearArgs) == 200, "SkyrlW8A8LinearArgs layout");
SKYRL_ABI_ASSERT(offsetof(SkyrlW8A8LinearArgs, x) == 32 && offsetof(SkyrlW8A8LinearArgs, wq) == 64 &&
                     offsetof(SkyrlW8A8LinearArgs, out) == 128 && offsetof(SkyrlW8A8LinearArgs, workspace) == 144 &&
                     offsetof(SkyrlW8A8LinearArgs, timing_events) == 168 &&
                     offsetof(SkyrlW8A8LinearArgs, lora_b_rows) == 184,
                 "SkyrlW8A8LinearArgs layout");

SKYRL_API size_t skyrl_w8a8_linear_workspace_bytes(int32_t m, int32_t n, int32_t k, int32_t num_adapters);
SKYRL_API int skyrl_w8a8_lora_forward_sm100_v1(const SkyrlW8A8LinearArgs* args, skyrl_stream_t stream);

/* One exported target per fused variant, so that a custom-call layer binds each operator to its own
 * symbol and no epilogue selector travels through the hot path (rocm/QUANTIZED_FFI.md:579-580).  Both
 * take the argument block above; `epilogue` is ignored and fixed by the entry point.
 *
 *   skyrl_rms_gate_up_w8a8_lora_swiglu_sm100_v1   h[m, n/2] = swiglu(W8A8-LoRA gate_up(rmsnorm(x))) on
 *       interleaved (gate, up) columns; `rms_delta` may be NULL (no normalisation), `residual` must be.
 *       Successor of bf16_rms_gate_up_lora_swiglu_contiguous
 *       (skyrl/tx/kernels/rocm/bf16_rms_gate_up_lora_swiglu_contiguous.py:698-757) and of the traced
 *       kernel skyrl_qwen35_bf16_contiguous_gate_up_lora_swiglu_forward
 *       (rocm/probe_bf16_rms_gate_up_lora_swiglu.py:143-188).
 *   skyrl_down_w8a8_lora_residual_sm100_v1        out[m, n] = bf16(W8A8-LoRA down(x)) + residual;
 *       `residual` is required, `rms_delta` must be NULL.  Successor of bf16_lora_residual
 *       (skyrl/tx/kernels/rocm/bf16_lora_residual.py:507-566) and of
 *       skyrl_qwen35_bf16_down_lora_residual_forward (rocm/probe_bf16_down_lora_residual.py:416-469). */
SKYRL_API int skyrl_rms_gate_up_w8a8_lora_swiglu_sm100_v1(const SkyrlW8A8LinearArgs* args, skyrl_stream_t stream);
SKYRL_API int skyrl_down_w8a8_lora_residual_sm100_v1(const SkyrlW8A8LinearArgs* args, skyrl_stream_t stream);

/* The same W8A8 LoRA linear for callers that cannot hand over a workspace.
 * This entry point has no counterpart in the reference.
 *
 * Some hosts of this library may not allocate device memory at all at the point
 * where they call it: an XLA custom-call handler that was not given a scratch
 * result runs while XLA's allocator owns every byte it planned for the program,
 * and a serving loop that has handed the whole device to another pool has
 * nothing left to ask cudaMalloc for.  For them the scratch of the call
 * (row permutation, tile list, int8 codes, scales, gathered activations and the
 * LoRA intermediate) lives in a fixed SKYRL_NOALLOC_SCRATCH_BYTES array inside
 * the library's own device image.  Every GPU on which the library is loaded
 * holds that array until the process exits.
 *
 *  - `args` is the argument block of skyrl_w8a8_lora_forward_sm100_v1; its
 *    `workspace` and `workspace_bytes` fields are ignored.  Inputs, outputs and
 *    the status word are still the caller's.
 *  - A request whose scratch need, skyrl_w8a8_linear_workspace_bytes(m, n, k,
 *    num_adapters) (about 3 * m * k bytes; m * k + 4 * m * n for m <= 128), exceeds the array is refused with
 *    SKYRL_ERR_WORKSPACE and a message naming both sizes; nothing is enqueued.
 *  - The first call on each device looks the array's device address up (with
 *    that device current).  Make that first call outside any stream capture.
 *  - The call itself allocates nothing and frees nothing.
 *  - All calls on a device share the one array, and it keeps what the previous
 *    call left in it.  Nothing in it has to start at zero (each region is fully
 *    rewritten before it is read); the tile-count word is cleared on every call
 *    all the same.  Two calls that overlap on the GPU (different streams, or
 *    different host threads without ordering between their streams) race on the
 *    array: order them. */
#define SKYRL_NOALLOC_SCRATCH_BYTES (32u << 20)
SKYRL_API int skyrl_w8a8_lora_forward_noalloc_sm100_v1(const SkyrlW8A8LinearArgs* args, skyrl_stream_t stream);

/* flags of SkyrlW8A8MlpArgs */
#define SKYRL_MLP_REUSE_ROUTING 1u /* the workspace still holds the routing (row permutation, tile list) of an
                                      earlier call with the same m and adapter_ids: skip the routing kernel.
                                      Adapter ids do not change between the layers of one forward pass. */
#define SKYRL_MLP_INPUT_PREPARED 2u /* the workspace already holds the int8 codes, scales and LoRA-A projection of
                                       this call's rows of rmsnorm(x) (written by skyrl_w8a8_mlp_tp_prepare_sm100_v1
                                       here or, through a gather, on other ranks): skip that stage. */
#define SKYRL_MLP_FINALIZE_SORTED 4u /* skyrl_w8a8_mlp_tp_finalize_sm100_v1 writes row i to out[i] (sorted order)
                                        instead of out[perm[i]]; the residual is still read at perm[i]. */
#define SKYRL_MLP_NO_ROW_AMAX 8u /* the quantiser of h finds the row absmax itself (two passes over h) instead of
                                    taking it from the gate_up epilogue; results are bit-identical (a cross-check). */

#define SKYRL_MLP_KEEP_NORMALIZED 16u /* batches of at most SKYRL_TILE_ROWS rows: also store the normalised bf16
                                         activations rmsnorm(x) in the workspace (larger batches always do), so that
                                         a stage-by-stage check can feed the oracle what the kernels saw. */

#define SKYRL_MLP_FUSED_ROWS 32u /* as SKYRL_LINEAR_FUSED_ROWS, for both projections of the block */
#define SKYRL_FLAGS_GEMM_VARIANT_SHIFT 8 /* bits 8-10 of SkyrlW8A8LinearArgs.flags / SkyrlW8A8MlpArgs.flags: a
                                            SKYRL_GEMM_VARIANT_* forced on the call's GEMMs (0: the library chooses) */

/* Whole MLP block: out = residual + down(swiglu(gate_up(rmsnorm(x)))) with the
 * per-token adapter routing done once (Qwen3_5MLP.forward_with_post_attention_rms,
 * skyrl/tx/models/qwen3_5.py:786-826; Qwen3MLP, skyrl/tx/models/qwen3.py:100-131). */
typedef struct SkyrlW8A8MlpArgs {
  uint32_t struct_size;
  int32_t m, hidden, inter;  /* rows, hidden size H, intermediate size I (gate_up has 2*I columns) */
  int32_t rank, num_adapters;
  int32_t down_epilogue;     /* SKYRL_EPI_RESIDUAL, or SKYRL_EPI_PARTIAL_F32 for a row-parallel shard */
  float rms_eps;
  const void* x;             /* bf16 [m, H] */
  const void* rms_delta;     /* bf16 [H] or NULL */
  const void* residual;      /* bf16 [m, H]; NULL = x */
  const void* gu_wq;         /* int8 [ceil(H / 128), 2I, 128] packed */
  const float* gu_sw;        /* fp32 [2I] */
  const void* gu_a_packed;   /* bf16 [A, 64, H] */
  const void* gu_b_packed;   /* bf16 [A, 2I, 64] */
  const float* gu_scaling;
  const void* dn_wq;         /* int8 [ceil(I / 128), H, 128] packed */
  const float* dn_sw;        /* fp32 [H] */
  const void* dn_a_packed;   /* bf16 [A, 64, I] */
  const void* dn_b_packed;   /* bf16 [A, H, 64] */
  const float* dn_scaling;
  const int32_t* adapter_ids;/* int32 [m] or NULL */
  void* out;                 /* RESIDUAL / LINEAR: bf16 [m, H] in token order.  PARTIAL_F32: fp32 [m, H]
                                partial sums in adapter-sorted row order, without the residual (the
                                caller reduces over ranks, then calls skyrl_w8a8_mlp_tp_finalize_sm100_v1) */
  void* workspace;           /* >= skyrl_w8a8_mlp_workspace_bytes(m, hidden, inter, num_adapters) */
  size_t workspace_bytes;
  int32_t* status;
  void* timing_events[4];    /* optional cudaEvent_t recorded on the stream: before / after the gate_up
                                GEMM, before / after the down GEMM (NULL = not recorded)             */
  uint32_t flags;            /* SKYRL_MLP_* */
  int32_t b_rows_rank;       /* row length of the dense LoRA-B tables below */
  const void* gu_b_rows;     /* optional dense tables bf16 [A, 2I, b_rows_rank] / [A, H, b_rows_rank] for the */
  const void* dn_b_rows;     /* small-batch path (see SkyrlW8A8LinearArgs.lora_b_rows)                        */
  int32_t num_chunks;        /* > 1 (and m > 128): the adapter-sorted rows are cut into this many chunks of   */
  int32_t chunk_index;       /* ceil(m / num_chunks / 128) * 128 rows and this call computes chunk            */
                             /* chunk_index only (rows [chunk_index * chunk_rows, ...) of the sorted order),  */
                             /* so that a caller can reduce chunk c over ranks while chunk c + 1 computes.    */
                             /* The first call of a block (without SKYRL_MLP_REUSE_ROUTING) routes all chunks. */
  int32_t gemm_cta_limit;    /* > 0: cap on the CTAs of the GEMM launches (see SkyrlW8A8GemmArgs.cta_limit)   */
  int32_t tp_scatter_rows;   /* > 0 (down_epilogue PARTIAL_F32): the down GEMM scatters this call's rows to   */
  void* tp_scatter_bases[8]; /* their owners, tp_scatter_rows consecutive sorted rows each starting at the    */
                             /* first row of the call's chunk (see SkyrlW8A8GemmArgs.scatter_bases); `out` is  */
                             /* then not written.                                                             */
  const void* prefetch_next; /* Batches of at most SKYRL_TILE_ROWS rows: packed weight codes of the projection  */
  int64_t prefetch_next_bytes; /* that runs after this block (the next block's gate_up) and how many of their  */
                             /* leading bytes the down GEMM should bring into L2 (SkyrlW8A8GemmArgs.prefetch); */
  int64_t prefetch_down_bytes; /* leading bytes of dn_wq the gate_up GEMM brings into L2.  0: no prefetch.      */
} SkyrlW8A8MlpArgs;
SKYRL_ABI_ASSERT(sizeof(SkyrlW8A8MlpArgs) == 336, "SkyrlW8A8MlpArgs layout");
SKYRL_ABI_ASSERT(offsetof(SkyrlW8A8MlpArgs, x) == 32 && offsetof(SkyrlW8A8MlpArgs, gu_wq) == 56 &&
                     offsetof(SkyrlW8A8MlpArgs, out) == 144 && offsetof(SkyrlW8A8MlpArgs, timing_events) == 176 &&
                     offsetof(SkyrlW8A8MlpArgs, flags) == 208 && offsetof(SkyrlW8A8MlpArgs, num_chunks) == 232 &&
                     offsetof(SkyrlW8A8MlpArgs, tp_scatter_bases) == 248,
                 "SkyrlW8A8MlpArgs layout");

SKYRL_API size_t skyrl_w8a8_mlp_workspace_bytes(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters);
SKYRL_API int skyrl_w8a8_mlp_block_sm100_v1(const SkyrlW8A8MlpArgs* args, skyrl_stream_t stream);

/* Second half of a row-parallel (tensor-parallel) block, after the fp32 partial
 * sums of all ranks were added (one all-reduce per block, as GSPMD inserts for
 * the ("tp", "fsdp") sharding of down_proj: skyrl/tx/models/qwen3_5.py:644):
 *   out[perm[i], :] = bf16( bf16(reduced[i, :]) + residual[perm[i], :] )  for sorted rows
 * i in [row_begin, row_begin + row_count).  `args` is the argument block of the
 * skyrl_w8a8_mlp_block_sm100_v1 call that produced the partial sums (same
 * workspace: it holds the row permutation); `reduced` is fp32 [m, H] in sorted order. */
SKYRL_API int skyrl_w8a8_mlp_tp_finalize_sm100_v1(const SkyrlW8A8MlpArgs* args, const float* reduced, void* out,
                                        int32_t row_begin, int32_t row_count, skyrl_stream_t stream);
/* The same for partial sums that were scattered to their owner (tp_scatter_bases) and not yet added:
 * slabs[s] holds rank s's fp32 partial sums of sorted rows [row_begin, row_begin + row_count), row i at
 * slabs[s] + (i - row_begin) * H.  The slabs are added in ascending s in fp32, the order of the group sum
 * of skyrl/tx/kernels/quantized_lora.py:253, then cast and finalized as above. */
SKYRL_API int skyrl_w8a8_mlp_tp_finalize_slabs_sm100_v1(const SkyrlW8A8MlpArgs* args, const float* const* slabs,
                                              int32_t num_slabs, void* out, int32_t row_begin, int32_t row_count,
                                              skyrl_stream_t stream);

/* Sequence-parallel form of the tensor-parallel block.  Every stage but the two GEMMs is row-wise, so a
 * rank of a tensor-parallel group need only run the stage in front of gate_up (RMSNorm, int8 codes,
 * scales, LoRA-A projection) on ITS share of the sorted rows and gather the other ranks' results, which
 * are a quarter of the bytes of the bf16 rows; behind down_proj a reduce-scatter replaces the all-reduce
 * and each rank finalizes its share only.  The reference leaves this choice to GSPMD (activations carry no
 * "tp" axis in skyrl/tx/models/qwen3_5.py:633,644, so XLA is free to shard them by rows between the two
 * collectives); the values computed per row are the same either way.
 *
 * skyrl_w8a8_mlp_tp_prepare_sm100_v1 runs that front stage for sorted rows [row_begin, row_begin +
 * row_count), which must lie inside the chunk (num_chunks, chunk_index) of `args`, and routes first unless
 * SKYRL_MLP_REUSE_ROUTING is set.  It reads args->x at perm[i] for the rows i of the range only, so x may
 * be a buffer in which only this rank's rows are current.  The caller then gathers the three regions
 * named by skyrl_w8a8_mlp_workspace_regions over the ranks and calls skyrl_w8a8_mlp_block_sm100_v1 with
 * SKYRL_MLP_INPUT_PREPARED. */
SKYRL_API int skyrl_w8a8_mlp_tp_prepare_sm100_v1(const SkyrlW8A8MlpArgs* args, int32_t row_begin, int32_t row_count,
                                       skyrl_stream_t stream);
/* Byte offsets inside an MLP workspace of the regions a gather moves, each indexed by sorted row:
 * offsets[0] int8 codes [m, hidden], offsets[1] fp32 scales [m], offsets[2] bf16 LoRA-A parts [m, 6, 64]. */
SKYRL_API int skyrl_w8a8_mlp_workspace_regions(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters,
                                     size_t* offsets);
/* Fused exchange between two blocks of a sequence-parallel stack: flag words and this library's own kernels
 * (two launches per rank and row chunk, or one with SKYRL_TP_EXCHANGE_SINGLE_KERNEL) in place of a
 * reduce-scatter, the finalize kernel, the next block's quantiser stage and the gathers of its results.
 * XLA inserts separate collectives around separately scheduled fusions here (the all-reduce behind the
 * ("tp", "fsdp") sharded down_proj, skyrl/tx/models/qwen3_5.py:644).
 *
 * For this rank's sorted rows [row_begin, row_begin + row_count) of a chunk the call
 *   - waits (bounded) until wait_flags[s] >= wait_value for every rank s: rank s raises its word in this
 *     rank's memory with skyrl_w8a8_tp_signal_sm100_v1 once its down GEMM of the chunk has completed,
 *   - reads the row's fp32 partial sums from partials[s] of EVERY rank (own buffer and peer mappings, or slabs in
 *     this rank's memory that the ranks filled; plain loads) and adds them in ascending s
 *     (skyrl/tx/kernels/quantized_lora.py:253),
 *   - writes bf16(sum) + residual to `out` (row perm[i]; row i with SKYRL_MLP_FINALIZE_SORTED set in `block`),
 *   - and, when `next` is given, runs the next block's RMSNorm + int8 quantiser on that row and stores the codes
 *     and the scale into the workspace of EVERY rank (peer_workspaces[r], all of the layout of `next`; plain
 *     stores), then projects the normalised rows onto LoRA-A and stores the parts into every workspace too.
 * Finally signal_flags[r] (one word in each rank's memory, NULL entries skipped) are set to signal_value: the
 * rows this rank owns have arrived everywhere.  A rank starts the next block's GEMMs on a chunk once the
 * word of every rank has reached that value (skyrl_w8a8_tp_wait_sm100_v1 on the GEMM's stream).
 *
 * `block` is the argument block of the skyrl_w8a8_mlp_block_sm100_v1 call that produced the partial sums (its
 * workspace holds the row permutation; x / residual give the residual), `next` that of the next block's call
 * on the same chunk (NULL behind the last block: finalize only).  Flag values must only grow from call to call.
 * No TMA and no multicast instruction touches peer memory; if a wait runs out, status 105 is recorded and the
 * kernel returns. */
#define SKYRL_TP_EXCHANGE_SINGLE_KERNEL 1u /* sum, finalize and quantise row by row in ONE kernel.  The default is
                                            * two launches on the stream: a streaming kernel that waits, sums the
                                            * slabs and finalizes (every thread keeps loads in flight all the time),
                                            * then the row-wise quantiser over the bf16 rows it wrote.  Same bits;
                                            * on the few SMs the GEMMs spare the two launches are about twice as
                                            * fast as the single kernel. */
#define SKYRL_TP_EXCHANGE_MULTIMEM 2u /* partials[0] is the MULTICAST address of a symmetric buffer that holds every
                                       * rank's partial sums at the same offset (an NVSwitch multicast object, e.g.
                                       * torch symmetric memory's multicast_ptr): the sum over ranks is formed in the
                                       * switch by one multimem.ld_reduce per 16 bytes instead of tp peer loads, so
                                       * each row crosses this GPU's links once.  fp32 additions in an order the
                                       * switch chooses: results agree with the rank-ordered forms to fp32 rounding,
                                       * not bit for bit.  partials[1..] are ignored.  Two-launch form only. */
#define SKYRL_TP_EXCHANGE_PROFILE 4u /* diagnostic: CTA 0 of the two-launch kernels adds, in units of 1.024 us, to the
                                      * words status[1], status[2], status[3] of `block` the time it spent waiting for
                                      * the flags, in the streaming sum and in the row-wise quantiser */
#define SKYRL_TP_EXCHANGE_WIDE 8u /* two-launch form: grid_ctas CTAs of 256 threads and no shared memory, which the
                                   * hardware places on every SM, also beside the persistent CTAs of a GEMM that runs
                                   * at the same time (shorter exchange, slightly slower GEMM).  Default: grid_ctas fat
                                   * CTAs (1024 threads and a shared-memory request of more than half an SM's), one
                                   * per SM and never beside a GEMM CTA: they stay on the SMs the GEMM leaves free. */
typedef struct SkyrlW8A8TpExchangeArgs {
  uint32_t struct_size;
  int32_t tp;                  /* ranks of the group, 1 ... 8                                       */
  int32_t row_begin, row_count;/* this rank's sorted rows                                           */
  int32_t wait_value;
  int32_t signal_value;
  int32_t grid_ctas;           /* CTAs of each exchange kernel; 0 = 48                              */
  uint32_t flags;              /* SKYRL_TP_EXCHANGE_*                                               */
  const float* partials[8];    /* rank s's fp32 [m, hidden] partial sums in sorted row order        */
  const int32_t* wait_flags;   /* tp words in this rank's memory, or NULL (no wait)                 */
  void* peer_workspaces[8];    /* rank r's workspace of the next block (used when next != NULL)     */
  int32_t* signal_flags[8];
  void* out;                   /* bf16 [m, hidden]                                                  */
} SkyrlW8A8TpExchangeArgs;
SKYRL_ABI_ASSERT(sizeof(SkyrlW8A8TpExchangeArgs) == 240, "SkyrlW8A8TpExchangeArgs layout");
SKYRL_ABI_ASSERT(offsetof(SkyrlW8A8TpExchangeArgs, partials) == 32 && offsetof(SkyrlW8A8TpExchangeArgs, wait_flags) == 96 &&
                     offsetof(SkyrlW8A8TpExchangeArgs, peer_workspaces) == 104 &&
                     offsetof(SkyrlW8A8TpExchangeArgs, signal_flags) == 168 && offsetof(SkyrlW8A8TpExchangeArgs, out) == 232,
                 "SkyrlW8A8TpExchangeArgs layout");
SKYRL_API int skyrl_w8a8_mlp_tp_exchange_sm100_v1(const SkyrlW8A8MlpArgs* block, const SkyrlW8A8MlpArgs* next,
                                        const SkyrlW8A8TpExchangeArgs* exchange, skyrl_stream_t stream);
/* After everything enqueued so far on `stream` has completed, set `count` (<= 8) flag words, each possibly in
 * another rank's memory (NULL entries skipped), to `value` with release semantics at system scope. */
SKYRL_API int skyrl_w8a8_tp_signal_sm100_v1(int32_t* const* flags, int32_t count, int32_t value, skyrl_stream_t stream);
/* Hold `stream` until `count` flag words in this rank's memory have all reached `value` (bounded: after 2 s
 * status 105 is recorded in *status and the stream continues). */
SKYRL_API int skyrl_w8a8_tp_wait_sm100_v1(const int32_t* flags, int32_t count, int32_t value, int32_t* status,
                                skyrl_stream_t stream);

/* Byte offsets of the intermediate results a finished skyrl_w8a8_mlp_block_sm100_v1 call leaves in its
 * workspace, for stage-by-stage parity checks: offsets[0] row permutation int32 [m] (sorted position ->
 * token row; meaningful for m > 128 with adapter ids, otherwise rows keep token order), offsets[1]
 * h = swiglu(gate_up(...)) bf16 [m, inter] in the GEMM's row order, offsets[2] int8 codes of h [m, inter],
 * offsets[3] fp32 scales of h [m], offsets[4] normalised activations rmsnorm(x) bf16 [m, hidden] in the same
 * row order (batches of at most SKYRL_TILE_ROWS rows: only with SKYRL_MLP_KEEP_NORMALIZED). */
SKYRL_API int skyrl_w8a8_mlp_workspace_stage_regions(int32_t m, int32_t hidden, int32_t inter, int32_t num_adapters,
                                           size_t* offsets);
/* out[perm[i], :] = sorted_rows[i, :] for all m rows of a bf16 [m, H] matrix (perm from the workspace of
 * `args`): the last block of a sequence-parallel stack gathers its rows in sorted order, then restores
 * token order with this. */
SKYRL_API int skyrl_w8a8_mlp_tp_unsort_sm100_v1(const SkyrlW8A8MlpArgs* args, const void* sorted_rows, void* out,
                                      skyrl_stream_t stream);

/* ------------------------------------------------------------------------- *
 * Pack helpers (load-time, device to device)
 * ------------------------------------------------------------------------- */
/* int8 [K, N] reference codes (quantized_lora.py:20-41) -> packed [ceil(K / 128), N, 128]. */
SKYRL_API int skyrl_pack_weight_kn_sm100_v1(const void* codes_kn, int32_t k, int32_t n, void* wq_blocked, skyrl_stream_t stream);
/* int8 [N, K] codes (K contiguous, as checkpoints store [out, in]) -> the same packed layout. */
SKYRL_API int skyrl_pack_weight_nk_sm100_v1(const void* codes_nk, int32_t n, int32_t k, void* wq_blocked, skyrl_stream_t stream);
/* bf16 [A, K, r] -> bf16 [A, 64, K] (skyrl/tx/layers/lora.py:259-268).                   */
SKYRL_API int skyrl_pack_lora_a_sm100_v1(const void* a_akr, int32_t num_adapters, int32_t k, int32_t rank, void* a_packed,
                               skyrl_stream_t stream);
/* bf16 [A, r, N] -> dense bf16 [A, N, rr], rr = rank rounded up to a multiple of 8 (small-batch path). */
SKYRL_API int skyrl_pack_lora_b_rows_sm100_v1(const void* b_arn, int32_t num_adapters, int32_t rank, int32_t n, void* b_rows,
                                    skyrl_stream_t stream);
/* bf16 [A, r, N] -> bf16 [A, N, 64].                                                     */
SKYRL_API int skyrl_pack_lora_b_sm100_v1(const void* b_arn, int32_t num_adapters, int32_t rank, int32_t n, void* b_packed,
                               skyrl_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SKYRL_W8A8_SM100_H_ */
