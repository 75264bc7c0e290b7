"""Tensor-parallel form of the W8A8 multi-LoRA MLP block.

Sharding follows the reference's GSPMD specs: `gate_up_proj` is sharded on its
output features ("fsdp", "tp") and `down_proj` on its input features
("tp", "fsdp") (skyrl/tx/models/qwen3_5.py:633,644; skyrl/tx/models/qwen3.py:108,119);
LoRA A follows the in-feature sharding and LoRA B the out-feature sharding
(skyrl/tx/layers/lora.py:264-265).  XLA then inserts ONE all-reduce after the
row-parallel down projection; here that is an explicit NCCL all-reduce of the
fp32 partial sums.

The helpers in the first half are pure indexing (NumPy or torch tensors alike)
and run on any machine; `TensorParallelMLP` drives the CUDA library.
"""

from __future__ import annotations


def shard_bounds(inter: int, tp: int, rank: int) -> tuple[int, int]:
    """Intermediate features [lo, hi) owned by `rank`."""
    if tp <= 0 or not 0 <= rank < tp:
        raise ValueError(f"rank {rank} outside a tensor-parallel group of {tp}")
    if inter % tp:
        raise ValueError(f"intermediate size {inter} does not divide by tp={tp}")
    shard = inter // tp
    return rank * shard, (rank + 1) * shard


def shard_gate_up(codes_kn, scales_gn, lora_b, tp: int, rank: int):
    """Column shard of the fused, interleaved gate_up projection.

    The physical columns are (gate0, up0, gate1, up1, ...), so the pair range
    [lo, hi) is the contiguous column range [2*lo, 2*hi): a rank always holds
    both halves of every pair it owns.  codes [H, 2I], scales [G, 2I],
    lora_b [A, r, 2I]; LoRA A of gate_up is replicated.
    """
    inter = codes_kn.shape[1] // 2
    lo, hi = shard_bounds(inter, tp, rank)
    return codes_kn[:, 2 * lo: 2 * hi], scales_gn[:, 2 * lo: 2 * hi], lora_b[:, :, 2 * lo: 2 * hi]


def shard_down(codes_kn, lora_a, tp: int, rank: int):
    """Row shard of the down projection: codes [I, H] -> [I/tp, H], LoRA A
    [A, I, r] -> [A, I/tp, r]; the per-output-channel weight scale and LoRA B
    are replicated (the scale of a channel does not depend on the K slice)."""
    lo, hi = shard_bounds(codes_kn.shape[0], tp, rank)
    return codes_kn[lo:hi], lora_a[:, lo:hi, :]


def exchange_plan(m: int, num_chunks: int, tp: int, rank: int, tile_rows: int = 128):
    """Row bookkeeping of the sequence-parallel exchange, as plain integers.

    The sorted rows are cut into chunks of ceil(m / num_chunks) rows rounded up to the tile height; inside a
    chunk rank r owns the r-th of tp equal runs of rows.  Returns a dict with
      spans    [(first row, rows)] of the chunks,
      own      [(first row, rows)] of this rank's run in every chunk,
      own_off  offset of each chunk's run inside the rank's [m / tp]-row slab (runs stored chunk after chunk),
      own_rows m // tp, rows of one slab,
      even     whether every chunk divides by tp (otherwise the all-reduce form is used).
    """
    per = (m + num_chunks - 1) // num_chunks
    rows = (per + tile_rows - 1) // tile_rows * tile_rows
    spans = [(c * rows, min(rows, m - c * rows)) for c in range(num_chunks) if c * rows < m]
    even = all(cnt % tp == 0 for _, cnt in spans)
    own = [(r0 + rank * (cnt // tp), cnt // tp) for r0, cnt in spans]
    own_off = [sum(cnt // tp for _, cnt in spans[:c]) for c in range(len(spans))]
    return {"spans": spans, "own": own, "own_off": own_off, "own_rows": m // tp, "even": even}


class TensorParallelMLP:
    """One rank's share of an MLP block: partial sums -> all-reduce -> finalize.

    Each rank quantises its slice of `h` with its own per-token scale, which is
    the reference's group format with group_size = I / tp on the down input
    (skyrl/tx/kernels/quantized_lora.py:199-212 per group); the fp32 partial
    outputs (base and LoRA term, both linear in the K slice) are summed over
    ranks exactly like the group sum of quantized_lora.py:253.
    """

    def __init__(self, rms_delta, gate_up_weight, gate_up_lora, down_weight, down_lora, *, group=None, eps=1e-6):
        self.rms_delta = rms_delta
        self.gate_up_weight, self.gate_up_lora = gate_up_weight, gate_up_lora
        self.down_weight, self.down_lora = down_weight, down_lora
        self.group = group
        self.eps = eps
        self._partial = None

    def forward(self, x, adapter_ids=None, *, out=None, residual=None, timing_events=None, all_reduce=None,
                reuse_routing=False):
        import torch

        from . import ops

        m, hidden = x.shape[0], self.gate_up_weight.in_features
        if self._partial is None or self._partial.shape != (m, hidden) or self._partial.device != x.device:
            self._partial = torch.empty((m, hidden), dtype=torch.float32, device=x.device)
        if out is None:
            out = torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device)
        _, call = ops.w8a8_mlp_block(
            x, self.rms_delta, self.gate_up_weight, self.gate_up_lora, self.down_weight, self.down_lora, adapter_ids,
            residual=residual, enabled=True, eps=self.eps, out=self._partial, down_epilogue=ops.EPI_PARTIAL_F32,
            timing_events=timing_events, return_call=True, reuse_routing=reuse_routing)
        if all_reduce is not None:
            all_reduce(self._partial)
        else:
            import torch.distributed as dist

            dist.all_reduce(self._partial, group=self.group)
        return ops.w8a8_mlp_tp_finalize(call, self._partial, out)


class TensorParallelMLPStack:
    """A stack of tensor-parallel MLP blocks with the collectives hidden behind compute.

    Every operation of the block but the two GEMMs is row-wise, so the adapter-sorted
    rows are cut into `num_chunks` chunks and a second stream carries chunk c's
    collectives while the GEMMs of chunk c + 1 (then of the next block's chunk c) run
    on the main stream.  The GEMMs claim their tiles dynamically, so CTAs whose SM is
    held by a collective's kernels simply take fewer tiles; with `reserve_sms` > 0 the
    GEMMs additionally launch that many CTAs fewer.

    Two forms of the exchange:

    * `sequence_parallel=True` (default; needs every chunk's row count to divide by the
      group size): each rank owns 1/tp of a chunk's sorted rows between the blocks.
      Behind down_proj a reduce-scatter of the fp32 partial sums leaves a rank the sums
      of its rows, it adds the residual for them, runs the NEXT block's RMSNorm, int8
      quantisation and LoRA-A projection on them, and an all-gather hands every rank
      the codes, scales and projections of all rows (1.15 bytes per element instead of
      the 4 + 4 of an fp32 all-reduce, and none of the row-wise work is replicated).
      The last block gathers its bf16 rows in sorted order and restores token order.
    * otherwise: one fp32 all-reduce per chunk, every rank finalizes all rows and
      repeats the row-wise stages.

    With `peer_scatter` (sequence-parallel form only) the reduce-scatter is not a
    collective at all: each owner has a slab per source rank in symmetric memory, the
    ranks deliver their fp32 partial sums of the owner's rows into it, a one-word
    all-reduce orders the ranks, and the owner adds the slabs in rank order while
    finalizing.  Two ways to deliver:
      "epilogue"  the down GEMM's epilogue stores the rows straight into the owner's slab
                  (plain stores over NVLink, tile by tile while the tensor cores work on
                  the next tile); best while the GEMM is long enough to cover the
                  transfer (2 ranks);
      "copy"      the GEMM writes its partial sums locally and the copy engines push each
                  owner's rows on the second stream (no SM involved), so the transfer
                  also overlaps the other chunk's gate_up GEMM; best once the transfer
                  outlasts the down GEMM (4 and 8 ranks).
      "fused"     no collective and no copy at all between two blocks: the down GEMM leaves its partial
                  sums in this rank's symmetric buffer and raises a flag on every peer; this rank's exchange
                  kernels then pull the owned rows' partial sums from every rank over NVLink, add them
                  in rank order, finalize, run the next block's RMSNorm + quantiser and store codes,
                  scales and (after the LoRA-A projection) the projection parts straight into every
                  rank's workspace, which lives in symmetric memory too; a second flag tells the peers
                  that the rows have arrived (`ops.w8a8_mlp_tp_exchange`).  Block 0 is prepared by every
                  rank for all rows (x is replicated), so the first exchange is the one behind block 0.
      "fused_copy" the same exchange fed by the copy engines: every rank pushes each owner's rows of its partial
                  sums into a slab in the owner's memory (no SM involved, the transfer overlaps the other
                  chunk's GEMMs), raises the flag, and the owner's kernels add LOCAL slabs.  SM-issued loads over
                  NVLink ("fused", "fused_mc") move the same bytes at half the copy engines' rate and slow the
                  GEMM that runs beside them; with local slabs the exchange kernels take under 0.1 ms.
      "fused_mc"  as "fused", but the sum over ranks is formed inside NVSwitch: the exchange's streaming kernel
                  reads the MULTICAST address of the symmetric buffer with multimem.ld_reduce, so each owned row
                  crosses this GPU's links once (not tp - 1 times) and nobody pushes anything.  fp32 additions
                  in the switch's order: equal to the rank-ordered forms to fp32 rounding, not bit for bit.
                  Falls back to "fused_copy" when the fabric offers no multicast object.
    "auto" (default) = "fused_copy" on more than 2 ranks, "epilogue" on 2.
    The exchange itself is two launches (a streaming sum + finalize kernel, then a warp-per-row quantiser that
    stores codes and scales into every rank's workspace) followed by the LoRA-A projection and the flag signal;
    `exchange_wide` / `exchange_single_kernel` / `exchange_ctas` choose its launch form.  If symmetric memory cannot be set
    up the NCCL reduce-scatter is used.

    Blocks of fewer than 129 rows take the small-batch path and are not chunked.
    """

    def __init__(self, blocks, *, group=None, num_chunks: int = 2, reserve_sms: int = 8, sm_count: int = 148,
                 sequence_parallel: bool = True, peer_scatter="auto", exchange_ctas: int = 0,
                 exchange_single_kernel: bool = False, exchange_wide: bool = True, exchange_splits: int = 1):
        self.blocks = list(blocks)
        self.group = group
        self.num_chunks = num_chunks
        self.cta_limit = max(1, sm_count - reserve_sms) if reserve_sms > 0 else 0
        self.sequence_parallel = sequence_parallel
        self.peer_scatter = peer_scatter
        # Grid of the exchange kernels.  Wide form (default): four 256-thread CTAs per SM on ALL SMs, beside the GEMM's CTAs
        # (measured on 4 GPUs with the copy engines delivering the slabs: 7.26 ms per 4 layers against 8.46 for fat
        # CTAs on 8 spare SMs and 7.55 for the chain of separate kernels + NCCL gathers); fat form: one CTA per spare
        # SM; one-kernel form: six small CTAs on each spare SM.
        if exchange_ctas > 0:
            self.exchange_ctas = exchange_ctas
        elif exchange_single_kernel:
            self.exchange_ctas = max(8, 6 * reserve_sms)
        else:
            self.exchange_ctas = 4 * sm_count if exchange_wide else max(4, reserve_sms)
        self.exchange_single_kernel = bool(exchange_single_kernel)
        self.exchange_wide = bool(exchange_wide)
        self.exchange_splits = max(1, int(exchange_splits))
        self.scatter_mode = None
        self._fused = None        # symmetric buffers of the fused exchange
        self._seq = 0             # flag values only grow: one per block and forward pass
        self._slabs = None        # (shape key, local tensor, handle, per-rank base addresses, peer views)
        self._coalesce = True     # gathers of the three prepared regions go out as one NCCL group
        self._token = None
        self._comm = None
        self._copy = None
        self._partial = None
        self._act = None
        self._sorted = None
        self.trace = None   # set to a list to collect (label, stream name, event) marks of the next forward

    def _mark(self, label, stream, name):
        if self.trace is not None:
            import torch

            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            self.trace.append((label, name, ev))

    def trace_ms(self):
        """Marks of the traced forward as (label, stream name, milliseconds since the first mark)."""
        t0 = self.trace[0][2]
        return [(label, name, t0.elapsed_time(ev)) for label, name, ev in self.trace]

    def _buffers(self, x):
        import torch

        m, hidden = x.shape
        if self._comm is None:
            # high priority: its short kernels (finalize, quantise, the collectives) take the SMs first
            # whenever a GEMM launch of the main stream ends
            self._comm = torch.cuda.Stream(priority=-1)
            self._copy = torch.cuda.Stream(priority=-1)   # copy-engine pushes of the fused exchange (its kernels stay on _comm)
        if self._partial is None or self._partial.shape != (m, hidden):
            self._partial = torch.empty((m, hidden), dtype=torch.float32, device=x.device)
            self._act = [torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device) for _ in range(2)]
            self._sorted = torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device)

    def _peer_slabs(self, x, tp):
        """Symmetric fp32 [source rank, m / tp own rows, hidden] slab buffer; returns every rank's base
        address as seen from this process, or None when symmetric memory is unavailable (decided together)."""
        import torch
        import torch.distributed as dist

        m, hidden = x.shape
        key = (m, hidden, tp, x.device)
        if self._slabs is not None and self._slabs[0] == key:
            return self._slabs[3]
        ptrs, ok = None, 1
        try:
            import torch.distributed._symmetric_memory as symm

            local = symm.empty((tp * (m // tp) * hidden,), dtype=torch.float32, device=x.device)
            handle = symm.rendezvous(local, self.group if self.group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            if len(ptrs) != tp or ptrs[dist.get_rank(self.group)] != local.data_ptr():
                ok = 0
        except Exception as exc:  # noqa: BLE001 - any failure means "use the collective"
            import warnings

            warnings.warn(f"symmetric memory unavailable ({exc}); using the NCCL reduce-scatter")
            ok = 0
        flag = torch.tensor([ok], device=x.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.peer_scatter = False
            return None
        peers = [handle.get_buffer(r, (tp, m // tp, hidden), torch.float32) for r in range(tp)]
        self._slabs = (key, local, handle, ptrs, peers)
        return ptrs

    def forward(self, x, adapter_ids=None, *, timing_events=None):
        import torch
        import torch.distributed as dist

        from . import ops

        m, hidden = x.shape
        chunks = self.num_chunks if m > ops.TILE_ROWS else 1
        tp = dist.get_world_size(self.group)
        plan = exchange_plan(m, chunks, tp, dist.get_rank(self.group), ops.TILE_ROWS)
        spans = plan["spans"]
        self._buffers(x)
        if self.sequence_parallel and tp > 1 and m > ops.TILE_ROWS and self.blocks and plan["even"]:
            mode = self.peer_scatter
            if mode == "auto":
                mode = "fused_copy" if tp > 2 else "epilogue"
            if mode in ("fused", "fused_copy", "fused_mc") and self._fused_buffers(x, tp):
                if mode == "fused_mc" and not self._fused["multicast"]:
                    mode = "fused_copy"         # no multicast object on this fabric (decided together)
                return self._forward_fused(x, adapter_ids, spans, chunks, tp, timing_events, form=mode)
            return self._forward_sequence_parallel(x, adapter_ids, spans, chunks, tp, timing_events)
        main = torch.cuda.current_stream()
        prev_done = [None] * len(spans)
        cur = x
        for l, blk in enumerate(self.blocks):
            dst = self._act[l & 1]
            done = []
            for c, (r0, cnt) in enumerate(spans):
                if prev_done[c] is not None:
                    main.wait_event(prev_done[c])          # the rows this chunk gathers were finalized
                ev = timing_events[l] if (timing_events is not None and c == 0) else None
                _, call = ops.w8a8_mlp_block(
                    cur, blk.rms_delta, blk.gate_up_weight, blk.gate_up_lora, blk.down_weight, blk.down_lora,
                    adapter_ids, enabled=True, eps=blk.eps, out=self._partial, down_epilogue=ops.EPI_PARTIAL_F32,
                    timing_events=ev, return_call=True, reuse_routing=(l > 0 or c > 0),
                    chunk=(c, chunks) if chunks > 1 else None, gemm_cta_limit=self.cta_limit if chunks > 1 else 0)
                computed = torch.cuda.Event()
                computed.record(main)
                with torch.cuda.stream(self._comm):
                    self._comm.wait_event(computed)
                    dist.all_reduce(self._partial[r0:r0 + cnt], group=self.group)
                    ops.w8a8_mlp_tp_finalize(call, self._partial, dst, r0, cnt)
                    fin = torch.cuda.Event()
                    fin.record(self._comm)
                done.append(fin)
            prev_done = done
            cur = dst
        for fin in prev_done:
            main.wait_event(fin)
        return cur

    def _forward_sequence_parallel(self, x, adapter_ids, spans, chunks, tp, timing_events):
        import torch
        import torch.distributed as dist

        from . import ops

        m, hidden = x.shape
        rank = dist.get_rank(self.group)
        main, comm = torch.cuda.current_stream(), self._comm
        chunk_arg = lambda c: (c, chunks) if chunks > 1 else None
        plan = exchange_plan(m, chunks, tp, rank, ops.TILE_ROWS)
        own, own_off, own_rows = plan["own"], plan["own_off"], plan["own_rows"]
        first = self.blocks[0]
        na = first.gate_up_lora.num_adapters if first.gate_up_lora is not None else 1
        codes, scales, parts = ops.w8a8_mlp_workspace_regions(m, hidden, first.down_weight.in_features, na, x.device)
        lora = first.gate_up_lora is not None
        slab_ptrs = self._peer_slabs(x, tp) if self.peer_scatter else None
        mode = self.peer_scatter if slab_ptrs is not None else False
        if mode in (True, "auto", "fused", "fused_copy", "fused_mc"):   # the fused forms land here only when their buffers could not be set up
            mode = "epilogue" if tp <= 2 else "copy"
        peers = self._slabs[4] if slab_ptrs is not None else None
        self.scatter_mode = mode or "nccl"     # what actually delivers the partial sums, for reports
        row_bytes = hidden * 4
        if slab_ptrs is not None and self._token is None:
            self._token = torch.zeros(1, dtype=torch.int32, device=x.device)

        def scatter_arg(c):
            # owner o keeps source rank s's rows at [s, own rows of chunk 0, own rows of chunk 1, ...]
            if mode != "epilogue":
                return None
            return (own[c][1], [slab_ptrs[o] + (rank * own_rows + own_off[c]) * row_bytes for o in range(tp)])

        def push_partial(c):
            # copy engines: this rank's partial sums of owner o's rows -> o's slab for this rank.  One stream:
            # alternating the pushes between two streams made their duration erratic on 8 GPUs (0.3 to 1.1 ms
            # per chunk instead of a steady 0.3 ms).
            (r0, cnt), ocnt = spans[c], own[c][1]
            for step in range(1, tp):
                o = (rank + step) % tp       # every rank starts with a different owner
                peers[o][rank, own_off[c]:own_off[c] + ocnt].copy_(
                    self._partial[r0 + o * ocnt:r0 + (o + 1) * ocnt], non_blocking=True)

        def my_slabs(c):
            ptrs = [slab_ptrs[rank] + (s * own_rows + own_off[c]) * row_bytes for s in range(tp)]
            if mode == "copy":
                ptrs[rank] = self._partial.data_ptr() + own[c][0] * row_bytes   # own rows were never moved
            return ptrs

        def block_call(blk, src, c, **kw):
            return ops.w8a8_mlp_block(
                src, blk.rms_delta, blk.gate_up_weight, blk.gate_up_lora, blk.down_weight, blk.down_lora, adapter_ids,
                enabled=True, eps=blk.eps, out=self._partial, down_epilogue=ops.EPI_PARTIAL_F32, return_call=True,
                chunk=chunk_arg(c), gemm_cta_limit=self.cta_limit if chunks > 1 else 0, **kw)[1]

        def gather_prepared(c):
            (r0, cnt), (o0, ocnt) = spans[c], own[c]
            pairs = [(codes[r0:r0 + cnt], codes[o0:o0 + ocnt]), (scales[r0:r0 + cnt], scales[o0:o0 + ocnt])]
            if lora:
                pairs.append((parts[r0:r0 + cnt], parts[o0:o0 + ocnt]))
            done = False
            if self._coalesce:
                # one NCCL group launch for the three regions instead of three kernels
                try:
                    with dist._coalescing_manager(group=self.group, device=x.device):
                        for full, mine in pairs:
                            dist.all_gather_into_tensor(full, mine, group=self.group)
                    done = True
                except (AttributeError, RuntimeError, ValueError, TypeError):
                    self._coalesce = False
            if not done:
                for full, mine in pairs:
                    dist.all_gather_into_tensor(full, mine, group=self.group)
            ev = torch.cuda.Event()
            ev.record(comm)
            return ev

        # block 0: x is complete on every rank; each prepares its rows, the gathers run on the second stream
        gathered = []
        self._mark("begin", main, "main")
        for c in range(len(spans)):
            block_call(first, x, c, reuse_routing=c > 0, prepare_rows=own[c])
            prepared = torch.cuda.Event()
            prepared.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(prepared)
                gathered.append(gather_prepared(c))
        cur = x
        final = []
        for l, blk in enumerate(self.blocks):
            dst = self._act[l & 1]
            last = l + 1 == len(self.blocks)
            for c, (r0, cnt) in enumerate(spans):
                o0, ocnt = own[c]
                main.wait_event(gathered[c])
                self._mark(f"L{l}c{c} gemms>", main, "main")
                ev = timing_events[l] if (timing_events is not None and c == 0) else None
                call = block_call(blk, cur, c, reuse_routing=True, input_prepared=True, timing_events=ev,
                                  scatter=scatter_arg(c))
                self._mark(f"L{l}c{c} gemms<", main, "main")
                computed = torch.cuda.Event()
                computed.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(computed)
                    self._mark(f"L{l}c{c} reduce_scatter>", comm, "comm")
                    if slab_ptrs is None:
                        dist.reduce_scatter_tensor(self._partial[o0:o0 + ocnt], self._partial[r0:r0 + cnt],
                                                   group=self.group)

                        def finalize(dst_rows, **kw):
                            return ops.w8a8_mlp_tp_finalize(call, self._partial, dst_rows, o0, ocnt, **kw)
                    else:
                        if mode == "copy":
                            push_partial(c)
                        # every rank's down GEMM (or copies) of this chunk has finished once this one-word sum
                        # returns, and with it the stores into this rank's slabs
                        dist.all_reduce(self._token, group=self.group)

                        def finalize(dst_rows, **kw):
                            return ops.w8a8_mlp_tp_finalize_slabs(call, my_slabs(c), dst_rows, o0, ocnt, **kw)
                    self._mark(f"L{l}c{c} reduce_scatter<", comm, "comm")
                    if last:
                        finalize(self._sorted, sorted_out=True)
                        dist.all_gather_into_tensor(self._sorted[r0:r0 + cnt], self._sorted[o0:o0 + ocnt],
                                                    group=self.group)
                        fin = torch.cuda.Event()
                        fin.record(comm)
                        final.append((fin, call))
                    else:
                        finalize(dst)
                        block_call(self.blocks[l + 1], dst, c, reuse_routing=True, prepare_rows=own[c])
                        self._mark(f"L{l}c{c} finalize+prepare<", comm, "comm")
                        gathered[c] = gather_prepared(c)
                        self._mark(f"L{l}c{c} gather<", comm, "comm")
            cur = dst
        for fin, _ in final:
            main.wait_event(fin)
        return ops.w8a8_mlp_tp_unsort(final[-1][1], self._sorted, cur)

    # ------------------------------------------------------------------ fused exchange (no collective between blocks)
    MAX_CHUNK_SLOTS = 16

    def _fused_buffers(self, x, tp):
        """One symmetric allocation per rank: [fp32 partial sums m x hidden | slabs tp x m/tp x hidden fp32 (the other
        ranks' partial sums of this rank's rows, when the copy engines deliver them) | MLP workspace | flag words].
        Returns False (decided together) when symmetric memory is unavailable."""
        import torch
        import torch.distributed as dist

        from . import _lib, ops

        m, hidden = x.shape
        first = self.blocks[0]
        inter = first.down_weight.in_features
        na = first.gate_up_lora.num_adapters if first.gate_up_lora is not None else 1
        key = (m, hidden, inter, na, tp, x.device)
        if self._fused is not None and self._fused["key"] == key:
            return True
        ws_bytes = _lib.load().skyrl_w8a8_mlp_workspace_bytes(m, hidden, inter, na)
        up = lambda v: (v + 1023) // 1024 * 1024
        off_slabs = up(m * hidden * 4)
        off_ws = off_slabs + up(tp * (m // tp) * hidden * 4)
        off_flags = off_ws + up(ws_bytes + 1024)
        total = off_flags + 2 * self.MAX_CHUNK_SLOTS * 8 * 4
        ok, local, ptrs, mc_ptr = 1, None, None, 0
        try:
            import torch.distributed._symmetric_memory as symm

            local = symm.empty((total,), dtype=torch.uint8, device=x.device)
            handle = symm.rendezvous(local, self.group if self.group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            if len(ptrs) != tp or ptrs[dist.get_rank(self.group)] != local.data_ptr() or any(p % 1024 for p in ptrs):
                ok = 0
            mc_ptr = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception as exc:  # noqa: BLE001 - any failure means "use the collective"
            import warnings

            warnings.warn(f"symmetric memory unavailable ({exc}); using the NCCL reduce-scatter")
            ok = 0
        flag = torch.tensor([ok, 1 if (ok and mc_ptr and mc_ptr % 1024 == 0) else 0], device=x.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag[0].item()) == 0:
            self.peer_scatter = "copy"
            return False
        local[off_flags:].zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)       # every rank's flag words are zero before anyone raises one
        self._fused = {
            "key": key, "local": local, "handle": handle, "ptrs": ptrs, "off_ws": off_ws, "off_flags": off_flags,
            "multicast": mc_ptr if int(flag[1].item()) else 0,
            "off_slabs": off_slabs,
            "peer_slabs": [handle.get_buffer(r, (tp, m // tp, hidden), torch.float32, off_slabs // 4) for r in range(tp)],
            "partial": local[: m * hidden * 4].view(torch.float32).view(m, hidden),
            "workspace": local[off_ws: off_ws + ws_bytes + 1024],
            "flags": local[off_flags:].view(torch.int32).view(2, self.MAX_CHUNK_SLOTS, 8),
        }
        ops.use_workspace(self._fused["workspace"])
        self._seq = 0
        return True

    def _forward_fused(self, x, adapter_ids, spans, chunks, tp, timing_events, form="fused_copy"):
        import torch
        import torch.distributed as dist

        from . import ops

        m, hidden = x.shape
        rank = dist.get_rank(self.group)
        main, comm = torch.cuda.current_stream(), self._comm
        fb = self._fused
        ptrs, off_ws, off_flags = fb["ptrs"], fb["off_ws"], fb["off_flags"]
        partial, flags = fb["partial"], fb["flags"]
        plan = exchange_plan(m, chunks, tp, rank, ops.TILE_ROWS)
        own, own_off, own_rows = plan["own"], plan["own_off"], plan["own_rows"]
        chunk_arg = lambda c: (c, chunks) if chunks > 1 else None
        layers = len(self.blocks)
        base = self._seq
        self._seq += layers
        pull = form in ("fused", "fused_mc")   # partial sums stay where the GEMM wrote them; the exchange reads across NVLink
        multimem = form == "fused_mc"
        self.scatter_mode = form
        row_bytes = hidden * 4
        peer_slabs, slab_base = fb["peer_slabs"], ptrs[rank] + fb["off_slabs"]

        def partial_sources(c):
            """Address of every rank's partial sums such that `address + sorted_row * row_bytes` is the row: the
            ranks' own buffers (pull over NVLink), or this rank's slabs (rank s's rows sit at slab s, chunk after
            chunk) with its own buffer for its own share."""
            if multimem:
                return [fb["multicast"]]      # one address: the switch adds every rank's copy
            if pull:
                return [p for p in ptrs]
            o0 = own[c][0]
            return [ptrs[rank] if s == rank else slab_base + ((s * own_rows + own_off[c]) - o0) * row_bytes
                    for s in range(tp)]

        # what does not change from pass to pass is built once per (shape, ids buffer): at 8 ranks a chunk's GEMMs
        # take under half a millisecond, and the host has to enqueue a whole (block, chunk) iteration in that time
        ckey = (m, hidden, tp, chunks, form, adapter_ids.data_ptr() if adapter_ids is not None else 0, x.data_ptr())
        caches = fb.setdefault("caches", {})
        cache = caches.get(ckey)
        if cache is None:
            if len(caches) >= 8:            # a caller that feeds ever new buffers keeps only the latest few
                caches.clear()
            cache = caches[ckey] = {"push": {}, "next": {}}

        # A chunk's delivery and exchange may be cut into `splits` runs of the own rows: the copy engines push run j + 1
        # while the exchange kernels work on run j, so what follows a chunk's GEMMs is one run's push plus the runs'
        # exchanges instead of the whole push plus the whole exchange.  The GEMMs stay one launch per chunk.
        splits = self.exchange_splits if not pull else 1
        if any(cnt_own % splits for _, cnt_own in own) or len(spans) * splits > self.MAX_CHUNK_SLOTS:
            splits = 1
        slot = lambda c, j: c * splits + j

        def push_partial(c, j):
            # copy engines: this rank's partial sums of run j of owner o's rows -> o's slab for this rank
            pairs = cache["push"].get((c, j))
            if pairs is None:
                (r0, cnt), ocnt = spans[c], own[c][1]
                sub = ocnt // splits
                pairs = cache["push"][c, j] = [
                    (peer_slabs[o][rank, own_off[c] + j * sub:own_off[c] + (j + 1) * sub],
                     partial[r0 + o * ocnt + j * sub:r0 + o * ocnt + (j + 1) * sub])
                    for o in ((rank + step) % tp for step in range(1, tp))]   # every rank starts with a different owner
            for dst_view, src_view in pairs:
                dst_view.copy_(src_view, non_blocking=True)

        def flag_addr(r, kind, c, src):
            # word [kind][c][src] of rank r's flag block: raised by rank `src`
            return ptrs[r] + off_flags + ((kind * self.MAX_CHUNK_SLOTS + c) * 8 + src) * 4

        def block_call(blk, src, c, **kw):
            return ops.w8a8_mlp_block(
                src, blk.rms_delta, blk.gate_up_weight, blk.gate_up_lora, blk.down_weight, blk.down_lora, adapter_ids,
                enabled=True, eps=blk.eps, out=partial, down_epilogue=ops.EPI_PARTIAL_F32, return_call=True,
                chunk=chunk_arg(c), gemm_cta_limit=self.cta_limit if chunks > 1 else 0, **kw)[1]

        # block 0: x is complete on every rank, so every rank prepares all rows itself (once per pass)
        first = self.blocks[0]
        self._mark("begin", main, "main")
        for c, (r0, cnt) in enumerate(spans):
            block_call(first, x, c, reuse_routing=c > 0, prepare_rows=(r0, cnt))
        cur = x
        final = []
        exchanged = [None] * len(spans)
        for l, blk in enumerate(self.blocks):
            dst = self._act[l & 1]
            last = l + 1 == layers
            value = base + l + 1
            for c, (r0, cnt) in enumerate(spans):
                o0, ocnt = own[c]
                sub = ocnt // splits
                if l > 0:
                    main.wait_event(exchanged[c])               # this rank's own exchange first (an event, not a spin) ...
                    for j in range(splits):                     # ... then every other rank's rows of this chunk
                        ops.tp_wait(flags[1, slot(c, j)], tp, value - 1)
                self._mark(f"L{l}c{c} gemms>", main, "main")
                ev = timing_events[l] if (timing_events is not None and c == 0) else None
                call = block_call(blk, cur, c, reuse_routing=True, input_prepared=True, timing_events=ev)
                if pull:
                    ops.tp_signal([flag_addr(r, 0, c, rank) for r in range(tp)], value)   # my partial sums are complete
                self._mark(f"L{l}c{c} gemms<", main, "main")
                computed = torch.cuda.Event()
                computed.record(main)
                pushed = []
                if not pull:
                    # Copy engines on a stream of their own: the pushes of this chunk overlap the exchange kernels of
                    # the chunk (or run) before it (one stream for both made every exchange wait for the previous one's
                    # kernels: 0.33 ms of pushes + 0.35 ms of kernels per chunk in series on 8 GPUs, more than a
                    # chunk's GEMMs).  The exchange kernels are ordered behind this rank's OWN signal by an event, so
                    # that they only ever spin on flags other GPUs raise.
                    with torch.cuda.stream(self._copy):
                        self._copy.wait_event(computed)
                        self._mark(f"L{l}c{c} push>", self._copy, "copy")
                        for j in range(splits):
                            push_partial(c, j)
                            ops.tp_signal([flag_addr(r, 0, slot(c, j), rank) for r in range(tp)], value)   # my rows have arrived
                            ev_pushed = torch.cuda.Event()
                            ev_pushed.record(self._copy)
                            pushed.append(ev_pushed)
                        self._mark(f"L{l}c{c} pushed", self._copy, "copy")
                with torch.cuda.stream(comm):
                    if pull:
                        comm.wait_event(computed)
                    nxt = None
                    if not last:
                        nxt = cache["next"].get((l, c))
                        if nxt is None:
                            nb = self.blocks[l + 1]
                            nxt = cache["next"][l, c] = ops.w8a8_mlp_block(
                                dst, nb.rms_delta, nb.gate_up_weight, nb.gate_up_lora, nb.down_weight, nb.down_lora,
                                adapter_ids, enabled=True, eps=nb.eps, out=partial, down_epilogue=ops.EPI_PARTIAL_F32,
                                chunk=chunk_arg(c), reuse_routing=True, build_only=True)[1]
                    for j in range(splits):
                        if not pull:
                            comm.wait_event(pushed[j])
                        if j == 0:
                            self._mark(f"L{l}c{c} exchange>", comm, "comm")
                        ops.w8a8_mlp_tp_exchange(
                            call, nxt, self._sorted if last else dst, tp=tp, row_begin=o0 + j * sub, row_count=sub,
                            partials=partial_sources(c), wait_flags=flags[0, slot(c, j)], wait_value=value,
                            peer_workspaces=[p + off_ws for p in ptrs] if nxt is not None else None,
                            signal_flags=[flag_addr(r, 1, slot(c, j), rank) for r in range(tp)] if nxt is not None else None,
                            signal_value=value, sorted_out=last, grid_ctas=self.exchange_ctas,
                            single_kernel=self.exchange_single_kernel and not multimem, multimem=multimem,
                            profile=self.trace is not None, wide=self.exchange_wide)
                    self._mark(f"L{l}c{c} exchange<", comm, "comm")
                    exchanged[c] = torch.cuda.Event()
                    exchanged[c].record(comm)
                    if last:
                        dist.all_gather_into_tensor(self._sorted[r0:r0 + cnt], self._sorted[o0:o0 + ocnt], group=self.group)
                        fin = torch.cuda.Event()
                        fin.record(comm)
                        final.append((fin, call))
            cur = dst
        for fin, _ in final:
            main.wait_event(fin)
        return ops.w8a8_mlp_tp_unsort(final[-1][1], self._sorted, cur)
