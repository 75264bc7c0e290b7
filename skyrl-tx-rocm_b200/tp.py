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
    """A stack of tensor-parallel MLP blocks with the all-reduce hidden behind compute.

    Every operation of the block is row-wise, so the adapter-sorted rows are cut
    into `num_chunks` chunks: while NCCL reduces chunk c of a block on a second
    stream, the kernels of chunk c + 1 (and then of the next block's chunk c)
    run on the main stream.  The GEMMs claim their tiles dynamically, so CTAs
    whose SM is held by the collective's kernels simply take fewer tiles; with
    `reserve_sms` > 0 the GEMMs additionally launch that many CTAs fewer.
    Measured on 4 GPUs (c5): 2 chunks 18.4 ms per step, 4 chunks 19.9 ms,
    unchunked 21.3 ms.  Blocks shorter than 129 rows take the small-batch path
    and are not chunked.
    """

    def __init__(self, blocks, *, group=None, num_chunks: int = 2, reserve_sms: int = 0, sm_count: int = 148):
        self.blocks = list(blocks)
        self.group = group
        self.num_chunks = num_chunks
        self.cta_limit = max(1, sm_count - reserve_sms) if reserve_sms > 0 else 0
        self._comm = None
        self._partial = None
        self._act = None

    def forward(self, x, adapter_ids=None, *, timing_events=None):
        import torch
        import torch.distributed as dist

        from . import ops

        m, hidden = x.shape
        chunks = self.num_chunks if m > ops.TILE_ROWS else 1
        if self._comm is None:
            self._comm = torch.cuda.Stream()
        if self._partial is None or self._partial.shape != (m, hidden):
            self._partial = torch.empty((m, hidden), dtype=torch.float32, device=x.device)
            self._act = [torch.empty((m, hidden), dtype=torch.bfloat16, device=x.device) for _ in range(2)]
        main = torch.cuda.current_stream()
        rows = ops.chunk_rows(m, chunks)
        spans = [(c * rows, min(rows, m - c * rows)) for c in range(chunks) if c * rows < m]
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
