"""A stack of W8A8 multi-LoRA MLP blocks on one GPU, with row-wise stages run beside the other rows' GEMMs.

Every stage of the block is row-wise (RMSNorm, quantiser, LoRA-A projection, the two projections, SwiGLU, the
residual: qwen3_5.py:786-826), so a subset of the token rows runs through the whole stack without ever meeting
the other rows.  `MLPStack` cuts the adapter-sorted rows into chunks (the chunk form of `ops.w8a8_mlp_block`,
bit-identical with the whole call) and runs even and odd chunks on two streams.  The GEMMs are persistent
kernels with one CTA per SM, so the two streams' GEMMs follow one another on the tensor cores; the quantisers
between them are HBM-bound kernels of small CTAs without shared memory, which fit on an SM beside a GEMM CTA
and run while the OTHER chunk's GEMM computes.  (The LoRA-A projection holds shared memory and tensor memory and
waits for an SM without a GEMM CTA.)  Routing happens once per forward.

Measured on one B200 at 16384 rows x 8 Qwen3-32B-shaped blocks, two chunks: 1.5-2.5 % less time per step than
the plain loop on the same GPU (49.1-49.7 ms against 50.4-50.6 ms).  The step runs at the board's power limit,
so hiding the quantisers (13 % of the time, little of the energy) buys less than their duration, and a chunk's
GEMM beside them runs 3-4 % longer.  `num_chunks=1` is the plain loop.
"""

from __future__ import annotations

import torch

from . import ops

__all__ = ["MLPStack"]


class MLPStack:
    """blocks: sequence of (rms_delta, gate_up_weight, gate_up_lora, down_weight, down_lora) with packed weights
    and tables (`ops.PackedW8Weight`, `ops.PackedLoRA` or None).  `num_chunks=1` is the plain loop over the blocks."""

    MIN_ROWS_PER_CHUNK = 1024   # below this a chunk's GEMM is too short to hide anything behind

    def __init__(self, blocks, *, num_chunks: int = 2, eps: float = ops.RMS_EPS, gemm_variant: int = 0,
                 gemm_cta_limit: int = 0):
        self.blocks = [tuple(b) for b in blocks]
        if not self.blocks:
            raise ValueError("MLPStack needs at least one block")
        if num_chunks < 1 or num_chunks > 8:
            raise ValueError("num_chunks must be in [1, 8]")
        self.num_chunks = int(num_chunks)
        self.eps = float(eps)
        self.gemm_variant = int(gemm_variant)
        self.gemm_cta_limit = int(gemm_cta_limit)   # > 0: the GEMMs of a cut forward leave the other SMs to the other stream
        self._act = None
        self._side = None

    def chunks_for(self, m: int) -> int:
        """Chunks a forward over m rows is cut into."""
        c = self.num_chunks
        while c > 1 and ops.chunk_rows(m, c) < self.MIN_ROWS_PER_CHUNK:
            c -= 1
        return c

    def _buffers(self, x2):
        key = (tuple(x2.shape), x2.device)
        if self._act is None or self._act[0] != key:
            self._act = (key, [torch.empty(x2.shape, dtype=torch.bfloat16, device=x2.device) for _ in range(2)])
            self._side = torch.cuda.Stream(device=x2.device)
        return self._act[1]

    def forward(self, x, adapter_ids=None, *, out=None, timing_events=None):
        """x [..., hidden] bf16 -> the last block's output (a buffer of the stack that the next forward reuses,
        unless `out` is given).  `timing_events[l]` = four CUDA events recorded around block l's two GEMM
        launches (of chunk 0 when the rows are cut)."""
        ops._require_cuda(x, "x")
        x2 = x.reshape(-1, x.shape[-1])
        m = x2.shape[0]
        act = self._buffers(x2)
        layers = len(self.blocks)
        chunks = self.chunks_for(m)

        def dst_of(l):
            return out.reshape(m, -1) if (out is not None and l + 1 == layers) else act[l & 1]

        def run_chunk(c, first_prepared):
            cur = x2
            for l, blk in enumerate(self.blocks):
                ev = timing_events[l] if (timing_events is not None and c == 0) else None
                dst = dst_of(l)
                ops.w8a8_mlp_block(cur, *blk, adapter_ids, enabled=True, eps=self.eps, out=dst, timing_events=ev,
                                   chunk=(c, chunks) if chunks > 1 else None, reuse_routing=(l > 0 or chunks > 1),
                                   input_prepared=first_prepared and l == 0, gemm_variant=self.gemm_variant,
                                   gemm_cta_limit=self.gemm_cta_limit if chunks > 1 else 0)
                cur = dst
            return cur

        if chunks == 1:
            return run_chunk(0, False).reshape(*x.shape[:-1], -1)

        main, side = torch.cuda.current_stream(x2.device), self._side
        rows = ops.chunk_rows(m, chunks)
        # routing, and chunk 0's stage in front of its first GEMM, before the streams part
        ops.w8a8_mlp_block(x2, *self.blocks[0], adapter_ids, enabled=True, eps=self.eps, out=dst_of(0),
                           chunk=(0, chunks), prepare_rows=(0, min(rows, m)))
        routed = torch.cuda.Event()
        routed.record(main)
        side.wait_event(routed)
        result = None
        for c in range(chunks):
            if c * rows >= m:
                break
            with torch.cuda.stream(main if c % 2 == 0 else side):
                result = run_chunk(c, c == 0)
        joined = torch.cuda.Event()
        joined.record(side)
        main.wait_event(joined)
        return result.reshape(*x.shape[:-1], -1)

    __call__ = forward
