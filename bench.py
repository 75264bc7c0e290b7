"""Benchmark of the B200 W8A8 multi-LoRA MLP path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1..c5] [--impl reference]

Prints ONE JSON line on rank 0.  A step is one pass of the hot path over one
batch of seeded synthetic input:

  c5 (default)  Qwen3-32B-shaped MLP stack: hidden 5120, intermediate 25600,
                M = 16384 tokens, 16 adapters of rank 64 with uniform per-token
                ids, 8 stacked layers.  With --gpus N > 1 the block is
                tensor-parallel (gate_up column-sharded on gate/up pairs, down
                row-sharded, one NCCL all-reduce per block): total work is
                fixed, so scaling is "strong".
  c2            decode-shape Qwen3-8B MLP: hidden 4096, intermediate 12288,
                M = 64, 32 adapters of rank 16, 36 layers (HBM-bound).
  c1, c3, c4    single linear / prefill gate_up / prefill down configurations.

`value` is tokens/s with every input resident in HBM; `e2e` is the same metric
through the public Python operator with HOST input and output buffers (pinned),
host<->device copies inside the timed region.  `--impl reference` times the CPU
statement of the reference's algorithm (NumPy port, all host threads) on a
bounded row sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: kind, M, hidden(K), inter(N/2 or N), rank, adapters, layers, ids
    "c1": dict(kind="linear", m=256, k=1024, n=3072, rank=8, adapters=1, layers=1, ids="single", bound="tensor"),
    "c2": dict(kind="mlp", m=64, hidden=4096, inter=12288, rank=16, adapters=32, layers=36, ids="uniform", bound="hbm"),
    "c3": dict(kind="gate_up", m=8192, k=4096, n=24576, rank=32, adapters=4, layers=1, ids="runs512", bound="tensor"),
    "c4": dict(kind="down", m=16384, k=12288, n=4096, rank=32, adapters=8, layers=1, ids="uniform", bound="tensor"),
    "c5_gate_up": dict(kind="gate_up", m=16384, k=5120, n=51200, rank=64, adapters=16, layers=1, ids="uniform", bound="tensor"),
    "c5": dict(kind="mlp", m=16384, hidden=5120, inter=25600, rank=64, adapters=16, layers=8, ids="uniform", bound="tensor"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        mx.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = sorted(sm)[len(sm) // 2:]  # upper half: samples taken under load
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# --------------------------------------------------------------------------- #
# synthetic, seeded inputs (generated on the device in the packed layout)
# --------------------------------------------------------------------------- #
def full_weight(torch, n, k, seed, device):
    """W ~ N(0, 0.02) bf16 [n, k] ([out, in]), the whole projection from ONE seed (every tensor-parallel rank
    draws the same matrix and cuts its shard from it, so that all GPU counts compute the same model)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = torch.empty((n, k), dtype=torch.bfloat16, device=device)
    rows = max(1, (64 << 20) // k)
    for r0 in range(0, n, rows):
        r1 = min(n, r0 + rows)
        w[r0:r1] = (torch.randn((r1 - r0, k), generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return w


def quantize_nk(torch, w):
    """Per-output-channel absmax int8 of a bf16 [n, k] matrix (quantized_lora.py:150-171 with one group over
    all of K: codes from the fp32 scale, stored scale rounded to bf16).  Returns (codes int8 [n, k], fp32 [n])."""
    n, k = w.shape
    wq = torch.empty((n, k), dtype=torch.int8, device=w.device)
    sw = torch.empty((n,), dtype=torch.float32, device=w.device)
    rows = max(1, (64 << 20) // k)
    for r0 in range(0, n, rows):
        r1 = min(n, r0 + rows)
        wf = w[r0:r1].float()
        amax = wf.abs().amax(dim=1)
        qmax = torch.full((), 127.0, dtype=torch.float32, device=w.device)   # tensor divisor: a true fp32 division
        scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
        wq[r0:r1] = torch.clamp(torch.round(wf / scale[:, None]), -127, 127).to(torch.int8)
        sw[r0:r1] = scale.to(torch.bfloat16).float()
    return wq, sw


def synth_weight(S, torch, n, k, seed, device, keep_host=False):
    """Packed per-output-channel W8 weight of a seeded [n, k] matrix; with `keep_host` also the oracle's view of
    it (codes [K, N], bf16 scales [1, N]) for the parity check."""
    wq, sw = quantize_nk(torch, full_weight(torch, n, k, seed, device))
    packed = S.pack_weight_nk(wq, sw)
    return (packed, host_weight(torch, [wq], [sw])) if keep_host else packed


def host_weight(torch, codes_nk_groups, scales_groups):
    """Oracle storage (quantized_lora.py:20-41) of a weight given as K groups of [n, k_g] codes with fp32 [n]
    scales each: codes int8 [K, N], scales bf16 [groups, N], group_size = k_g."""
    import ml_dtypes
    import numpy as np

    from oracle import w8a8_oracle as O

    codes = np.concatenate([c.t().contiguous().cpu().numpy() for c in codes_nk_groups], axis=0)
    scales = np.stack([s_.cpu().numpy() for s_ in scales_groups], axis=0).astype(ml_dtypes.bfloat16)
    k = codes.shape[0]
    return O.GroupQuantizedWeight(codes, scales, k, k, 8, k // len(codes_nk_groups))


def synth_lora(S, torch, adapters, k, rank, n, alpha, seed, device, rows=None, cols=None, keep_host=False):
    """LoRA tables A [adapters, k, rank] ~ N(0, 1/sqrt(k)), B [adapters, rank, n] ~ N(0, 0.02) from one seed.
    A tensor-parallel rank keeps rows [rows[0], rows[1]) of A's K axis or columns [cols[0], cols[1]) of B's N
    axis (skyrl/tx/layers/lora.py:264-265: A follows the in-feature sharding, B the out-feature sharding)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    a = (torch.randn((adapters, k, rank), generator=gen, device=device) / (k ** 0.5)).to(torch.bfloat16)
    b = (torch.randn((adapters, rank, n), generator=gen, device=device) * 0.02).to(torch.bfloat16)
    s = torch.full((adapters,), alpha / rank, dtype=torch.float32, device=device)
    host = None
    if keep_host:
        import ml_dtypes

        bf16 = ml_dtypes.bfloat16
        host = (a.cpu().view(torch.uint16).numpy().view(bf16), b.cpu().view(torch.uint16).numpy().view(bf16),
                s.cpu().numpy())
    a_sh = a[:, rows[0]:rows[1]].contiguous() if rows is not None else a
    b_sh = b[:, :, cols[0]:cols[1]].contiguous() if cols is not None else b
    packed = S.pack_lora(a_sh, b_sh, s, in_features=a_sh.shape[1], padded_out_features=b_sh.shape[2])
    return (packed, host) if keep_host else packed


def synth_ids(torch, m, adapters, mode, seed):
    gen = torch.Generator().manual_seed(seed)
    if mode == "single":
        return None
    if mode == "runs512":
        runs = torch.randint(0, adapters, ((m + 511) // 512,), generator=gen, dtype=torch.int32)
        return runs.repeat_interleave(512)[:m].contiguous()
    return torch.randint(0, adapters, (m,), generator=gen, dtype=torch.int32)


# --------------------------------------------------------------------------- #
# the device arm
# --------------------------------------------------------------------------- #
def load_traffic(workload, m):
    """DRAM bytes of one launch of the dominant kernel, from a committed ncu capture (profiles/gemm_traffic.json:
    dram__bytes_read.sum + dram__bytes_write.sum of one launch at `m` rows, scaled by the rows when the bench
    runs more, which every term of the traffic grows with).  None when no capture of this workload is committed."""
    path = os.path.join(ROOT, "profiles", "gemm_traffic.json")
    if not os.path.exists(path):
        return None, None
    try:
        with open(path) as f:
            entry = json.load(f).get(workload)
    except (OSError, ValueError):
        return None, None
    if not entry:
        return None, None
    scale = m / entry["m"]
    note = f"ncu capture at M={entry['m']}" + ("" if scale == 1 else f", scaled by {scale:g} (rows)")
    return (entry["dram_bytes_read"] + entry["dram_bytes_write"]) * scale, note


def init_distributed(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # The collectives left on this path are small (flags, the last block's gather, the upload gather); every
        # multi-GPU number of this repository was taken with NCCL's in-switch (NVLS) algorithms off, which also keeps
        # NCCL from binding multicast objects beside the symmetric-memory buffers.  Export NCCL_NVLS_ENABLE=1 to override.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        if args.nccl_max_ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.nccl_max_ctas))
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            del os.environ["NCCL_DEBUG"]  # its banner goes to stdout; this program prints exactly one JSON line
        dist.init_process_group("nccl", device_id=device)
    return rank, local_rank, world, device, dist


def run_device(args):
    rank, local_rank, world, device, dist = init_distributed(args)
    line, ok = measure(args, args.workload, args.steps, rank, local_rank, world, device, dist)
    if rank == 0 and world == 1 and args.workload == "c5" and not args.no_decode:
        # the HBM-bound decode configuration beside the tensor-bound headline, outside its timed region
        sub, sub_ok = measure(args, "c2", max(args.steps, 300), rank, local_rank, world, device, dist, sub=True)
        line["decode"] = {k_: sub[k_] for k_ in ("value", "unit", "ms_per_step", "steps", "config", "roofline", "clocks",
                                                 "e2e", "gpu_launches", "parity")}
        ok = ok and sub_ok
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    if not ok:
        raise SystemExit(3)   # the line above says which parity check failed


def measure(args, workload, steps, rank, local_rank, world, device, dist, sub=False):
    """Build one workload, check it against the oracle on sampled rows, time it.  Returns (line dict, parity ok)."""
    import torch

    import skyrl_tx_rocm_b200 as S

    wl = dict(WORKLOADS[workload])
    if args.m and not sub:
        wl["m"] = args.m
    if args.layers and not sub:
        wl["layers"] = args.layers
    kind, m, layers = wl["kind"], wl["m"], wl["layers"]
    tp = world
    if tp > 1 and kind != "mlp":
        raise SystemExit("tensor parallelism is benchmarked on the MLP workloads (c5, c2)")
    peaks = load_peaks()
    alpha = 2.0 * wl["rank"]
    want_parity = not args.no_parity

    # ---------------- build the workload ----------------
    ids_host = synth_ids(torch, m, wl["adapters"], wl["ids"], 7)
    ids = ids_host.to(device) if ids_host is not None else None
    ids_np = ids_host.numpy() if ids_host is not None else None
    gen = torch.Generator(device=device).manual_seed(11)
    parity_inputs = None
    if kind == "mlp":
        hidden, inter = wl["hidden"], wl["inter"]
        if inter % tp or (inter // tp) % 16:
            raise SystemExit("intermediate size must split into multiples of 16 per rank")
        ish = inter // tp
        lo, hi = rank * ish, (rank + 1) * ish
        x_host = torch.randn((m, hidden), generator=torch.Generator().manual_seed(5), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        blocks = []
        for l in range(layers):
            seed = ((5000 if workload == "c5" else 1000) + l) * 131
            keep = want_parity and l == 0 and rank == 0
            delta = (torch.randn((hidden,), generator=gen, device=device) * 0.02).to(torch.bfloat16)
            # ONE seeded full weight per projection; a rank keeps gate/up pairs [lo, hi) (rows 2 lo .. 2 hi of the
            # interleaved [2I, H] matrix) and columns [lo, hi) of down's [H, I], quantised over its own K slice
            w_full = full_weight(torch, 2 * inter, hidden, seed + 1, device)
            gq, gs = quantize_nk(torch, w_full[2 * lo:2 * hi])
            gu_w = S.pack_weight_nk(gq, gs)
            gu_host = None
            if keep:
                gu_host = host_weight(torch, [gq], [gs]) if tp == 1 else host_weight(torch, *[[t] for t in quantize_nk(torch, w_full)])
            del w_full, gq, gs
            w_full = full_weight(torch, hidden, inter, seed + 2, device)
            dq, ds = quantize_nk(torch, w_full[:, lo:hi].contiguous())
            dn_w = S.pack_weight_nk(dq, ds)
            dn_host = None
            if keep:
                shards = [quantize_nk(torch, w_full[:, r * ish:(r + 1) * ish].contiguous()) for r in range(tp)] if tp > 1 else [(dq, ds)]
                dn_host = host_weight(torch, [c for c, _ in shards], [s_ for _, s_ in shards])
                del shards
            del w_full, dq, ds
            gu_l = synth_lora(S, torch, wl["adapters"], hidden, wl["rank"], 2 * inter, alpha, seed + 3, device,
                              cols=(2 * lo, 2 * hi), keep_host=keep)
            dn_l = synth_lora(S, torch, wl["adapters"], inter, wl["rank"], hidden, alpha, seed + 4, device,
                              rows=(lo, hi), keep_host=keep)
            if keep:
                parity_inputs = dict(delta=delta, gate_up=(gu_host, gu_w, gu_l[1], gu_l[0]), down=(dn_host, dn_w, dn_l[1], dn_l[0]))
                gu_l, dn_l = gu_l[0], dn_l[0]
            blocks.append((delta, gu_w, gu_l, dn_w, dn_l))
            torch.cuda.empty_cache()
        tp_stack = None
        if tp > 1:
            from skyrl_tx_rocm_b200.tp import TensorParallelMLP, TensorParallelMLPStack

            def make_stack(blks):
                return TensorParallelMLPStack([TensorParallelMLP(*b) for b in blks], num_chunks=args.tp_chunks,
                                              reserve_sms=args.tp_reserve_sms,
                                              sequence_parallel=bool(args.tp_sequence_parallel),
                                              peer_scatter=False if args.tp_peer_scatter == "off" else args.tp_peer_scatter,
                                              exchange_ctas=args.tp_exchange_ctas)

            tp_stack = make_stack(blocks)
        x_dev = x_host.to(device)
        act = [torch.empty((m, hidden), dtype=torch.bfloat16, device=device) for _ in range(2)]
        ops_per_step = 2.0 * m * (hidden * 2 * inter + inter * hidden) * layers  # whole job, all ranks
        # one GPU, many rows: the rows run as chunks on two streams (skyrl_tx_rocm_b200.stack.MLPStack)
        row_stack, row_chunks = None, 1
        if tp == 1 and m > 128:
            from skyrl_tx_rocm_b200.stack import MLPStack

            row_stack = MLPStack(blocks, num_chunks=args.row_chunks, gemm_variant=args.gemm_variant,
                                 gemm_cta_limit=args.row_chunk_cta_limit)
            row_chunks = row_stack.chunks_for(m)
        # the timed GEMM launches are those of chunk 0 when the rows are cut into chunks
        m_launch = min(m, S.chunk_rows(m, args.tp_chunks)) if (tp > 1 and m > 128) else m
        if row_chunks > 1:
            m_launch = min(m, S.chunk_rows(m, row_chunks))
        gu_ops_launch = 2.0 * m_launch * hidden * 2 * ish
        dn_ops_launch = 2.0 * m_launch * ish * hidden
        gu_bytes_launch = 2 * ish * hidden + m * hidden + 4 * (2 * ish) + 4 * m + 3 * m * 64 * 2 \
            + wl["adapters"] * 2 * ish * wl["rank"] * 2 + m * ish * 2
        dn_bytes_launch = hidden * ish + m * ish + 4 * hidden + 4 * m + 3 * m * 64 * 2 \
            + wl["adapters"] * hidden * wl["rank"] * 2 + 2 * m * hidden * 2
        if m <= 128:
            # small-batch path: the GEMM reads weights + codes and writes the int32 accumulator; the LoRA
            # tables are read by the row kernels, not by the GEMM
            gu_bytes_launch = 2 * ish * hidden + m * hidden + 4 * m * 2 * ish
            dn_bytes_launch = hidden * ish + m * ish + 4 * m * hidden * S._lib.load().skyrl_w8a8_gemm_k_splits(m, hidden, ish, 16)
        # whole job per step: the rows of x once (shared out over the ranks), the adapter ids on every rank
        h2d = x_host.numel() * 2 + (ids_host.numel() * 4 * tp if ids_host is not None else 0)
        d2h = m * hidden * 2
        out_host = torch.empty((m, hidden), dtype=torch.bfloat16).pin_memory()
        if tp > 1 and m > 128:
            # per layer and row chunk: quantiser of h, LoRA-A of h, two GEMMs, finalize, next layer's quantiser and
            # LoRA-A projection of the own rows; one routing launch and one row un-sort per step
            launches_per_step = layers * args.tp_chunks * 7 + 2
            if args.tp_peer_scatter in ("auto", "fused", "fused_copy", "fused_mc") and (tp > 2 or args.tp_peer_scatter != "auto"):
                # fused exchange, per layer and chunk: flag wait, quantiser of h, LoRA-A of h, two GEMMs, flag signal, sum
                # kernel, row quantiser, LoRA-A projection, flag signal (the last layer has no next block: three fewer);
                # per step: routing, the first block's quantiser + LoRA-A per chunk, un-sort
                launches_per_step = layers * args.tp_chunks * 10 - 3 * args.tp_chunks + 2 * args.tp_chunks + 2
        else:
            # per layer: two quantiser launches, two LoRA-A (or LoRA-B row) launches, two GEMMs; one routing launch
            launches_per_step = layers * 6 * row_chunks + 1

        prefetch_bytes = (args.prefetch_mb << 20) if (m <= 128 and tp == 1) else 0

        def step(x_in, ids_in, events=None):
            if tp > 1:
                return tp_stack.forward(x_in, ids_in, timing_events=events)
            if row_stack is not None:
                return row_stack.forward(x_in, ids_in, timing_events=events)
            cur = x_in
            for l, (delta, gu_w, gu_l, dn_w, dn_l) in enumerate(blocks):
                ev = events[l] if events is not None else None
                dst = act[l & 1]
                # adapter ids are the same for every layer of a step: route once, then reuse
                # decode: every GEMM asks the leading bytes of the next GEMM's weights into L2 (the next layer's
                # gate_up behind down; the step's first layer behind the last, for the next step)
                S.w8a8_mlp_block(cur, delta, gu_w, gu_l, dn_w, dn_l, ids_in, enabled=True, out=dst, timing_events=ev,
                                 reuse_routing=l > 0, gemm_variant=args.gemm_variant,
                                 prefetch_next=blocks[(l + 1) % len(blocks)][1] if prefetch_bytes else None,
                                 prefetch_bytes=prefetch_bytes)
                cur = dst
            return cur
    else:
        k, n = wl["k"], wl["n"]
        x_host = torch.randn((m, k), generator=torch.Generator().manual_seed(5), dtype=torch.float32)
        if kind == "down":
            g = torch.randn((m, k), generator=torch.Generator().manual_seed(6), dtype=torch.float32)
            x_host = torch.nn.functional.silu(x_host) * g
        x_host = x_host.to(torch.bfloat16).pin_memory()
        x_dev = x_host.to(device)
        w = synth_weight(S, torch, n, k, 3 if kind == "gate_up" else 4, device, keep_host=want_parity)
        lora = synth_lora(S, torch, wl["adapters"], k, wl["rank"], n, alpha, 9, device, keep_host=want_parity)
        if want_parity:
            (w, w_host), (lora, lora_host) = w, lora
        delta = (torch.randn((k,), generator=gen, device=device) * 0.02).to(torch.bfloat16) if kind == "gate_up" else None
        res_host = torch.randn((m, n), generator=torch.Generator().manual_seed(8), dtype=torch.float32).to(torch.bfloat16).pin_memory() if kind == "down" else None
        res_dev = res_host.to(device) if res_host is not None else None
        out_cols = n // 2 if kind == "gate_up" else n
        out_host = torch.empty((m, out_cols), dtype=torch.bfloat16).pin_memory()
        ops_per_step = 2.0 * m * k * n
        gu_ops_launch = dn_ops_launch = ops_per_step
        gu_bytes_launch = dn_bytes_launch = n * k + m * k + 4 * n + 4 * m + 3 * m * 64 * 2 \
            + wl["adapters"] * n * wl["rank"] * 2 + m * out_cols * 2 + (m * n * 2 if kind == "down" else 0)
        h2d = x_host.numel() * 2 + (ids_host.numel() * 4 if ids_host is not None else 0) + (res_host.numel() * 2 if res_host is not None else 0)
        d2h = m * out_cols * 2
        launches_per_step = 4
        res_holder = [res_dev]

        def step(x_in, ids_in, events=None):
            ev = events[0][:2] if events is not None else None
            if kind == "linear":
                return S.w8a8_lora_linear(x_in, w, lora, adapter_ids=ids_in, enabled=True, timing_events=ev,
                                          gemm_variant=args.gemm_variant)
            if kind == "gate_up":
                return S.w8a8_rms_gate_up_lora_swiglu(x_in, delta, w, lora, adapter_ids=ids_in, enabled=True, timing_events=ev,
                                                      gemm_variant=args.gemm_variant)
            return S.w8a8_down_lora_residual(x_in, w, lora, residual=res_holder[0], adapter_ids=ids_in, enabled=True,
                                             timing_events=ev, gemm_variant=args.gemm_variant)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def make_events():
        evs = []
        for _ in range(layers if kind == "mlp" else 1):
            quad = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            for e in quad:
                e.record()  # creates the underlying CUDA event so its handle can cross the C ABI
            evs.append(quad)
        return evs

    # ---------------- parity of the timed configuration, before anything is timed ----------------
    parity, ok = None, True
    if want_parity:
        parity, ok = parity_check(S, torch, dist, workload, wl, tp, rank, device, x_dev, ids, ids_np, parity_inputs,
                                  locals())
    parity_inputs = None

    # ---------------- warm-up ----------------
    for _ in range(max(args.warmup, 3)):
        step(x_dev, ids)
    barrier()
    S.check_status(device)

    # Launch-bound small-batch steps are replayed from a CUDA graph (one capture of the whole step);
    # the C ABI only enqueues on the current stream, so it is capturable as it stands.
    use_graph = (m <= 128 and tp == 1) if args.graph == "auto" else (args.graph == "on")
    graph = None
    if use_graph:
        graph_out = [None]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(x_dev, ids)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out[0] = step(x_dev, ids)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    # ---------------- timed region: inputs resident in HBM ----------------
    event_steps = min(steps, 20)   # per-kernel events of the first steps only (a decode run has hundreds of steps)
    step_events = [make_events() for _ in range(event_steps)]
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(steps):
        if graph is not None:
            graph.replay()
        else:
            step(x_dev, ids, step_events[i] if i < event_steps else None)
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t_begin.elapsed_time(t_end)
    S.check_status(device)
    if args.gemm_variant & 4 and rank == 0:
        prof = S.ops._status_word(device).tolist()
        print(f"issuer profile of CTA 0 (x1024 cycles, summed over all profiled launches): operands {prof[1]}, "
              f"accumulator {prof[2]}, total {prof[3]}", file=sys.stderr, flush=True)
    if graph is not None:
        # per-kernel durations cannot be read from events inside a graph: take them from an eager pass
        for i in range(event_steps):
            step(x_dev, ids, step_events[i])
        torch.cuda.synchronize()
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / steps
    gu_ms = [q[0].elapsed_time(q[1]) for evs in step_events for q in evs]
    dn_ms = [q[2].elapsed_time(q[3]) for evs in step_events for q in evs] if kind == "mlp" else gu_ms
    gu_avg, dn_avg = sum(gu_ms) / len(gu_ms), sum(dn_ms) / len(dn_ms)

    # ---------------- end to end: host buffers, copies inside the timed region ----------------
    e2e_steps = max(2, min(steps, 5)) if m > 128 else min(steps, 50)

    def e2e_once():
        if graph is not None:
            x_dev.copy_(x_host, non_blocking=True)      # the graph reads these fixed device buffers
            if ids is not None:
                ids.copy_(ids_host, non_blocking=True)
            graph.replay()
            out_host.copy_(graph_out[0], non_blocking=True)
            return
        idd = ids_host.to(device, non_blocking=True) if ids_host is not None else None
        if tp > 1 and m % tp == 0:
            # one job, one host input: every rank uploads its share of the rows and NVLink replicates them
            # (all-gather in place); every rank reads back its share of the result
            r0, r1 = rank * (m // tp), (rank + 1) * (m // tp)
            x_dev[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
            dist.all_gather_into_tensor(x_dev, x_dev[r0:r1])
            out_host[r0:r1].copy_(step(x_dev, idd)[r0:r1], non_blocking=True)
            return
        xd = x_host.to(device, non_blocking=True)
        if kind == "down":
            res_holder[0] = res_host.to(device, non_blocking=True)
        out_host.copy_(step(xd, idd), non_blocking=True)

    # One GPU, eager step: the copies of consecutive steps are pipelined against the compute (upload of step i + 1
    # and download of step i - 1 on streams of their own, double-buffered on both sides).  Every step still uploads
    # its inputs from pinned host memory and downloads its result inside the timed region.
    pipelined = graph is None and tp == 1 and kind != "down"
    pipelined_tp = graph is None and tp > 1 and kind == "mlp" and m % tp == 0
    if pipelined_tp:
        # N GPUs: the same pipeline; every rank uploads its share of the rows and the shares are all-gathered over NVLink
        # on the upload stream (a process group of its own, so that this collective never interleaves with the stack's)
        main_s, up_s, down_s = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        up_group = dist.new_group(list(range(world)))
        r0, r1 = rank * (m // tp), (rank + 1) * (m // tp)
        xbuf = [torch.empty_like(x_dev) for _ in range(2)]
        idbuf = [torch.empty_like(ids) for _ in range(2)] if ids is not None else [None, None]
        ostage = [torch.empty((r1 - r0, hidden), dtype=torch.bfloat16, device=device) for _ in range(2)]
        ohost = [torch.empty((r1 - r0, hidden), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        def e2e_run(n):
            consumed, downloaded = [None, None], [None, None]
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(up_s):
                    if consumed[b] is not None:
                        up_s.wait_event(consumed[b])
                    xbuf[b][r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                    dist.all_gather_into_tensor(xbuf[b], xbuf[b][r0:r1], group=up_group)
                    if ids is not None:
                        idbuf[b].copy_(ids_host, non_blocking=True)
                    uploaded = torch.cuda.Event()
                    uploaded.record(up_s)
                main_s.wait_event(uploaded)
                y = step(xbuf[b], idbuf[b])
                consumed[b] = torch.cuda.Event()
                consumed[b].record(main_s)
                if downloaded[b] is not None:
                    main_s.wait_event(downloaded[b])
                ostage[b].copy_(y[r0:r1])        # the stack's output buffer is reused by the next step
                staged = torch.cuda.Event()
                staged.record(main_s)
                with torch.cuda.stream(down_s):
                    down_s.wait_event(staged)
                    ohost[b].copy_(ostage[b], non_blocking=True)
                    downloaded[b] = torch.cuda.Event()
                    downloaded[b].record(down_s)
            for ev in downloaded:
                if ev is not None:
                    main_s.wait_event(ev)
    elif pipelined:
        main_s, up_s, down_s = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        xbuf = [torch.empty((m, x_host.shape[1]), dtype=torch.bfloat16, device=device) for _ in range(2)]
        idbuf = [torch.empty_like(ids) for _ in range(2)] if ids is not None else [None, None]
        probe = step(x_dev, ids)
        ostage = [torch.empty_like(probe) for _ in range(2)]
        ohost = [torch.empty(probe.shape, dtype=probe.dtype).pin_memory() for _ in range(2)]
        del probe

        def e2e_run(n):
            consumed = [None, None]      # compute of the step that last read xbuf[b] has finished
            downloaded = [None, None]    # download of the step that last wrote ostage[b] has finished
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(up_s):
                    if consumed[b] is not None:
                        up_s.wait_event(consumed[b])
                    xbuf[b].copy_(x_host, non_blocking=True)
                    if ids is not None:
                        idbuf[b].copy_(ids_host, non_blocking=True)
                    uploaded = torch.cuda.Event()
                    uploaded.record(up_s)
                main_s.wait_event(uploaded)
                y = step(xbuf[b], idbuf[b])
                consumed[b] = torch.cuda.Event()
                consumed[b].record(main_s)
                if downloaded[b] is not None:
                    main_s.wait_event(downloaded[b])
                ostage[b].copy_(y)               # the step's output buffer is reused by the next step
                staged = torch.cuda.Event()
                staged.record(main_s)
                with torch.cuda.stream(down_s):
                    down_s.wait_event(staged)
                    ohost[b].copy_(ostage[b], non_blocking=True)
                    downloaded[b] = torch.cuda.Event()
                    downloaded[b].record(down_s)
            for ev in downloaded:
                if ev is not None:
                    main_s.wait_event(ev)        # the timed region ends when the last result is on the host
    else:
        def e2e_run(n):
            for _ in range(n):
                e2e_once()

    e2e_run(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= e2e_steps
    S.check_status(device)

    if rank != 0:
        return None, ok

    tokens_per_s = m / (ms_per_step * 1e-3)
    i8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    if wl["bound"] == "tensor":
        achieved = gu_ops_launch / (gu_avg * 1e-3) / 1e12
        traffic, traffic_note = load_traffic(workload, m_launch if kind == "mlp" else m) if tp == 1 else (None, None)
        roofline = dict(bound="tensor", kernel="w8a8_gemm_kernel<gate_up/SwiGLU epilogue>" if kind in ("mlp", "gate_up") else "w8a8_gemm_kernel",
                        achieved=achieved, peak=i8_peak, unit="TFLOP/s", frac=achieved / i8_peak,
                        traffic=traffic, traffic_unit="bytes per launch" + (f" ({traffic_note})" if traffic_note else ""),
                        algorithmic_bytes=gu_bytes_launch,
                        peak_source=f"2 x bf16_tflops_sustained of {peaks['source']} (no int8 figure is measured; the int8 tcgen05 rate is twice bf16); 1 int8 multiply-add = 2 ops",
                        launch_ms=gu_avg, ops_per_launch=gu_ops_launch,
                        down_gemm=dict(achieved=dn_ops_launch / (dn_avg * 1e-3) / 1e12, launch_ms=dn_avg,
                                       frac=dn_ops_launch / (dn_avg * 1e-3) / 1e12 / i8_peak) if kind == "mlp" else None)
    else:
        achieved = gu_bytes_launch / (gu_avg * 1e-3) / 1e9
        step_bytes = layers * (hidden * 3 * inter + 2 * wl["adapters"] * wl["rank"] * (hidden + 2 * inter + inter + hidden)) if kind == "mlp" else None
        roofline = dict(bound="hbm", kernel="w8a8_gemm_kernel (gate_up weights)", achieved=achieved, peak=peaks["hbm_gbs"],
                        unit="GB/s", frac=achieved / peaks["hbm_gbs"], traffic=None, peak_source=f"hbm_gbs of {peaks['source']}",
                        launch_ms=gu_avg, bytes_per_launch=gu_bytes_launch,
                        step_bytes=step_bytes,
                        step_frac=(step_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"]) if kind == "mlp" else None,
                        down_gemm=dict(achieved=dn_bytes_launch / (dn_avg * 1e-3) / 1e9, launch_ms=dn_avg,
                                       frac=dn_bytes_launch / (dn_avg * 1e-3) / 1e9 / peaks["hbm_gbs"]))
    cpu = None
    if world == 1 and not args.no_cpu_baseline and not sub:
        cpu = cpu_baseline(workload, wl)

    line = {
        "metric": "tokens_per_s_w8a8_lora_mlp", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if kind == "mlp" else "replicas", "vs_baseline": None, "dtype": "int8 x int8 -> int32 (+ bf16 LoRA, fp32 epilogue)",
        "data": "synthetic, seeded; random-init weights of the named shapes (one seeded model, sharded for N > 1)",
        "config": {"workload": workload, "kind": kind, "tokens": m, "layers": layers,
                   **{k_: wl[k_] for k_ in ("hidden", "inter", "k", "n", "rank", "adapters") if k_ in wl},
                   "adapter_ids": wl["ids"], "parallelism": f"tp{tp}", "cuda_graph": graph is not None,
                   **({"tp_chunks": args.tp_chunks, "tp_sequence_parallel": bool(args.tp_sequence_parallel),
                       "tp_peer_scatter": (tp_stack.scatter_mode or "all_reduce") if tp_stack is not None else "off",
                       "tp_reserve_sms": args.tp_reserve_sms} if tp > 1 else {}), "l2": "inputs_exceed_l2" if ops_per_step > 1e11 else "weights_stream_once_per_layer",
                   **({"l2_prefetch_mb": args.prefetch_mb} if (kind == "mlp" and m <= 128 and tp == 1) else {}),
                   **({"row_chunks": row_chunks} if (kind == "mlp" and tp == 1 and m > 128) else {})},
        "int8_tops": ops_per_step / (ms_per_step * 1e-3) / 1e12,
        "int8_tops_frac_of_peak": ops_per_step / (ms_per_step * 1e-3) / 1e12 / (i8_peak * world),
        "e2e": {"value": m / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms,
                "copies": "every step uploads its inputs and downloads its result; consecutive steps' copies overlap the "
                          "compute (double-buffered, streams of their own)" if (pipelined or pipelined_tp) else "in line with the compute"},
        "gpu_launches": launches_per_step * steps,
        "clocks": clocks,
        # time x clock: what a comparison across runs at different SM clocks (a power-capped 1-GPU run against an
        # 8-GPU run at full clock) should divide by
        "ms_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
        "roofline": roofline,
        "parity": parity,
        "cpu_baseline": cpu,
    }
    return line, ok


def parity_check(S, torch, dist, workload, wl, tp, rank, device, x_dev, ids, ids_np, inputs, env):
    """Sampled-row check of the configured workload against the oracle, run before the timed region.
    Returns (dict for the JSON line, ok).  A failed bar is reported in the line, not raised."""
    from oracle import parity_checks as P
    from oracle import w8a8_oracle as O

    kind, m = wl["kind"], wl["m"]
    rows = min(m, 192)   # more than one 128-row tile, so that the sampled rows take the same kernels as the full launch
    try:
        if kind == "mlp" and tp == 1:
            res = P.check_mlp_layer(S, x_dev, inputs["delta"], ids_np, inputs["gate_up"], inputs["down"], rows=rows, seed=1)
            res.update(scope=f"layer 0 of {wl['layers']} at the full launch shape, {res['rows']} sampled token rows, stage by stage")
        elif kind == "mlp":
            # tensor-parallel: block 0 through the same exchange the timed stack uses, against the oracle's statement
            # of the sharded block (per-shard activation scales = group_size I / tp) on sampled rows
            stack = env["make_stack"](env["blocks"][:1])
            out = stack.forward(x_dev, ids)
            torch.cuda.synchronize()
            S.check_status(device)
            res = None
            if rank == 0:
                import numpy as np

                sampled = P.sample_rows(m, rows, 1)
                rt = torch.from_numpy(sampled).to(device)
                gu_host, _, gu_tab, _ = inputs["gate_up"]
                dn_host, _, dn_tab, _ = inputs["down"]
                want = O.tp_shard_mlp_reference(P.to_np(x_dev[rt]), P.to_np(inputs["delta"]), gu_host, *gu_tab, dn_host,
                                                *dn_tab, ids_np[sampled], tp)
                got = P.to_np(out[rt])
                diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
                ulp = O.bf16_ulp_distance(got, want)
                res = {"rows": int(len(sampled)), "rel_l2": O.relative_l2(got, want), "max_abs": float(diff.max()),
                       "max_ulp_ge1": int(ulp[np.abs(want.astype(np.float32)) >= 1.0].max()),
                       "beyond_bar": int(((diff > P.MAX_ABS) & (ulp > 1)).sum()),
                       "exchange": stack.scatter_mode,
                       "scope": f"tp_parity: block 0 through the {tp}-rank exchange against the oracle's sharded block "
                                f"(activation scales per shard, group_size I/{tp}), {len(sampled)} sampled rows"}
                # a composed block: downstream of rounding ties one bf16 step of h can move an int8 code, which the
                # oracle alone amplifies to about 1e-3 (see oracle/parity_checks.py); the bar is relative L2 2e-3
                assert res["rel_l2"] < 2e-3, res
            del stack
        else:
            import numpy as np

            sampled = P.sample_rows(m, rows, 1)
            rt = torch.from_numpy(sampled).to(device)
            got = env["step"](x_dev, ids)
            S.check_status(device)
            ids_r = ids_np[sampled] if ids_np is not None else None
            xin = x_dev[rt].contiguous()
            if kind == "gate_up":
                xin = S.rms_quant(xin, env["delta"], want_normalized=True)[2]
            res = P.check_projection_chain(
                S, workload, P.to_np(xin), env["w_host"], env["w"], env["lora_host"], env["lora"], ids_r, P.to_np(got[rt]),
                {"linear": "linear", "gate_up": "swiglu", "down": "residual"}[kind],
                residual=P.to_np(env["res_dev"][rt]) if kind == "down" else None)
            acc = S.w8a8_int32_accumulator(xin if m <= 128 else (S.rms_quant(x_dev, env["delta"], want_normalized=True)[2]
                                                                  if kind == "gate_up" else x_dev), env["w"], enabled=True)
            codes, _ = O.dynamic_group_quantize(P.to_np(xin), wl["k"])
            want_acc = O.int8_group_gemm(codes, env["w_host"].codes.reshape(1, wl["k"], wl["n"]))[:, 0, :]
            res["acc_bit_exact"] = bool(np.array_equal(P.to_np(acc if m <= 128 else acc[rt]), want_acc))
            res["rows"] = int(len(sampled))
            res["scope"] = f"{res['rows']} sampled token rows of the full launch shape"
            assert res["acc_bit_exact"], "int32 accumulator is not bit-exact"
        ok = True
        if res is not None:
            res["ok"] = True
    except AssertionError as exc:
        res, ok = {"ok": False, "failed": str(exc)[:400]}, False
    if dist is not None:
        flag = torch.tensor([0 if ok else 1], device=device, dtype=torch.int32)
        dist.all_reduce(flag)
        ok = int(flag.item()) == 0
    torch.cuda.empty_cache()
    return res, ok


# --------------------------------------------------------------------------- #
# CPU statement of the reference algorithm (oracle port), bounded sample
# --------------------------------------------------------------------------- #
def cpu_sample(workload: str, wl: dict, rows: int):
    """One layer of the workload on `rows` token rows through the NumPy port; returns seconds."""
    import ml_dtypes
    import numpy as np

    from oracle import w8a8_oracle as O

    bf16 = ml_dtypes.bfloat16
    rng = np.random.default_rng(0)
    na, r = wl["adapters"], wl["rank"]
    ids = rng.integers(0, na, size=rows).astype(np.int32)

    def weight(k, n):
        codes = rng.integers(-127, 128, size=(k, n), dtype=np.int8)
        scales = np.full((1, n), 1e-3, dtype=np.float32).astype(bf16)
        return O.GroupQuantizedWeight(codes, scales, k, k, 8, k)

    def lora(k, n):
        a = (rng.standard_normal((na, k, r)) / np.sqrt(k)).astype(np.float32).astype(bf16)
        b = (rng.standard_normal((na, r, n)) * 0.02).astype(np.float32).astype(bf16)
        return a, b, np.full((na,), 2.0, dtype=np.float32)

    if wl["kind"] == "mlp":
        hidden, inter = wl["hidden"], wl["inter"]
        x = rng.standard_normal((rows, hidden)).astype(np.float32).astype(bf16)
        delta = (rng.standard_normal(hidden) * 0.02).astype(np.float32).astype(bf16)
        wgu, wd = weight(hidden, 2 * inter), weight(inter, hidden)
        ga, gb, gs = lora(hidden, 2 * inter)
        da, db, ds = lora(inter, hidden)
        t0 = time.perf_counter()
        O.mlp_block(x, delta, wgu, ga, gb, gs, wd, da, db, ds, ids)
        return time.perf_counter() - t0
    k, n = wl["k"], wl["n"]
    x = rng.standard_normal((rows, k)).astype(np.float32).astype(bf16)
    w = weight(k, n)
    a, b, s = lora(k, n)
    t0 = time.perf_counter()
    if wl["kind"] == "gate_up":
        O.rms_gate_up_lora_swiglu(x, (rng.standard_normal(k) * 0.02).astype(np.float32).astype(bf16), w, a, b, s, ids)
    elif wl["kind"] == "down":
        O.down_lora_residual(x, w, a, b, s, rng.standard_normal((rows, n)).astype(np.float32).astype(bf16), ids)
    else:
        O.quantized_lora_linear(x, w, a, b, s, ids)
    return time.perf_counter() - t0


CPU_SAMPLE_ROWS = 2048   # token rows of one layer the CPU arms time per sample (about 4.7 s on 16 cores at the c5 shape)


def cpu_baseline(workload: str, wl: dict, rows: int | None = None, reps: int = 2):
    cores = host_threads()
    rows = rows or min(wl["m"], CPU_SAMPLE_ROWS)
    cpu_sample(workload, wl, min(rows, 16))  # warm BLAS threads
    secs = min(cpu_sample(workload, wl, rows) for _ in range(reps))
    per_layer_rows_per_s = rows / secs
    value = per_layer_rows_per_s / wl["layers"]
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{rows} token rows through 1 of {wl['layers']} layers with the NumPy port of the reference's "
                      f"pure-JAX path (int8 contraction through float64 BLAS, exact), {secs:.2f} s; scaled by 1/{wl['layers']} layers",
            "seconds": secs}


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def run_reference(args):
    """The reference's CPU path for the same workload: the NumPy port of its pure-JAX quantised-LoRA functions
    (JAX itself cannot be installed here), on all host threads.  Launchers that start one process per GPU pin
    every process to ONE OpenMP thread (OMP_NUM_THREADS=1); main() lifts that before NumPy is imported, so the
    figure is the same whatever N the arm is launched with."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = dict(WORKLOADS[args.workload])
    rows = min(wl["m"], CPU_SAMPLE_ROWS)
    for _ in range(max(args.warmup, 1)):
        cpu_sample(args.workload, wl, min(rows, 16))
    times = [cpu_sample(args.workload, wl, rows) for _ in range(max(1, min(args.steps, 30)))]
    secs = sum(times) / len(times)
    value = rows / secs / wl["layers"]
    cores = host_threads()
    threads = {k_: os.environ.get(k_) for k_ in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS")}
    sample = (f"{rows} token rows through 1 of {wl['layers']} layers per step, NumPy port of the reference's pure-JAX "
              f"quantised-LoRA path (JAX is not installable here; the int8 contraction runs through float64 BLAS, which is "
              f"exact and faster than the reference's int32 einsum), scaled by 1/{wl['layers']} layers; thread settings {threads}")
    line = {
        "impl": "reference", "metric": "tokens_per_s_w8a8_lora_mlp", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": max(args.warmup, 1), "ms_per_step": secs * 1e3,
        "higher_is_better": True, "scaling": "strong" if wl["kind"] == "mlp" else "replicas", "vs_baseline": None,
        "dtype": "int8 x int8 -> int32 (+ fp32 LoRA)", "data": "synthetic, seeded",
        "config": {"workload": args.workload, "kind": wl["kind"], "tokens": wl["m"], "layers": wl["layers"],
                   **{k_: wl[k_] for k_ in ("hidden", "inter", "k", "n", "rank", "adapters") if k_ in wl},
                   "adapter_ids": wl["ids"], "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--m", type=int, default=0, help="override the token count (debugging)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging / small ncu captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-row oracle check in front of the timed region")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode (c2) sub-benchmark of the default c5 line")
    ap.add_argument("--tp-chunks", type=int, default=2,
                    help="row chunks per block whose exchange overlaps the next chunk's kernels (N > 1).  On 8 GPUs two and "
                         "three chunks measure the same within the box-to-box spread (11.05-11.3 ms per step); two keep the "
                         "host's enqueue time at a third of the step")
    ap.add_argument("--tp-sequence-parallel", type=int, default=1,
                    help="1: ranks own row slices between blocks (reduce-scatter + gather of int8 codes); "
                         "0: one fp32 all-reduce per chunk")
    ap.add_argument("--row-chunks", type=int, default=1,
                    help="one GPU, more than 128 rows: chunks of the sorted rows that run on two streams, so that "
                         "one chunk's quantisers and LoRA-A projections run beside the other chunk's GEMM (1 = off)")
    ap.add_argument("--row-chunk-cta-limit", type=int, default=0,
                    help="with --row-chunks > 1: CTAs a GEMM may use (0 = one per SM); the SMs left over run the other "
                         "stream's LoRA-A projection, which cannot share an SM with a GEMM CTA")
    ap.add_argument("--prefetch-mb", type=int, default=0,
                    help="decode shapes (at most 128 rows, one GPU): MiB of the next GEMM's weights every GEMM asks into L2 "
                         "after its own loads (0 = off, the default: measured slower on B200, 2.62 -> 2.70 ms per c2 step at 48 MiB)")
    ap.add_argument("--tp-reserve-sms", type=int, default=-1,
                    help="SMs the GEMMs leave to the second stream's small kernels while chunks overlap (N > 1): the "
                         "fused exchange kernel (or the one-word all-reduce, finalize / quantise kernels and gathers of the "
                         "other forms); -1 = 8 on two GPUs, 4 on more (the exchange kernels there run on all SMs beside the GEMM)")
    ap.add_argument("--tp-exchange-ctas", type=int, default=0, help="CTAs of the fused exchange kernel (0 = 4 per reserved SM)")
    ap.add_argument("--tp-peer-scatter", default="auto", choices=["auto", "fused", "fused_copy", "fused_mc", "epilogue", "copy", "off"],
                    help="how the fp32 partial sums reach the rank that owns the rows: stores from the down GEMM's "
                         "epilogue into the owner's memory, copy-engine pushes on the second stream, the fused exchange "
                         "kernel (fused: it pulls them over NVLink; fused_copy: the copy engines push them and it adds "
                         "local slabs; no collective between blocks either way), or (off) the NCCL reduce-scatter; "
                         "auto = epilogue on 2 GPUs, fused_copy on more")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="> 0: sets NCCL_MAX_CTAS (tuning aid)")
    ap.add_argument("--gemm-variant", type=int, default=0, choices=[0, 1, 2, 3, 4, 5, 6, 7],
                    help="force a kernel variant of the large GEMMs (0: the library chooses; 1 single tile per CTA, "
                         "2 two M tiles per CTA, 3 CTA pair per 256 x 256 tile); all give the same bits")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: small-batch workloads on one GPU)")
    args = ap.parse_args()
    if args.tp_reserve_sms < 0:
        args.tp_reserve_sms = 8 if args.gpus <= 2 else 4
    if args.impl == "reference":
        # before NumPy loads its BLAS: all host threads, whatever the launcher set for its per-GPU workers
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(host_threads())
        run_reference(args)
    else:
        run_device(args)


if __name__ == "__main__":
    main()
