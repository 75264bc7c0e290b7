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
def synth_weight(S, torch, n, k, seed, device):
    """W ~ N(0, 0.02) bf16 [n, k], per-output-channel absmax int8 (quantized_lora.py:150-171 with group = K)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    wq = torch.empty((n, k), dtype=torch.int8, device=device)
    sw = torch.empty((n,), dtype=torch.float32, device=device)
    rows = max(1, (64 << 20) // k)
    for r0 in range(0, n, rows):
        r1 = min(n, r0 + rows)
        w = (torch.randn((r1 - r0, k), generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16).float()
        amax = w.abs().amax(dim=1)
        scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
        wq[r0:r1] = torch.clamp(torch.round(w / scale[:, None]), -127, 127).to(torch.int8)
        sw[r0:r1] = scale.to(torch.bfloat16).float()
    return S.pack_weight_nk(wq, sw)


def synth_lora(S, torch, adapters, k, rank, n, alpha, seed, device, seed_b=None):
    """`seed_b` seeds B separately: a tensor-parallel rank shares the replicated half of a LoRA pair with the
    other ranks (A of gate_up, B of down) and draws only its shard of the other half from its own seed."""
    gen = torch.Generator(device=device).manual_seed(seed)
    a = (torch.randn((adapters, k, rank), generator=gen, device=device) / (k ** 0.5)).to(torch.bfloat16)
    if seed_b is not None:
        gen = torch.Generator(device=device).manual_seed(seed_b)
    b = (torch.randn((adapters, rank, n), generator=gen, device=device) * 0.02).to(torch.bfloat16)
    s = torch.full((adapters,), alpha / rank, dtype=torch.float32, device=device)
    return S.pack_lora(a, b, s, in_features=k, padded_out_features=n)


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
def run_device(args):
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
        if args.nccl_max_ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.nccl_max_ctas))
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            del os.environ["NCCL_DEBUG"]  # its banner goes to stdout; this program prints exactly one JSON line
        dist.init_process_group("nccl", device_id=device)

    import skyrl_tx_rocm_b200 as S

    wl = dict(WORKLOADS[args.workload])
    if args.m:
        wl["m"] = args.m
    if args.layers:
        wl["layers"] = args.layers
    kind, m, layers = wl["kind"], wl["m"], wl["layers"]
    tp = world
    if tp > 1 and kind != "mlp":
        raise SystemExit("tensor parallelism is benchmarked on the MLP workloads (c5, c2)")
    peaks = load_peaks()
    alpha = 2.0 * wl["rank"]

    # ---------------- build the workload ----------------
    ids_host = synth_ids(torch, m, wl["adapters"], wl["ids"], 7)
    ids = ids_host.to(device) if ids_host is not None else None
    gen = torch.Generator(device=device).manual_seed(11)
    if kind == "mlp":
        hidden, inter = wl["hidden"], wl["inter"]
        if inter % tp or (inter // tp) % 16:
            raise SystemExit("intermediate size must split into multiples of 16 per rank")
        ish = inter // tp
        x_host = torch.randn((m, hidden), generator=torch.Generator().manual_seed(5), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        blocks = []
        for l in range(layers):
            seed = (5000 if args.workload == "c5" else 1000) + l
            delta = (torch.randn((hidden,), generator=gen, device=device) * 0.02).to(torch.bfloat16)
            gu_w = synth_weight(S, torch, 2 * ish, hidden, seed * 131 + rank * 7 + 1, device)
            dn_w = synth_weight(S, torch, hidden, ish, seed * 131 + rank * 7 + 2, device)
            gu_l = synth_lora(S, torch, wl["adapters"], hidden, wl["rank"], 2 * ish, alpha, seed * 131 + 3, device,
                              seed_b=seed * 131 + rank * 7 + 3)
            dn_l = synth_lora(S, torch, wl["adapters"], ish, wl["rank"], hidden, alpha, seed * 131 + rank * 7 + 4, device,
                              seed_b=seed * 131 + 4)
            blocks.append((delta, gu_w, gu_l, dn_w, dn_l))
        tp_stack = None
        if tp > 1:
            from skyrl_tx_rocm_b200.tp import TensorParallelMLP, TensorParallelMLPStack

            tp_stack = TensorParallelMLPStack([TensorParallelMLP(*b) for b in blocks], num_chunks=args.tp_chunks,
                                              reserve_sms=args.tp_reserve_sms,
                                              sequence_parallel=bool(args.tp_sequence_parallel),
                                              peer_scatter=False if args.tp_peer_scatter == "off" else args.tp_peer_scatter)
        x_dev = x_host.to(device)
        act = [torch.empty((m, hidden), dtype=torch.bfloat16, device=device) for _ in range(2)]
        ops_per_step = 2.0 * m * (hidden * 2 * inter + inter * hidden) * layers  # whole job, all ranks
        # the timed GEMM launches are those of chunk 0 when the tensor-parallel stack cuts the rows into chunks
        m_launch = min(m, S.chunk_rows(m, args.tp_chunks)) if (tp > 1 and m > 128) else m
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
        # per layer: 2 quantiser, 2 LoRA-A / LoRA-B-rows, 2 GEMM launches (+ finalize under TP); one routing launch per step
        if tp > 1 and m > 128:
            # per layer and row chunk: quantiser of h, LoRA-A of h, two GEMMs, finalize, next layer's quantiser and
            # LoRA-A projection of the own rows; one routing launch and one row un-sort per step
            launches_per_step = layers * args.tp_chunks * 7 + 2
        else:
            launches_per_step = layers * 6 + 1

        def step(x_in, ids_in, events=None):
            if tp > 1:
                return tp_stack.forward(x_in, ids_in, timing_events=events)
            cur = x_in
            for l, (delta, gu_w, gu_l, dn_w, dn_l) in enumerate(blocks):
                ev = events[l] if events is not None else None
                dst = act[l & 1]
                # adapter ids are the same for every layer of a step: route once, then reuse
                S.w8a8_mlp_block(cur, delta, gu_w, gu_l, dn_w, dn_l, ids_in, enabled=True, out=dst, timing_events=ev,
                                 reuse_routing=l > 0)
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
        w = synth_weight(S, torch, n, k, 3 if kind == "gate_up" else 4, device)
        lora = synth_lora(S, torch, wl["adapters"], k, wl["rank"], n, alpha, 9, device)
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
                return S.w8a8_lora_linear(x_in, w, lora, adapter_ids=ids_in, enabled=True, timing_events=ev)
            if kind == "gate_up":
                return S.w8a8_rms_gate_up_lora_swiglu(x_in, delta, w, lora, adapter_ids=ids_in, enabled=True, timing_events=ev)
            return S.w8a8_down_lora_residual(x_in, w, lora, residual=res_holder[0], adapter_ids=ids_in, enabled=True,
                                             timing_events=ev)

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
    step_events = [make_events() for _ in range(args.steps)]
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step(x_dev, ids, step_events[i])
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = t_begin.elapsed_time(t_end)
    S.check_status(device)
    if graph is not None:
        # per-kernel durations cannot be read from events inside a graph: take them from an eager pass
        for i in range(args.steps):
            step(x_dev, ids, step_events[i])
        torch.cuda.synchronize()
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    gu_ms = [q[0].elapsed_time(q[1]) for evs in step_events for q in evs]
    dn_ms = [q[2].elapsed_time(q[3]) for evs in step_events for q in evs] if kind == "mlp" else gu_ms
    gu_avg, dn_avg = sum(gu_ms) / len(gu_ms), sum(dn_ms) / len(dn_ms)

    # ---------------- end to end: host buffers, copies inside the timed region ----------------
    e2e_steps = max(2, min(args.steps, 5))

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

    for _ in range(2):
        e2e_once()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_once()
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
        if dist is not None:
            dist.destroy_process_group()
        return

    tokens_per_s = m / (ms_per_step * 1e-3)
    i8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    if wl["bound"] == "tensor":
        achieved = gu_ops_launch / (gu_avg * 1e-3) / 1e12
        roofline = dict(bound="tensor", kernel="w8a8_gemm_kernel<gate_up/SwiGLU epilogue>" if kind in ("mlp", "gate_up") else "w8a8_gemm_kernel",
                        achieved=achieved, peak=i8_peak, unit="TFLOP/s", frac=achieved / i8_peak,
                        # DRAM bytes of one gate_up launch: ncu capture at M = 4096 (660.5 MB read + 195.9 MB written,
                        # profiles/w8a8_gemm_c5_layer_m4096.md) scaled by the rows, which every term grows with
                        traffic=(856.3e6 * m / 4096 if (args.workload == "c5" and tp == 1) else None),
                        traffic_unit="bytes per launch (ncu at M=4096, scaled by M)",
                        peak_source=f"2 x bf16_tflops_sustained of {peaks['source']} (int8 tcgen05 rate is twice bf16); 1 int8 multiply-add = 2 ops",
                        launch_ms=gu_avg, ops_per_launch=gu_ops_launch,
                        down_gemm=dict(achieved=dn_ops_launch / (dn_avg * 1e-3) / 1e12, launch_ms=dn_avg,
                                       frac=dn_ops_launch / (dn_avg * 1e-3) / 1e12 / i8_peak) if kind == "mlp" else None)
    else:
        achieved = gu_bytes_launch / (gu_avg * 1e-3) / 1e9
        roofline = dict(bound="hbm", kernel="w8a8_gemm_kernel<int32 epilogue> (gate_up weights)", achieved=achieved, peak=peaks["hbm_gbs"],
                        unit="GB/s", frac=achieved / peaks["hbm_gbs"], traffic=None, peak_source=f"hbm_gbs of {peaks['source']}",
                        launch_ms=gu_avg, bytes_per_launch=gu_bytes_launch,
                        step_bytes=layers * (hidden * 3 * inter + 2 * wl["adapters"] * wl["rank"] * (hidden + 2 * inter + inter + hidden)) if kind == "mlp" else None,
                        step_frac=(layers * (hidden * 3 * inter + 2 * wl["adapters"] * wl["rank"] * (hidden + 2 * inter + inter + hidden)) / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"]) if kind == "mlp" else None,
                        down_gemm=dict(achieved=dn_bytes_launch / (dn_avg * 1e-3) / 1e9, launch_ms=dn_avg,
                                       frac=dn_bytes_launch / (dn_avg * 1e-3) / 1e9 / peaks["hbm_gbs"]))
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args.workload, wl)

    line = {
        "metric": "tokens_per_s_w8a8_lora_mlp", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if kind == "mlp" else "replicas", "vs_baseline": None, "dtype": "int8 x int8 -> int32 (+ bf16 LoRA, fp32 epilogue)",
        "data": "synthetic, seeded; random-init weights of the named shapes",
        "config": {"workload": args.workload, "kind": kind, "tokens": m, "layers": layers,
                   **{k_: wl[k_] for k_ in ("hidden", "inter", "k", "n", "rank", "adapters") if k_ in wl},
                   "adapter_ids": wl["ids"], "parallelism": f"tp{tp}", "cuda_graph": graph is not None,
                   **({"tp_chunks": args.tp_chunks, "tp_sequence_parallel": bool(args.tp_sequence_parallel),
                       "tp_peer_scatter": (tp_stack.scatter_mode or "all_reduce") if tp_stack is not None else "off",
                       "tp_reserve_sms": args.tp_reserve_sms} if tp > 1 else {}), "l2": "inputs_exceed_l2" if ops_per_step > 1e11 else "weights_stream_once_per_layer"},
        "int8_tops": ops_per_step / (ms_per_step * 1e-3) / 1e12,
        "int8_tops_frac_of_peak": ops_per_step / (ms_per_step * 1e-3) / 1e12 / (i8_peak * world),
        "e2e": {"value": m / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


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


def cpu_baseline(workload: str, wl: dict, rows: int | None = None, reps: int = 2):
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    rows = rows or min(wl["m"], 256)
    cpu_sample(workload, wl, min(rows, 16))  # warm BLAS threads
    secs = min(cpu_sample(workload, wl, rows) for _ in range(reps))
    per_layer_rows_per_s = rows / secs
    value = per_layer_rows_per_s / wl["layers"]
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{rows} token rows through 1 of {wl['layers']} layers with the NumPy port of the reference's "
                      f"pure-JAX path (int8 contraction through float64 BLAS, exact), {secs:.2f} s; scaled by 1/{wl['layers']} layers",
            "seconds": secs}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = dict(WORKLOADS[args.workload])
    rows = min(wl["m"], 256)
    for _ in range(max(args.warmup, 1)):
        cpu_sample(args.workload, wl, min(rows, 16))
    times = [cpu_sample(args.workload, wl, rows) for _ in range(max(1, min(args.steps, 3)))]
    secs = sum(times) / len(times)
    value = rows / secs / wl["layers"]
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    sample = (f"{rows} token rows through 1 of {wl['layers']} layers per step, NumPy port of the reference's pure-JAX "
              f"quantised-LoRA path (JAX is not installable here), scaled by 1/{wl['layers']} layers")
    line = {
        "impl": "reference", "metric": "tokens_per_s_w8a8_lora_mlp", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": max(args.warmup, 1), "ms_per_step": secs * 1e3,
        "higher_is_better": True, "scaling": "strong" if wl["kind"] == "mlp" else "replicas", "vs_baseline": None,
        "dtype": "int8 x int8 -> int32 (+ fp32 LoRA)", "data": "synthetic, seeded",
        "config": {"workload": args.workload, "kind": wl["kind"], "tokens": wl["m"], "layers": wl["layers"],
                   "parallelism": "cpu"},
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
    ap.add_argument("--tp-chunks", type=int, default=2,
                    help="row chunks per block whose all-reduce overlaps the next chunk's kernels (N > 1)")
    ap.add_argument("--tp-sequence-parallel", type=int, default=1,
                    help="1: ranks own row slices between blocks (reduce-scatter + gather of int8 codes); "
                         "0: one fp32 all-reduce per chunk")
    ap.add_argument("--tp-reserve-sms", type=int, default=8,
                    help="SMs the GEMMs leave to the second stream's small kernels while chunks overlap (N > 1): the "
                         "one-word all-reduce, the finalize / quantise kernels of the rank's own rows, the gathers")
    ap.add_argument("--tp-peer-scatter", default="auto", choices=["auto", "epilogue", "copy", "off"],
                    help="how the fp32 partial sums reach the rank that owns the rows: stores from the down GEMM's "
                         "epilogue into the owner's memory, copy-engine pushes on the second stream, or (off) the "
                         "NCCL reduce-scatter; auto = epilogue on 2 GPUs, copy on more")
    ap.add_argument("--nccl-max-ctas", type=int, default=0, help="> 0: sets NCCL_MAX_CTAS (tuning aid)")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: small-batch workloads on one GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_device(args)


if __name__ == "__main__":
    main()
