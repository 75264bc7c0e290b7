"""Tensor-parallel sharding math on CPU: two gloo ranks, each evaluating its
shard with the oracle, summed by an all-reduce, against the unsharded statement.

The sharding is the reference's (gate_up on output features, down on input
features: skyrl/tx/models/qwen3_5.py:633,644), the reduction its GSPMD
all-reduce.  The reference tests the same thing on two CPU devices of a JAX
mesh (tests/tx/models/test_qwen3_5.py:110-133)."""

import os
import socket

import ml_dtypes
import numpy as np
import pytest

torch = pytest.importorskip("torch")

BF16 = ml_dtypes.bfloat16


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    from oracle import w8a8_oracle as O

    rng = np.random.default_rng(21)
    m, hidden, inter, r, na = 24, 64, 128, 8, 3
    x = rng.standard_normal((m, hidden)).astype(np.float32).astype(BF16)
    delta = (rng.standard_normal(hidden) * 0.02).astype(np.float32).astype(BF16)
    wgu = O.quantize_frozen_weight((rng.standard_normal((hidden, 2 * inter)) * 0.05).astype(np.float32).astype(BF16), group_size=hidden)
    wd_dense = (rng.standard_normal((inter, hidden)) * 0.05).astype(np.float32).astype(BF16)
    gu_a = (rng.standard_normal((na, hidden, r)) / 8).astype(np.float32).astype(BF16)
    gu_b = (rng.standard_normal((na, r, 2 * inter)) * 0.05).astype(np.float32).astype(BF16)
    dn_a = (rng.standard_normal((na, inter, r)) / 11).astype(np.float32).astype(BF16)
    dn_b = (rng.standard_normal((na, r, hidden)) * 0.05).astype(np.float32).astype(BF16)
    s = np.asarray([2.0, 1.0, 0.5], dtype=np.float32)
    ids = rng.integers(0, na, size=m).astype(np.int32)
    return x, delta, wgu, wd_dense, gu_a, gu_b, dn_a, dn_b, s, ids


def _rank_main(rank, world, port, result_path):
    import torch.distributed as dist

    from oracle import w8a8_oracle as O
    from skyrl_tx_rocm_b200 import tp as T

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, delta, wgu, wd_dense, gu_a, gu_b, dn_a, dn_b, s, ids = _problem()
    inter = wd_dense.shape[0]
    # front half on this rank's column shard (pairs stay together)
    codes, scales, gb = T.shard_gate_up(wgu.codes, wgu.scales, gu_b, world, rank)
    w_shard = O.GroupQuantizedWeight(np.ascontiguousarray(codes), np.ascontiguousarray(scales), wgu.original_in_features,
                                     wgu.padded_in_features, 8, wgu.group_size)
    h_p = O.rms_gate_up_lora_swiglu(x, delta, w_shard, gu_a, np.ascontiguousarray(gb), s, ids)
    lo, hi = T.shard_bounds(inter, world, rank)
    assert h_p.shape == (x.shape[0], hi - lo)
    # back half: row shard, own per-token scale, fp32 partial sums
    wd_p = O.quantize_frozen_weight(wd_dense[lo:hi], group_size=hi - lo)
    _, da_p = T.shard_down(wd_dense, dn_a, world, rank)
    part = O.quantized_frozen_linear_f32(h_p, wd_p) + O.low_rank_f32(h_p, np.ascontiguousarray(da_p), dn_b, s, ids)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    out = O.residual_add(t.numpy().astype(BF16), x)
    if rank == 0:
        np.save(result_path, out.view(np.uint16))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_block_matches_group_format(tmp_path):
    import torch.multiprocessing as mp

    from oracle import w8a8_oracle as O

    result = str(tmp_path / "tp_out.npy")
    mp.spawn(_rank_main, args=(2, _free_port(), result), nprocs=2, join=True)
    got = np.load(result).view(BF16)
    x, delta, wgu, wd_dense, gu_a, gu_b, dn_a, dn_b, s, ids = _problem()
    want = O.tp_shard_mlp_reference(x, delta, wgu, gu_a, gu_b, s, wd_dense, dn_a, dn_b, s, ids, 2)
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    # and equal (up to fp32 association of the LoRA partial sums) to the reference's own
    # group format evaluated unsharded with group_size = I / tp
    grouped = O.mlp_block(x, delta, wgu, gu_a, gu_b, s, O.quantize_frozen_weight(wd_dense, group_size=64), dn_a, dn_b, s, ids)
    assert O.bf16_ulp_distance(got, grouped).max() <= 1


def test_shard_helpers():
    from skyrl_tx_rocm_b200 import tp as T

    assert T.shard_bounds(128, 4, 3) == (96, 128)
    with pytest.raises(ValueError):
        T.shard_bounds(100, 3, 0)
    codes = np.arange(4 * 16).reshape(4, 16)
    c, sc, b = T.shard_gate_up(codes, codes[:1], np.zeros((2, 3, 16)), 2, 1)
    # rank 1 of 2 owns pairs 4..7 = physical columns 8..15 (gate and up of each pair together)
    np.testing.assert_array_equal(c, codes[:, 8:16])
    assert sc.shape == (1, 8) and b.shape == (2, 3, 8)


def _exchange_rank(rank, world, port, result_path):
    """The sequence-parallel exchange with NumPy rows instead of kernels: every rank holds fp32 partial sums of
    all rows, pushes each owner's runs into the owner's [source rank, own rows] slab, the
    owner adds the slabs in rank order, and the owned runs are gathered back into sorted order."""
    import torch.distributed as dist

    from skyrl_tx_rocm_b200 import tp as T

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, hidden, chunks = 1280, 8, 3
    plans = [T.exchange_plan(m, chunks, world, r) for r in range(world)]
    me = plans[rank]
    assert me["even"] and me["own_rows"] == m // world
    part = torch.from_numpy(np.random.default_rng(100 + rank).standard_normal((m, hidden)).astype(np.float32))
    # what this rank sends to owner o: o's runs of every chunk, laid out as o stores them (chunk after chunk)
    send = []
    for o in range(world):
        buf = torch.empty((me["own_rows"], hidden))
        for (r0, cnt), off in zip(plans[o]["own"], plans[o]["own_off"]):
            buf[off:off + cnt] = part[r0:r0 + cnt]
        send.append(buf)
    # the pushes: gloo has no all_to_all, so every rank publishes all it sends and an owner picks its part
    outbox = torch.stack(send)
    boxes = [torch.empty_like(outbox) for _ in range(world)]
    dist.all_gather(boxes, outbox)
    slabs = [boxes[src][rank] for src in range(world)]                      # [source rank] of this owner
    total = slabs[0].clone()
    for s in range(1, world):
        total += slabs[s]                                                   # ascending rank order
    gathered = [torch.empty_like(total) for _ in range(world)]
    dist.all_gather(gathered, total)
    full = torch.empty((m, hidden))
    for o in range(world):
        for (r0, cnt), off in zip(plans[o]["own"], plans[o]["own_off"]):
            full[r0:r0 + cnt] = gathered[o][off:off + cnt]
    if rank == 0:
        np.save(result_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_parallel_exchange_bookkeeping(tmp_path):
    import torch.multiprocessing as mp

    from skyrl_tx_rocm_b200 import tp as T

    result = str(tmp_path / "exchange.npy")
    mp.spawn(_exchange_rank, args=(2, _free_port(), result), nprocs=2, join=True)
    got = np.load(result)
    want = sum(np.random.default_rng(100 + r).standard_normal((1280, 8)).astype(np.float32) for r in range(2))
    np.testing.assert_array_equal(got, want)

    plan = T.exchange_plan(16384, 2, 8, 3)
    assert plan["spans"] == [(0, 8192), (8192, 8192)] and plan["own"] == [(3072, 1024), (11264, 1024)]
    assert plan["own_off"] == [0, 1024] and plan["own_rows"] == 2048 and plan["even"]
    assert not T.exchange_plan(1001, 2, 8, 0)["even"]          # 512 + 489 rows: the second chunk does not divide
    runs = sorted(r for k in range(4) for r in T.exchange_plan(1280, 3, 4, k)["own"])
    assert runs[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(runs, runs[1:])) and sum(r[1] for r in runs) == 1280
