"""Host logic of the model wiring and of the weight pipeline (no GPU): which kernel path the MLP module
selects for which call, in the style of the reference's selector tests (tests/tx/models/test_qwen3_5.py:350-448:
spies on the fused entry points, fallbacks when a geometry is not qualified), and the pack / unpack / cache
round trips of the weight format."""

import numpy as np
import pytest
import torch

import skyrl_tx_rocm_b200 as S
from skyrl_tx_rocm_b200 import mlp as M
from skyrl_tx_rocm_b200 import ops
from skyrl_tx_rocm_b200 import weights as W


def fake_weights(hidden=64, inter=96):
    gu = S.PackedW8Weight(torch.zeros((1, 2 * inter, 128), dtype=torch.int8), torch.ones(2 * inter), hidden, 2 * inter)
    dn = S.PackedW8Weight(torch.zeros((1, hidden, 128), dtype=torch.int8), torch.ones(hidden), inter, hidden)
    return W.PackedMLPWeights(gu, dn)


def fake_lora(k, n, rank=8, na=3):
    return S.PackedLoRA(torch.zeros((na, 64, k), dtype=torch.bfloat16), torch.zeros((na, n, 64), dtype=torch.bfloat16),
                        torch.ones(na), rank, na)


@pytest.fixture
def spies(monkeypatch):
    calls = []
    monkeypatch.setattr(M, "_is_device_tensor", lambda t: isinstance(t, torch.Tensor))

    def block(x, delta, gu, gul, dn, dnl, ids=None, *, residual=None, enabled=False, eps=1e-6):
        calls.append(("w8a8_mlp_block", delta is not None, ids, eps))
        return torch.zeros_like(x)

    def gate_up(x, delta, w, lora, lora_b=None, scaling=None, adapter_ids=None, *, enabled=False, eps=1e-6):
        calls.append(("w8a8_rms_gate_up_lora_swiglu", delta is not None, adapter_ids))
        return torch.zeros((*x.shape[:-1], w.out_features // 2), dtype=torch.bfloat16)

    def down(x, w, lora, lora_b=None, scaling=None, residual=None, adapter_ids=None, *, enabled=False):
        calls.append(("w8a8_down_lora_residual", residual is not None, adapter_ids))
        return torch.zeros((*x.shape[:-1], w.out_features), dtype=torch.bfloat16)

    def rms_quant(x, delta=None, *, eps=1e-6, row_map=None, want_normalized=False):
        calls.append(("rms_quant",))
        return None, None, x.clone()

    monkeypatch.setattr(ops, "w8a8_mlp_block", block)
    monkeypatch.setattr(ops, "w8a8_rms_gate_up_lora_swiglu", gate_up)
    monkeypatch.setattr(ops, "w8a8_down_lora_residual", down)
    monkeypatch.setattr(ops, "rms_quant", rms_quant)
    return calls


def make_module(**cfg):
    config = M.W8A8BackendConfig(w8a8_mlp=True, max_lora_adapters=3, max_lora_rank=8, **cfg)
    w = fake_weights()
    return M.Qwen3_5MLP(config, w, fake_lora(64, 192), fake_lora(96, 64))


def test_whole_block_is_selected_for_the_qualified_call(spies):
    mlp = make_module()
    x = torch.zeros((2, 5, 64), dtype=torch.bfloat16)
    norm = M.RMSNormWeights(torch.zeros(64, dtype=torch.bfloat16))
    ids = torch.tensor([2, 0], dtype=torch.int32)
    out = mlp.forward_with_post_attention_rms(x, norm, ids, residual=x)
    assert out.shape == x.shape and mlp.last_path == "w8a8_mlp_block"
    assert [c[0] for c in spies] == ["w8a8_mlp_block"]
    # per-sequence adapter ids are repeated over the sequence
    np.testing.assert_array_equal(spies[0][2].numpy(), [2] * 5 + [0] * 5)


def test_missing_residual_falls_back_to_the_two_fused_halves(spies):
    mlp = make_module()
    x = torch.zeros((1, 4, 64), dtype=torch.bfloat16)
    norm = M.RMSNormWeights(torch.zeros(64, dtype=torch.bfloat16))
    mlp.forward_with_post_attention_rms(x, norm, torch.zeros(1, dtype=torch.int32), residual=None)
    assert [c[0] for c in spies] == ["w8a8_rms_gate_up_lora_swiglu", "w8a8_down_lora_residual"]
    assert spies[0][1] is True and spies[1][1] is False        # norm fused in front, no residual behind
    assert mlp.last_path == "w8a8_rms_gate_up_swiglu+down"


def test_unqualified_norm_weight_falls_back_to_the_unfused_norm(spies):
    mlp = make_module()
    x = torch.zeros((1, 4, 64), dtype=torch.bfloat16)
    norm = M.RMSNormWeights(torch.zeros(64, dtype=torch.float32))      # fp32 norm weight: not qualified
    mlp.forward_with_post_attention_rms(x, norm, torch.zeros(1, dtype=torch.int32), residual=x)
    assert [c[0] for c in spies] == ["rms_quant", "w8a8_mlp_block"]
    assert spies[1][1] is False and mlp.last_path == "w8a8_mlp_block(no norm)"


def test_wrong_eps_falls_back(spies):
    mlp = make_module()
    x = torch.zeros((1, 4, 64), dtype=torch.bfloat16)
    norm = M.RMSNormWeights(torch.zeros(64, dtype=torch.bfloat16), eps=1e-5)
    mlp.forward_with_post_attention_rms(x, norm, torch.zeros(1, dtype=torch.int32), residual=x)
    assert [c[0] for c in spies][0] == "w8a8_rms_gate_up_lora_swiglu"


def test_call_on_normalised_input(spies):
    mlp = make_module()
    x = torch.zeros((3, 64), dtype=torch.bfloat16)
    mlp(x, torch.zeros(3, dtype=torch.int32), residual=x)
    assert [c[0] for c in spies] == ["w8a8_mlp_block"] and spies[0][1] is False
    spies.clear()
    qwen3 = M.Qwen3MLP(mlp.config, mlp.weights, mlp.gate_up_lora, mlp.down_lora)
    qwen3(x, torch.zeros(3, dtype=torch.int32))
    assert [c[0] for c in spies] == ["w8a8_rms_gate_up_lora_swiglu", "w8a8_down_lora_residual"]


def test_disabled_flag_and_config_validation(spies):
    w = fake_weights()
    off = M.Qwen3_5MLP(M.W8A8BackendConfig(max_lora_adapters=3), w, fake_lora(64, 192), fake_lora(96, 64))
    with pytest.raises(RuntimeError, match="disabled by default"):
        off(torch.zeros((3, 64), dtype=torch.bfloat16))
    assert spies == []
    with pytest.raises(TypeError, match="exact bool"):
        M.W8A8BackendConfig(w8a8_mlp=1)
    with pytest.raises(ValueError, match="ranks up to 64"):
        M.W8A8BackendConfig(w8a8_mlp=True, max_lora_rank=128)
    with pytest.raises(ValueError, match="tensor-parallel"):
        M.W8A8BackendConfig(w8a8_mlp=True, tensor_parallel_size=16)
    with pytest.raises(ValueError, match="exceeds max_lora_rank"):
        M.Qwen3_5MLP(M.W8A8BackendConfig(w8a8_mlp=True, max_lora_rank=4, max_lora_adapters=3), w, fake_lora(64, 192),
                     fake_lora(96, 64))
    with pytest.raises(ValueError, match="adapter_indices"):
        make_module()(torch.zeros((2, 5, 64), dtype=torch.bfloat16), torch.zeros(3, dtype=torch.int32), residual=None)


# ----------------------------------------------------------------------------- weight pipeline
def test_fuse_gate_up_matches_the_interleave_contract():
    rng = np.random.default_rng(0)
    gate, up = torch.from_numpy(rng.standard_normal((8, 5))), torch.from_numpy(rng.standard_normal((8, 5)))
    fused = W.fuse_gate_up(gate, up)
    assert fused.shape == (8, 10)
    assert torch.equal(fused[:, 0::2], gate) and torch.equal(fused[:, 1::2], up)
    g2, u2 = W.split_gate_up(fused)
    assert torch.equal(g2, gate) and torch.equal(u2, up)


@pytest.mark.parametrize("k,n", [(128, 32), (200, 64), (16, 96), (384, 160)])
def test_pack_unpack_is_the_identity(k, n):
    rng = np.random.default_rng(k + n)
    codes = torch.from_numpy(rng.integers(-127, 128, size=(k, n), dtype=np.int8))
    scales = torch.from_numpy(rng.random((1, n)).astype(np.float32)).to(torch.bfloat16)
    packed = S.PackedW8Weight(W.pack_weight_host(codes), scales[0].float(), k, n)
    assert packed.wq.shape == ((k + 127) // 128, n, 128)
    # layout: wq[kb, n, kk] = codes[kb * 128 + kk, n], zero beyond K
    kb, kk, col = (k - 1) // 128, (k - 1) % 128, n // 2
    assert packed.wq[kb, col, kk] == codes[k - 1, col]
    if k % 128:
        assert int(packed.wq[kb, :, k % 128:].abs().max()) == 0
    back = W.unpack_weight(packed)
    assert torch.equal(back.codes, codes) and torch.equal(back.scales.view(torch.int16), scales.view(torch.int16))
    again = W.pack_weight_host(back.codes)
    assert torch.equal(again, packed.wq)


def test_packed_weight_file_round_trip_and_disk_cache(tmp_path):
    rng = np.random.default_rng(1)
    codes = torch.from_numpy(rng.integers(-127, 128, size=(256, 64), dtype=np.int8))
    scales = torch.from_numpy(rng.random((1, 64)).astype(np.float32)).to(torch.bfloat16)
    packed = S.PackedW8Weight(W.pack_weight_host(codes), scales[0].float(), 256, 64)
    path = tmp_path / "w.w8pack"
    W.save_packed_weight(path, packed)
    loaded = W.load_packed_weight(path)
    assert torch.equal(loaded.wq, packed.wq) and torch.equal(loaded.sw, packed.sw)
    assert (loaded.in_features, loaded.out_features, loaded.group_size) == (256, 64, 0)
    cache = W.PackedWeightCache(tmp_path / "cache")
    built = []
    key = W.tensor_digest(codes, scales)
    for _ in range(3):
        got = cache.get_or_build(key, lambda: built.append(1) or packed)
        assert torch.equal(got.wq, packed.wq)
    assert len(built) == 1 and cache.hits == 2 and cache.misses == 1
    assert W.tensor_digest(codes, scales) != W.tensor_digest(codes + 1, scales)


def test_identity_cache_converts_once_per_tensor_version():
    cache = W.IdentityCache(capacity=4)
    a, b = torch.zeros(4), torch.ones(4)
    built = []
    make = lambda: built.append(1) or object()
    first = cache.get((a, b), "x", make)
    assert cache.get((a, b), "x", make) is first and len(built) == 1
    a.add_(1)                                  # an in-place update (an optimizer step) is a new version
    assert cache.get((a, b), "x", make) is not first and len(built) == 2
    assert cache.get((a, b), "y", make) is not first and len(built) == 3
    c = torch.zeros(4)
    cache.get((c,), None, make)
    del c                                      # entries die with their source
    cache.get((a,), None, make)
    assert all(all(r() is not None for r in refs) for refs, _ in cache._items.values())


# ----------------------------------------------------------------------------- other projections, W4
def test_fuse_and_split_components_follow_the_group_interleave():
    from skyrl_tx_rocm_b200 import projections as P

    rng = np.random.default_rng(3)
    q, k, v = (torch.from_numpy(rng.standard_normal((5, n))) for n in (24, 6, 6))    # 3 kv groups: 8 + 2 + 2 each
    fused = P.fuse_components((q, k, v), (8, 2, 2))
    assert fused.shape == (5, 36)
    assert torch.equal(fused[:, :8], q[:, :8]) and torch.equal(fused[:, 8:10], k[:, :2]) and torch.equal(fused[:, 10:12], v[:, :2])
    assert torch.equal(fused[:, 12:20], q[:, 8:16])
    q2, k2, v2 = P.split_components(fused, (8, 2, 2))
    assert torch.equal(q2, q) and torch.equal(k2, k) and torch.equal(v2, v)
    gate, up = torch.from_numpy(rng.standard_normal((5, 7))), torch.from_numpy(rng.standard_normal((5, 7)))
    assert torch.equal(P.fuse_components((gate, up), (1, 1)), W.fuse_gate_up(gate, up))
    with pytest.raises(ValueError):
        P.split_components(fused, (8, 2, 3))


def test_w4_pack_bytes_and_quantiser_match_the_oracle():
    from oracle import w8a8_oracle as O

    values = torch.tensor([[-7, -1, 0], [-6, 1, 7], [-5, 2, 6], [-4, 3, 5]], dtype=torch.int8)
    packed = S.pack_signed_int4(values)
    np.testing.assert_array_equal(packed.numpy(), np.asarray([[0xA9, 0x1F, 0x70], [0xCB, 0x32, 0x56]], dtype=np.uint8))
    assert torch.equal(S.unpack_signed_int4(packed), values)
    rng = np.random.default_rng(5)
    w = rng.standard_normal((70, 13)).astype(np.float32)
    got = S.quantize_frozen_weight(torch.from_numpy(w), bits=4, group_size=14, scale_dtype=torch.float32)
    want = O.quantize_frozen_weight(w, bits=4, group_size=14, scale_dtype=np.float32)
    np.testing.assert_array_equal(got.codes.numpy(), want.codes)
    np.testing.assert_array_equal(got.scales.numpy(), want.scales)
    assert got.bits == 4 and got.codes.dtype == torch.uint8


def test_lora_parameter_grads_match_the_oracle_vjp_on_cpu():
    # the rank-r gradient reductions are host-orchestrated library matmuls: checked here without a GPU
    from oracle import w8a8_oracle as O
    from skyrl_tx_rocm_b200 import backward as B

    rng = np.random.default_rng(3)
    m, k, n, r, na = 40, 24, 20, 4, 3
    x = rng.standard_normal((m, k)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    a = rng.standard_normal((na, k, r)).astype(np.float32) * 0.2
    b = rng.standard_normal((na, r, n)).astype(np.float32) * 0.2
    s = np.asarray([0.5, 1.0, 2.0], dtype=np.float32)
    ids = rng.integers(0, na, size=m).astype(np.int32)
    ids[ids == 1] = 0                                             # an adapter with no rows keeps zero gradients
    q = O.quantize_frozen_weight(rng.standard_normal((k, n)).astype(np.float32), scale_dtype=np.float32)
    _, want_da, want_db, want_ds = O.quantized_lora_linear_vjp(x, q, a, b, s, dy, ids)
    d_a, d_b, d_s = B.lora_parameter_grads(torch.from_numpy(x), torch.from_numpy(dy), torch.from_numpy(a),
                                           torch.from_numpy(b), torch.from_numpy(s), torch.from_numpy(ids))
    np.testing.assert_allclose(d_a.numpy(), want_da, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(d_b.numpy(), want_db, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(d_s.numpy(), want_ds, rtol=1e-5, atol=1e-5)
    assert not d_a[1].any() and not d_b[1].any() and d_s[1] == 0


def test_row_chunk_stack_chooses_its_chunks_on_the_host():
    from skyrl_tx_rocm_b200.stack import MLPStack

    blk = (None, None, None, None, None)
    stack = MLPStack([blk], num_chunks=2)
    assert stack.chunks_for(16384) == 2          # 8192 rows per chunk
    assert stack.chunks_for(2048) == 2           # exactly the 1024-row floor
    assert stack.chunks_for(1500) == 1           # a 768-row chunk hides nothing: the plain loop
    assert MLPStack([blk], num_chunks=4).chunks_for(3000) == 3   # 768 rows per chunk with four, 1024 (tile-rounded) with three
    with pytest.raises(ValueError):
        MLPStack([], num_chunks=2)
    with pytest.raises(ValueError):
        MLPStack([blk], num_chunks=0)
