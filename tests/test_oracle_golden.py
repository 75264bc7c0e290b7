"""The CPU oracle against the reference's own known answers (no GPU needed).

Sources (paths inside the reference project):
* rocm/probe_w8a8_lora_forward.py:210-218 ........ SHA-256 pins of the host case
* tests/rocm/test_w8a8_lora_forward_probe.py:368-392 . host oracle == portable oracle
* tests/tx/kernels/test_quantized_lora.py:45-74 ... hand-computed group-scale vectors
* tests/tx/kernels/test_quantized_lora.py:162-199 . zero groups finite; single bf16 cast
* rocm/probe_w8a8_lora_forward.py:1127-1190 ....... 35 sensitivity mutations > 3 %
"""

import hashlib
import json
from pathlib import Path

import ml_dtypes
import numpy as np
import pytest

from oracle import w8a8_oracle as O

GOLDEN = Path(__file__).parent / "golden"
BF16 = ml_dtypes.bfloat16


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes(order="C")).hexdigest()


def _host_case():
    z = np.load(GOLDEN / "w8a8_host_case.npz")
    g = int(z["group_size"])
    codes = z["weight_codes"]
    weight = O.GroupQuantizedWeight(
        codes=codes, scales=z["weight_scales_bf16"].view(BF16),
        original_in_features=codes.shape[0], padded_in_features=codes.shape[0], bits=8, group_size=g,
    )
    return z, weight


def test_host_case_inputs_match_reference_pins():
    z, _ = _host_case()
    pins = json.loads((GOLDEN / "w8a8_host_case_sha256.json").read_text())
    assert pins["expected"] == "964b0c1fe5f5c4cdbd60658717fee50a835006adf03011717b4914061ab4f88f"
    assert _sha(z["x_bf16"]) == pins["x"]
    assert _sha(z["weight_codes"]) == pins["weight_codes"]
    assert _sha(z["weight_scales_bf16"]) == pins["weight_scales"]
    assert _sha(z["lora_a_bf16"]) == pins["lora_a"]
    assert _sha(z["lora_b_bf16"]) == pins["lora_b"]
    assert _sha(z["lora_scaling"]) == pins["lora_scaling"]
    assert _sha(z["expected_bf16"]) == pins["expected"]


def test_oracle_reproduces_reference_pinned_output_bitwise():
    z, weight = _host_case()
    pins = json.loads((GOLDEN / "w8a8_host_case_sha256.json").read_text())
    n = int(z["out_features"])
    for exact in (True, False):
        y = O.quantized_lora_linear(
            z["x_bf16"].view(BF16), weight, z["lora_a_bf16"].view(BF16), z["lora_b_bf16"].view(BF16),
            z["lora_scaling"], exact_blas=exact,
        )
        y = np.ascontiguousarray(y[:, :n])
        assert y.dtype == BF16
        assert _sha(y) == pins["expected"]
        np.testing.assert_array_equal(y.view(np.uint16), z["expected_bf16"])


def test_host_case_weight_quantiser_reproduces_reference_codes():
    # the dense weight formula of rocm/probe_w8a8_lora_forward.py:1203-1216
    z, weight = _host_case()
    n = int(z["out_features"])
    k = weight.codes.shape[0]
    ki = np.arange(k, dtype=np.int32)[:, None]
    ni = np.arange(n, dtype=np.int32)[None, :]
    dense = (((ki * 7 + ni * 3) % 41) - 20).astype(np.float32) / 16.0
    q = O.quantize_frozen_weight(dense, group_size=64)
    np.testing.assert_array_equal(q.codes, weight.codes[:, :n])
    np.testing.assert_array_equal(q.scales.view(np.uint16), weight.scales[:, :n].view(np.uint16))


@pytest.mark.parametrize("name", ["pertoken_k256", "group64_k128", "pertoken_k512_r16", "zero_rows"])
def test_oracle_matches_reference_host_oracle_outputs(name):
    z = np.load(GOLDEN / "w8a8_ref_oracle_cases.npz")
    g = int(z[f"{name}.group_size"])
    codes = z[f"{name}.weight_codes"]
    weight = O.GroupQuantizedWeight(
        codes=codes, scales=z[f"{name}.weight_scales_bf16"].view(BF16),
        original_in_features=codes.shape[0], padded_in_features=codes.shape[0], bits=8, group_size=g,
    )
    y = O.quantized_lora_linear(
        z[f"{name}.x_bf16"].view(BF16), weight, z[f"{name}.lora_a_bf16"].view(BF16),
        z[f"{name}.lora_b_bf16"].view(BF16), z[f"{name}.lora_scaling"],
    )
    np.testing.assert_array_equal(y.view(np.uint16), z[f"{name}.expected_bf16"])
    assert np.all(np.isfinite(y.astype(np.float32)))


def test_hand_coded_group_scale_vectors():
    # int4 codes of test_quantized_lora.py:45-74 written out as signed values
    codes = np.asarray([[1, -2], [3, 4], [-5, 6], [0, -7]], dtype=np.int8)
    weight = O.GroupQuantizedWeight(
        codes=codes, scales=np.asarray([[0.5, 2.0], [1.5, 0.25]], dtype=np.float32),
        original_in_features=3, padded_in_features=4, bits=8, group_size=2,
    )
    np.testing.assert_array_equal(
        O.dequantize_frozen_weight(weight), np.asarray([[0.5, -4.0], [1.5, 8.0], [-7.5, 1.5]], dtype=np.float32)
    )
    x = np.asarray([[7.0, -3.0, -7.0], [0.0, 0.0, 3.0]], dtype=np.float32)
    out = O.quantized_frozen_linear_f32(x, weight, activation_bits=4)
    np.testing.assert_allclose(out, np.asarray([[51.5, -62.5], [-22.5, 4.5]], dtype=np.float32), rtol=1e-6, atol=1e-6)


def test_zero_groups_are_finite_and_exactly_zero():
    weight = O.quantize_frozen_weight(np.zeros((16, 5), dtype=BF16), group_size=8)
    assert np.all(weight.scales.astype(np.float32) == 1.0)
    x = np.zeros((2, 16), dtype=BF16)
    y = O.quantized_lora_linear(x, weight, np.ones((16, 2), dtype=BF16), np.zeros((2, 5), dtype=BF16), 1.0)
    assert y.dtype == BF16
    np.testing.assert_array_equal(y.astype(np.float32), np.zeros((2, 5), dtype=np.float32))


def test_single_bf16_cast_after_fp32_epilogue():
    rng = np.random.default_rng(41)
    x = rng.standard_normal((64, 16)).astype(BF16)
    w = rng.standard_normal((16, 9)).astype(BF16)
    a = (rng.standard_normal((16, 4)) * 0.2).astype(BF16)
    b = (rng.standard_normal((4, 9)) * 0.2).astype(BF16)
    weight = O.quantize_frozen_weight(w, group_size=8)
    y, parts = O.quantized_lora_linear(x, weight, a, b, 0.75, return_parts=True)
    base = O.quantized_frozen_linear_f32(x, weight)
    low = (x.astype(np.float32) @ a.astype(np.float32)) @ b.astype(np.float32)
    expected = (base + np.float32(0.75) * low).astype(BF16)
    early = (base.astype(BF16).astype(np.float32) + np.float32(0.75) * low).astype(BF16)
    np.testing.assert_array_equal(y.view(np.uint16), expected.view(np.uint16))
    assert np.count_nonzero(early.view(np.uint16) != expected.view(np.uint16)) > 0


def test_w8a8_accuracy_gate_against_dense():
    # test_quantized_lora.py:91-112: W8A8 vs x @ W relative L2 < 2.5 %
    rng = np.random.default_rng(18)
    x = rng.standard_normal((15, 70)).astype(np.float32)
    w = rng.standard_normal((70, 13)).astype(np.float32)
    q = O.quantize_frozen_weight(w, group_size=32, scale_dtype=np.float32)
    assert q.padded_in_features == 96 and q.scales.shape == (3, 13)
    assert O.relative_l2(O.dequantize_frozen_weight(q), w) < 0.012
    assert O.relative_l2(O.quantized_frozen_linear_f32(x, q), x @ w) < 0.025


def test_sensitivity_of_host_case():
    # every one of the reference's 35 omissions moves the output by more than 3 %
    z, weight = _host_case()
    n = int(z["out_features"])
    args = dict(
        x=z["x_bf16"].view(BF16), a=z["lora_a_bf16"].view(BF16), b=z["lora_b_bf16"].view(BF16), s=z["lora_scaling"],
    )
    expected = z["expected_bf16"].view(BF16)

    def run(x=None, codes=None, scales=None, a=None, b=None, s=None):
        w = O.GroupQuantizedWeight(
            codes=weight.codes if codes is None else codes, scales=weight.scales if scales is None else scales,
            original_in_features=64, padded_in_features=64, bits=8, group_size=64,
        )
        return O.quantized_lora_linear(
            args["x"] if x is None else x, w, args["a"] if a is None else a, args["b"] if b is None else b,
            args["s"] if s is None else s,
        )[:, :n]

    errs = [
        O.relative_l2(run(x=np.zeros_like(args["x"])), expected),
        O.relative_l2(run(codes=np.zeros_like(weight.codes)), expected),
        O.relative_l2(run(scales=np.zeros_like(weight.scales)), expected),
        O.relative_l2(run(a=np.zeros_like(args["a"])), expected),
        O.relative_l2(run(b=np.zeros_like(args["b"])), expected),
        O.relative_l2(run(s=np.zeros_like(args["s"])), expected),
        O.relative_l2(np.zeros_like(expected), expected),
    ]
    for row in range(expected.shape[0]):
        c = expected.copy(); c[row] = 0
        errs.append(O.relative_l2(c, expected))
    for col in range(n):
        c = expected.copy(); c[:, col] = 0
        errs.append(O.relative_l2(c, expected))
    for r in range(8):
        b = args["b"].copy(); b[r] = 0
        errs.append(O.relative_l2(run(b=b), expected))
    assert len(errs) == 35
    assert min(errs) > 0.03


def test_multi_adapter_gather_equals_per_token_formula():
    # tests/tx/layers/test_lora_fast_path.py:207-238: routed result == per-sample formula
    rng = np.random.default_rng(5)
    m, k, n, r, na = 37, 64, 24, 8, 4
    x = rng.standard_normal((m, k)).astype(BF16)
    w = O.quantize_frozen_weight((rng.standard_normal((k, n)) * 0.05).astype(BF16), group_size=k)
    a = (rng.standard_normal((na, k, r)) / 8).astype(BF16)
    b = (rng.standard_normal((na, r, n)) * 0.05).astype(BF16)
    s = np.asarray([2.0, 0.5, 1.0, 4.0], dtype=np.float32)
    ids = rng.integers(0, na, size=m).astype(np.int32)
    y = O.quantized_lora_linear(x, w, a, b, s, ids)
    for i in range(m):
        yi = O.quantized_lora_linear(x[i : i + 1], w, a[ids[i]], b[ids[i]], s[ids[i]])
        assert O.bf16_ulp_distance(y[i : i + 1], yi).max() <= 1
    sort_idx, sizes, unsort = O.prepare_routing(ids, na)
    assert np.all(np.diff(ids[sort_idx]) >= 0)
    np.testing.assert_array_equal(sort_idx[unsort], np.arange(m))
    tiles = O.row_tiles(sizes, 8)
    assert tiles[:, 1].sum() == m and np.all(tiles[:, 1] <= 8)
    sorted_ids = ids[sort_idx]
    for first, rows, adapter, second in tiles.tolist():
        owners = sorted_ids[first:first + rows]
        if second == 0:
            assert np.all(owners == adapter)
        else:
            split = second >> 16
            assert np.all(owners[:split] == adapter) and np.all(owners[split:] == (second & 0xffff) - 1)
    # at most one tile more than a dense packing per adapter boundary that a third adapter would cross
    assert tiles.shape[0] <= -(-m // 8) + na


def test_gate_then_up_pairing():
    # test_bf16_rms_gate_up_lora_swiglu.py:335-364: column 2i is gate_i, 2i+1 is up_i
    p = np.asarray([[1.0, 2.0, -3.0, 0.5]], dtype=BF16)
    h = O.swiglu_interleaved(p).astype(np.float32)
    silu = lambda t: t / (1 + np.exp(-t))
    np.testing.assert_allclose(h, [[silu(1.0) * 2.0, silu(-3.0) * 0.5]], rtol=1e-2)


def test_tp_statement_matches_group_format():
    rng = np.random.default_rng(9)
    m, hdim, inter, r, na, tp = 16, 64, 128, 8, 2, 2
    x = rng.standard_normal((m, hdim)).astype(BF16)
    delta = (rng.standard_normal(hdim) * 0.02).astype(BF16)
    wgu = O.quantize_frozen_weight((rng.standard_normal((hdim, 2 * inter)) * 0.05).astype(BF16), group_size=hdim)
    wd_dense = (rng.standard_normal((inter, hdim)) * 0.05).astype(BF16)
    gu_a = (rng.standard_normal((na, hdim, r)) / 8).astype(BF16); gu_b = (rng.standard_normal((na, r, 2 * inter)) * 0.05).astype(BF16)
    dn_a = (rng.standard_normal((na, inter, r)) / 11).astype(BF16); dn_b = (rng.standard_normal((na, r, hdim)) * 0.05).astype(BF16)
    s = np.asarray([2.0, 1.0], dtype=np.float32)
    ids = rng.integers(0, na, size=m).astype(np.int32)
    out_tp = O.tp_shard_mlp_reference(x, delta, wgu, gu_a, gu_b, s, wd_dense, dn_a, dn_b, s, ids, tp)
    wd_grouped = O.quantize_frozen_weight(wd_dense, group_size=inter // tp)
    out_grp = O.mlp_block(x, delta, wgu, gu_a, gu_b, s, wd_grouped, dn_a, dn_b, s, ids)
    # identical base term; LoRA partial sums differ only by fp32 association
    assert O.bf16_ulp_distance(out_tp, out_grp).max() <= 1
    assert O.relative_l2(out_tp, out_grp) < 1e-3


def test_composed_block_amplifies_one_step_differences():
    # Why the COMPOSED block is not held to the per-projection bars: move 0.2 % of the elements of h by one bf16
    # step (what proven rounding ties of the gate_up projection do) and the reference's own algorithm answers with
    # a relative L2 of about 1e-3 and elements off by several bf16 steps, because a step of a large h element is a
    # sizeable part of an int8 code step and one code is worth amax / 127.  Stage pins are therefore the parity
    # statement; the composed figure is reported.
    rng = np.random.default_rng(0)
    m, inter, hidden = 16, 12288, 256
    g = rng.standard_normal((m, inter)).astype(np.float32) * 1.3
    u = rng.standard_normal((m, inter)).astype(np.float32) * 1.3
    h = ((g / (1 + np.exp(-g))) * u).astype(BF16)
    w = (rng.standard_normal((inter, hidden)) * 0.02).astype(np.float32).astype(BF16)
    q = O.quantize_frozen_weight(w, group_size=inter)
    bits = h.view(np.uint16).copy()
    mask = rng.random(bits.shape) < 0.002
    bits[mask] += np.where(rng.random(int(mask.sum())) < 0.5, 1, -1).astype(np.uint16)
    moved = bits.view(BF16)
    assert O.bf16_ulp_distance(h, moved).max() == 1
    x = rng.standard_normal((m, hidden)).astype(np.float32).astype(BF16)
    y0 = O.residual_add(O.quantized_lora_linear(h, q), x)
    y1 = O.residual_add(O.quantized_lora_linear(moved, q), x)
    rel = O.relative_l2(y1, y0)
    assert 2e-4 < rel < 5e-3, rel
    c0, _ = O.dynamic_group_quantize(h, inter)
    c1, _ = O.dynamic_group_quantize(moved, inter)
    assert 0 < (c0 != c1).mean() < 1e-3          # a few int8 codes moved, each by one
    assert np.abs(c0.astype(np.int32) - c1.astype(np.int32)).max() == 1


def test_int4_pack_bytes_and_hand_coded_w4_vectors():
    # the reference's own W4 known answers (tests/tx/kernels/test_quantized_lora.py:30-74): nibble order of the
    # packing, independent dequantisation of hand-written codes / scales, and the W4A4 grouped linear
    values = np.asarray([[-7, -1, 0], [-6, 1, 7], [-5, 2, 6], [-4, 3, 5]], dtype=np.int8)
    packed = O.pack_signed_int4(values)
    assert packed.dtype == np.uint8 and packed.shape == (2, 3)
    np.testing.assert_array_equal(packed, np.asarray([[0xA9, 0x1F, 0x70], [0xCB, 0x32, 0x56]], dtype=np.uint8))
    np.testing.assert_array_equal(O.unpack_signed_int4(packed), values)
    weight = O.GroupQuantizedWeight(
        codes=np.asarray([[0x31, 0x4E], [0x0B, 0x96]], dtype=np.uint8),
        scales=np.asarray([[0.5, 2.0], [1.5, 0.25]], dtype=np.float32),
        original_in_features=3, padded_in_features=4, bits=4, group_size=2)
    np.testing.assert_array_equal(O.dequantize_frozen_weight(weight),
                                  np.asarray([[0.5, -4.0], [1.5, 8.0], [-7.5, 1.5]], dtype=np.float32))
    x = np.asarray([[7.0, -3.0, -7.0], [0.0, 0.0, 3.0]], dtype=np.float32)
    np.testing.assert_allclose(O.quantized_frozen_linear_f32(x, weight, activation_bits=4),
                               np.asarray([[51.5, -62.5], [-22.5, 4.5]], dtype=np.float32), rtol=1e-6, atol=1e-6)
    # the quantiser: W4 codes stay within [-7, 7] and round-trip through the packing
    rng = np.random.default_rng(4)
    w = rng.standard_normal((70, 13)).astype(np.float32)
    q4 = O.quantize_frozen_weight(w, group_size=14, bits=4, scale_dtype=np.float32)
    codes = O.unpacked_codes(q4)
    assert q4.codes.dtype == np.uint8 and codes.shape == (70, 13) and np.abs(codes).max() <= 7
    assert O.relative_l2(O.dequantize_frozen_weight(q4), w) < 0.20      # the reference's W4 round-trip gate


def test_vjp_matches_finite_differences_of_the_dequantised_model():
    # the reference pins its backward to these equations (tests/tx/kernels/test_quantized_lora.py:116-159:
    # jax.grad of the custom VJP == the documented closed form).  Here the closed form is checked against
    # central differences of the straight-through model y = x deq(W) + s (x A) B it is the gradient of.
    rng = np.random.default_rng(31)
    m, k, n, r, na = 6, 10, 7, 3, 2
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    a = (rng.standard_normal((na, k, r)) * 0.1).astype(np.float32)
    b = (rng.standard_normal((na, r, n)) * 0.1).astype(np.float32)
    s = np.asarray([0.75, 1.5], dtype=np.float32)
    ids = rng.integers(0, na, size=m).astype(np.int32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    q = O.quantize_frozen_weight(w, group_size=10, scale_dtype=np.float32)
    deq = O.dequantize_frozen_weight(q).astype(np.float64)

    def loss(x_, a_, b_, s_):
        y = x_.astype(np.float64) @ deq
        for i in range(m):
            y[i] += s_[ids[i]] * ((x_[i].astype(np.float64) @ a_[ids[i]].astype(np.float64)) @ b_[ids[i]].astype(np.float64))
        return float(np.sum(y * dy))

    dx, d_a, d_b, d_s = O.quantized_lora_linear_vjp(x, q, a, b, s, dy, ids)

    def numeric(arr, which):
        g = np.zeros(arr.shape, dtype=np.float64)
        it = np.nditer(arr, flags=["multi_index"])
        for _ in it:
            i = it.multi_index
            hi, lo = arr.astype(np.float64).copy(), arr.astype(np.float64).copy()
            hi[i] += 1e-3
            lo[i] -= 1e-3
            args_hi = [x, a, b, s]
            args_lo = [x, a, b, s]
            args_hi[which], args_lo[which] = hi, lo
            g[i] = (loss(*args_hi) - loss(*args_lo)) / 2e-3
        return g

    np.testing.assert_allclose(dx, numeric(x, 0), rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(d_a, numeric(a, 1), rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(d_b, numeric(b, 2), rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(d_s, numeric(s, 3), rtol=2e-4, atol=2e-4)
    # single-adapter form equals the reference's documented closed form
    dx1, da1, db1, ds1 = O.quantized_lora_linear_vjp(x, q, a[0], b[0], 0.75, dy)
    low = (dy @ b[0].T) * np.float32(0.75)
    np.testing.assert_allclose(dx1, dy @ O.dequantize_frozen_weight(q).T + low @ a[0].T, rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(da1[0], x.T @ low, rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(db1[0], ((x @ a[0]).T @ dy) * np.float32(0.75), rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(ds1[0], np.sum(dy * ((x @ a[0]) @ b[0])), rtol=2e-6, atol=2e-6)
