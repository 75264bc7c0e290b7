"""GPU parity at the benchmark configurations' full shapes, against the CPU oracle on sampled rows.

Every stage of the path is row-wise (a token row's result depends on that row, the weights and the row's
adapter only), so the oracle is evaluated on a few hundred sampled token rows of a full-size launch: what
is checked is the kernel configuration the benchmark times (tile plan, paired-tile kernel, split K,
two-adapter tiles, dynamic scheduler), at a CPU cost of seconds.

Bars.  Integer work (codes, scales, int32 accumulator) is bit-exact.  bf16 outputs: relative L2 < 1e-3 and
max-abs <= 2e-2 against the oracle, where an element may instead differ by ONE bf16 unit in the last place
if that difference is a PROVEN rounding tie: the float64 statement of the same formula lies on the
boundary between the two bf16 neighbours and the kernel's own fp32 pre-cast value agrees with it to
rounding noise (one bf16 spacing is 0.03 for |y| in [4, 8), so the absolute bar alone cannot be met by any
evaluation order there).  Outputs computed FROM the bf16 projection (SwiGLU product, residual sum) are
pinned in two steps: the fused epilogue applied to the kernel's own projection must reproduce the fused
kernel's output, and the projection itself must equal the oracle's up to proven ties.
"""

import ml_dtypes
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import w8a8_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
BF16 = ml_dtypes.bfloat16
MAX_ABS = 2e-2
REL_L2 = 1e-3


@pytest.fixture(scope="module")
def S():
    import skyrl_tx_rocm_b200 as S

    return S


from parity_util import (big_lora, big_weight, check_projection_chain, device_normal, sample_rows,  # noqa: E402
                         small_batch_accumulator, to_dev, to_np, uniform_ids)


# ----------------------------------------------------------------------------- a2: weight quantiser
@pytest.mark.parametrize("k,n,group", [(1024, 3072, None), (4096, 512, None), (130, 48, 64), (96, 40, 32)])
def test_weight_quantiser_bit_exact_on_device(S, k, n, group):
    # codes use the fp32 scale; the stored scale is rounded to bf16 afterwards (quantized_lora.py:150-171)
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:, 3] = 0.0                          # all-zero column -> scale 1.0, codes 0
    w[5, 7] = 0.127                        # column absmax set by one element
    w = w.astype(BF16)
    got = S.quantize_frozen_weight(to_dev(w), group_size=group)
    want = O.quantize_frozen_weight(w, group_size=group if group is not None else k + (k % 2))
    np.testing.assert_array_equal(to_np(got.codes), want.codes)
    np.testing.assert_array_equal(to_np(got.scales).view(np.uint16), want.scales.view(np.uint16))
    assert (got.original_in_features, got.padded_in_features, got.group_size) == (
        want.original_in_features, want.padded_in_features, want.group_size)


# ----------------------------------------------------------------------------- C2: decode layer, M = 64
def test_config2_decode_layer(S):
    m, hidden, inter, rank, na = 64, 4096, 12288, 16, 32
    x = device_normal((m, hidden), 1000)
    delta = device_normal((hidden,), 1001, 0.02)
    ids = uniform_ids(m, na, 1002)
    wgu, pgu = big_weight(S, hidden, 2 * inter, 1003)
    wd, pd = big_weight(S, inter, hidden, 1004)
    lgu_h, lgu = big_lora(S, na, hidden, rank, 2 * inter, 1005, 32.0)
    ld_h, ld = big_lora(S, na, inter, rank, hidden, 1007, 32.0)
    idd = to_dev(ids)
    out = S.w8a8_mlp_block(x, delta, pgu, lgu, pd, ld, idd, enabled=True, keep_normalized=True)
    S.check_status()
    _, h, hq, sh, xn = [t.clone() for t in S.w8a8_mlp_stage_regions(m, hidden, inter, na, x.device)]
    xq, sx, _ = [t.clone() for t in S.w8a8_mlp_workspace_regions(m, hidden, inter, na, x.device)]
    x_h, xn_k, h_k, out_k = to_np(x), to_np(xn), to_np(h), to_np(out)

    # RMSNorm: at most one bf16 step from the oracle (the reduction order of the sum of squares is not pinned)
    step = O.bf16_ulp_distance(xn_k, O.rms_norm(x_h, to_np(delta)))
    assert step.max() <= 1 and (step > 0).mean() < 2e-3
    # codes and scales of both projections' inputs: bit-exact given the rows the kernels saw
    codes, scales = O.dynamic_group_quantize(xn_k, hidden)
    np.testing.assert_array_equal(to_np(xq), codes[:, 0, :])
    np.testing.assert_array_equal(to_np(sx), scales[:, 0])
    hcodes, hscales = O.dynamic_group_quantize(h_k, inter)
    np.testing.assert_array_equal(to_np(hq), hcodes[:, 0, :])
    np.testing.assert_array_equal(to_np(sh), hscales[:, 0])

    # int32 accumulators of the decode GEMM plans (one wave of narrow tiles; split K over int32 slabs)
    for codes_dev, scales_dev, packed, host, want_codes in ((xq, sx, pgu, wgu, codes), (hq, sh, pd, wd, hcodes)):
        got_acc, _ = small_batch_accumulator(S, codes_dev, scales_dev, packed)
        k, n = host.codes.shape
        np.testing.assert_array_equal(got_acc, O.int8_group_gemm(want_codes, host.codes.reshape(1, k, n))[:, 0, :])
    lib = S._lib.load()
    assert lib.skyrl_w8a8_gemm_k_splits(m, hidden, inter, 16) > 1   # the down projection does split K here

    front = check_projection_chain(S, "c2 gate_up", xn_k, wgu, pgu, lgu_h, lgu, ids, h_k, "swiglu")
    back = check_projection_chain(S, "c2 down", h_k, wd, pd, ld_h, ld, ids, out_k, "residual", residual=x_h)
    # the composed layer: from the kernel's normalised rows within the bars; from x (the RMSNorm boundary is not
    # pinned by any reference test and re-draws bf16 roundings downstream) by relative L2 only
    want = O.residual_add(O.quantized_lora_linear(O.swiglu_interleaved(O.quantized_lora_linear(xn_k, wgu, *lgu_h, ids)),
                                                  wd, *ld_h, ids), x_h)
    rel = O.relative_l2(out_k, want)
    diff = np.abs(out_k.astype(np.float32) - want.astype(np.float32))
    ulp = O.bf16_ulp_distance(out_k, want)
    beyond = int(((diff > MAX_ABS) & (ulp > 1)).sum())
    rel_x = O.relative_l2(out_k, O.mlp_block(x_h, to_np(delta), wgu, *lgu_h, wd, *ld_h, ids))
    print(f"c2 layer: front {front} back {back} composed rel-L2 {rel:.2e} max-abs {diff.max():.4f} beyond {beyond}; "
          f"from x rel-L2 {rel_x:.2e}")
    # composed: downstream of the proven ties one bf16 step of h can move an int8 code of the down input, which
    # the oracle alone amplifies to ~1e-3 (test_composed_block_amplifies_one_step_differences): reported, loose bar
    assert rel < 2e-3 and rel_x < 2e-3


# ----------------------------------------------------------------------------- C3: prefill gate_up, M = 8192
def test_config3_gate_up_sampled_rows(S):
    m, k, inter, rank, na = 8192, 4096, 12288, 32, 4
    x = device_normal((m, k), 3)
    delta = device_normal((k,), 31, 0.02)
    runs = np.random.default_rng(32).integers(0, na, size=m // 512).astype(np.int32)
    ids = np.repeat(runs, 512)
    w_h, w_p = big_weight(S, k, 2 * inter, 33)
    l_h, l_p = big_lora(S, na, k, rank, 2 * inter, 34, 64.0)
    h = S.w8a8_rms_gate_up_lora_swiglu(x, delta, w_p, l_p, adapter_ids=to_dev(ids), enabled=True)
    S.check_status()
    assert h.shape == (m, inter)
    rows = sample_rows(m, 256, 35)
    rt = torch.from_numpy(rows).cuda()
    h_rows = to_np(h[rt])
    # the normalised rows exactly as the fused front stage produced them (same row kernel, one CTA per row)
    _, _, xn = S.rms_quant(x[rt].contiguous(), delta, want_normalized=True)
    xn_k = to_np(xn)
    step = O.bf16_ulp_distance(xn_k, O.rms_norm(to_np(x[rt]), to_np(delta)))
    assert step.max() <= 1 and (step > 0).mean() < 2e-3
    stats = check_projection_chain(S, "c3 gate_up", xn_k, w_h, w_p, l_h, l_p, ids[rows], h_rows, "swiglu")
    print(f"c3 gate_up, 256 sampled rows: {stats}")
    full = O.rms_gate_up_lora_swiglu(to_np(x[rt]), to_np(delta), w_h, *l_h, ids[rows])
    assert O.relative_l2(h_rows, full) < REL_L2


# ----------------------------------------------------------------------------- C4: prefill down + residual, M = 16384
def test_config4_down_residual_sampled_rows(S):
    m, k, n, rank, na = 16384, 12288, 4096, 32, 8
    g = device_normal((m, k), 4).float()
    hin = (torch.nn.functional.silu(g) * device_normal((m, k), 41).float()).to(torch.bfloat16)
    del g
    res = device_normal((m, n), 42)
    ids = uniform_ids(m, na, 43)
    w_h, w_p = big_weight(S, k, n, 44)
    l_h, l_p = big_lora(S, na, k, rank, n, 45, 64.0)
    out = S.w8a8_down_lora_residual(hin, w_p, l_p, residual=res, adapter_ids=to_dev(ids), enabled=True)
    S.check_status()
    rows = sample_rows(m, 256, 46)
    rt = torch.from_numpy(rows).cuda()
    stats = check_projection_chain(S, "c4 down", to_np(hin[rt]), w_h, w_p, l_h, l_p, ids[rows], to_np(out[rt]),
                                   "residual", residual=to_np(res[rt]))
    print(f"c4 down + residual, 256 sampled rows: {stats}")
    # the int32 accumulator of the same launch shape, sampled rows, bit-exact
    acc = S.w8a8_int32_accumulator(hin, w_p, enabled=True)
    S.check_status()
    codes, _ = O.dynamic_group_quantize(to_np(hin[rt]), k)
    np.testing.assert_array_equal(to_np(acc[rt]), O.int8_group_gemm(codes, w_h.codes.reshape(1, k, n))[:, 0, :])


@pytest.mark.parametrize("tp", [2, 8])
def test_config4_down_row_parallel_sampled_rows(S, tp):
    # C4 as the benchmark's 2/4/8-GPU configurations evaluate it: the input features are cut into tp shards, every
    # shard quantises its slice of the rows with its own per-token scale and its slice of the weight with its own
    # per-channel scale, the fp32 partial sums are added in ascending shard order, cast once and the residual added.
    # That is the reference's group format with group_size = K / tp (quantized_lora.py:199-254), so the oracle is its
    # plain quantised linear at that group size.  The shards run one after the other on this GPU, at the full launch
    # shape of a rank (M 16384, K 12288 / tp, N 4096, fp32 partial-sum epilogue).
    m, k, n, rank, na = 16384, 12288, 4096, 32, 8
    shard = k // tp
    g = device_normal((m, k), 4).float()
    hin = (torch.nn.functional.silu(g) * device_normal((m, k), 41).float()).to(torch.bfloat16)
    del g
    res = device_normal((m, n), 42)
    ids = uniform_ids(m, na, 43)
    w = device_normal((k, n), 47, 0.02)
    (a, b, s), _ = big_lora(S, na, k, rank, n, 45, 64.0)
    total = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    idd = to_dev(ids)
    for r in range(tp):
        sl = slice(r * shard, (r + 1) * shard)
        wq = S.pack_weight(S.quantize_frozen_weight(w[sl].contiguous()))
        part = S.w8a8_lora_linear_f32(hin[:, sl].contiguous(), wq, to_dev(a[:, sl].copy()), to_dev(b), to_dev(s), idd, enabled=True)
        total += part            # ascending shard order, fp32
    S.check_status()
    out = (total.to(torch.bfloat16).float() + res.float()).to(torch.bfloat16)
    rows = sample_rows(m, 192, 48)
    rt = torch.from_numpy(rows).cuda()
    q = O.quantize_frozen_weight(to_np(w), group_size=shard)
    want = O.quantized_lora_linear(to_np(hin[rt]), q, a, b, s, ids[rows])
    want = O.residual_add(want, to_np(res[rt]))
    got = to_np(out[rt])
    rel = O.relative_l2(got.astype(np.float32), want.astype(np.float32))
    worst = float(np.max(np.abs(got.astype(np.float32) - want.astype(np.float32))))
    print(f"c4 row-parallel tp={tp}, 192 sampled rows: rel_l2={rel:.3e} max_abs={worst:.4f}")
    assert rel < 1e-3 and worst <= 2e-2 + 2 ** -6          # one bf16 step at |y| < 4 on top of the 2e-2 bar


# ----------------------------------------------------------------------------- C5: one Qwen3-32B-shaped layer, M = 16384
def test_config5_layer_sampled_rows(S):
    m, hidden, inter, rank, na = 16384, 5120, 25600, 64, 16
    x = device_normal((m, hidden), 5000)
    delta = device_normal((hidden,), 5001, 0.02)
    ids = uniform_ids(m, na, 5002)
    wgu, pgu = big_weight(S, hidden, 2 * inter, 5003)
    wd, pd = big_weight(S, inter, hidden, 5004)
    lgu_h, lgu = big_lora(S, na, hidden, rank, 2 * inter, 5005, 128.0)
    ld_h, ld = big_lora(S, na, inter, rank, hidden, 5007, 128.0)
    idd = to_dev(ids)
    out = S.w8a8_mlp_block(x, delta, pgu, lgu, pd, ld, idd, enabled=True)
    S.check_status()
    perm, h, hq, sh, xn = S.w8a8_mlp_stage_regions(m, hidden, inter, na, x.device)
    rows = sample_rows(m, 192, 5009)
    # sorted position of every sampled token row
    inv = torch.empty(m, dtype=torch.int64, device="cuda")
    inv[perm.long()] = torch.arange(m, device="cuda")
    pos = inv[torch.from_numpy(rows).cuda()]
    np.testing.assert_array_equal(to_np(perm), O.prepare_routing(ids, na)[0])
    h_k, hq_k, sh_k, xn_k = to_np(h[pos]), to_np(hq[pos]), to_np(sh[pos]), to_np(xn[pos])
    rt = torch.from_numpy(rows).cuda()
    x_h, out_k = to_np(x[rt]), to_np(out[rt])

    step = O.bf16_ulp_distance(xn_k, O.rms_norm(x_h, to_np(delta)))
    assert step.max() <= 1 and (step > 0).mean() < 2e-3
    hcodes, hscales = O.dynamic_group_quantize(h_k, inter)      # row absmax collected by the gate_up epilogue
    np.testing.assert_array_equal(hq_k, hcodes[:, 0, :])
    np.testing.assert_array_equal(sh_k, hscales[:, 0])

    front = check_projection_chain(S, "c5 gate_up", xn_k, wgu, pgu, lgu_h, lgu, ids[rows], h_k, "swiglu")
    back = check_projection_chain(S, "c5 down", h_k, wd, pd, ld_h, ld, ids[rows], out_k, "residual", residual=x_h)
    want = O.residual_add(O.quantized_lora_linear(
        O.swiglu_interleaved(O.quantized_lora_linear(xn_k, wgu, *lgu_h, ids[rows])), wd, *ld_h, ids[rows]), x_h)
    rel = O.relative_l2(out_k, want)
    diff = np.abs(out_k.astype(np.float32) - want.astype(np.float32))
    ulp = O.bf16_ulp_distance(out_k, want)
    beyond = int(((diff > MAX_ABS) & (ulp > 1)).sum())
    rel_x = O.relative_l2(out_k, O.mlp_block(x_h, to_np(delta), wgu, *lgu_h, wd, *ld_h, ids[rows]))
    print(f"c5 layer, 192 sampled rows: front {front} back {back} composed rel-L2 {rel:.2e} "
          f"max-abs {diff.max():.4f} beyond {beyond}; from x rel-L2 {rel_x:.2e}")
    # composed: downstream of the proven ties one bf16 step of h can move an int8 code of the down input, which
    # the oracle alone amplifies to ~1e-3 (test_composed_block_amplifies_one_step_differences): reported, loose bar
    assert rel < 2e-3 and rel_x < 2e-3

    # int32 accumulator of the down projection at the full launch shape (K = 25600: the paired-tile kernel)
    hfull = h.clone()
    acc = S.w8a8_int32_accumulator(hfull, pd, enabled=True)
    S.check_status()
    np.testing.assert_array_equal(to_np(acc[pos]), O.int8_group_gemm(hcodes, wd.codes.reshape(1, inter, hidden))[:, 0, :])


# ----------------------------------------------------------------------------- small-batch path: bad adapter ids
def test_small_batch_bad_adapter_id_is_clamped_and_reported(S):
    # M <= 128 never goes through the routing kernel: the row kernels clamp the id (no load leaves the
    # tables) and record the status word, for the linear and for the MLP block alike
    rng = np.random.default_rng(9)
    m, hidden, inter, rank, na = 24, 256, 384, 16, 3
    x = device_normal((m, hidden), 91)
    w_h, w_p = big_weight(S, hidden, 2 * inter, 92)
    d_h, d_p = big_weight(S, inter, hidden, 93)
    _, l_p = big_lora(S, na, hidden, rank, 2 * inter, 94, 32.0)
    _, ld_p = big_lora(S, na, inter, rank, hidden, 96, 32.0)
    for bad in (-1, na, 1 << 20):
        ids = rng.integers(0, na, size=m).astype(np.int32)
        ids[m // 2] = bad
        S.w8a8_lora_linear(x, w_p, l_p, adapter_ids=to_dev(ids), enabled=True)
        with pytest.raises(S.SkyrlKernelError, match="adapter id"):
            S.check_status()
        S.w8a8_mlp_block(x, None, w_p, l_p, d_p, ld_p, to_dev(ids), enabled=True)
        with pytest.raises(S.SkyrlKernelError, match="adapter id"):
            S.check_status()
    ids = rng.integers(0, na, size=m).astype(np.int32)
    y = S.w8a8_mlp_block(x, None, w_p, l_p, d_p, ld_p, to_dev(ids), enabled=True)
    S.check_status()
    assert torch.isfinite(y.float()).all()
