"""GPU parity of the backward pass (straight-through VJP of the W8A8 LoRA linear) against the oracle.

The reference pins its backward to the closed form (tests/tx/kernels/test_quantized_lora.py:116-159, fp32,
2e-6); its production inputs are bf16.  Bars here: the cotangent's int8 planes bit-exact against their
restatement; dx (bf16) within relative-L2 1e-2 of the oracle's fp32 VJP as the task statement asks, with
the measured figure (about 2e-3: the bf16 rounding of dx itself) asserted at 4e-3; dA, dB, ds (fp32)
within 1e-4 relative L2.
"""

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import w8a8_oracle as O  # noqa: E402
from parity_util import big_lora, big_weight, device_normal, to_dev, to_np, uniform_ids  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S():
    import skyrl_tx_rocm_b200 as S

    return S


@pytest.fixture(scope="module")
def B():
    from skyrl_tx_rocm_b200 import backward

    return backward


def test_cotangent_planes_bit_exact(S):
    from skyrl_tx_rocm_b200 import _lib

    m, n = 37, 1072
    dy = device_normal((m, n), 5, 0.3)
    dy[3] = 0                                         # an all-zero row keeps scale 1
    col = torch.rand(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)) * 1e-2 + 1e-4
    perm = torch.randperm(m, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)).to(torch.int32)
    q = torch.empty((2, m, n), dtype=torch.int8, device="cuda")
    s = torch.empty((2, m), dtype=torch.float32, device="cuda")
    lib = _lib.load()
    _lib.check(lib.skyrl_w8a8_grad_quant_sm100_v1(dy.data_ptr(), dy.stride(0), col.data_ptr(), perm.data_ptr(), m, n,
                                                  q[0].data_ptr(), s[0].data_ptr(), q[1].data_ptr(), s[1].data_ptr(),
                                                  torch.cuda.current_stream().cuda_stream), "grad_quant")
    torch.cuda.synchronize()
    want = O.cotangent_int8_planes(to_np(dy)[to_np(perm)], to_np(col), planes=2)
    for p, (codes, scale) in enumerate(want):
        np.testing.assert_array_equal(to_np(s[p]), scale)
        np.testing.assert_array_equal(to_np(q[p]), codes)
    # the planes reproduce g to 2^-15 of the row's absmax
    g = to_np(dy)[to_np(perm)].astype(np.float32) * to_np(col)[None]
    rebuilt = sum(c.astype(np.float64) * sc.astype(np.float64)[:, None] for c, sc in want)
    assert np.max(np.abs(rebuilt - g)) <= np.max(np.abs(g)) / 127 / 254 * 1.01


@pytest.mark.parametrize("m,k,n,rank,na", [(300, 256, 384, 8, 3), (1024, 5120, 2048, 16, 4), (64, 512, 1024, 16, 2)])
def test_input_gradient_against_oracle(S, B, m, k, n, rank, na):
    w_host, w_packed = big_weight(S, k, n, 11)
    (a, b, s), _ = big_lora(S, na, k, rank, n, 13, 32.0)
    ids = uniform_ids(m, na, 17)
    dy = device_normal((m, n), 19, 0.05)
    x = device_normal((m, k), 23, 1.0)
    wb = B.pack_weight_backward(w_packed)
    lb = B.pack_lora_backward(to_dev(a), to_dev(b), to_dev(s), wb)
    want_dx, want_da, want_db, want_ds = O.quantized_lora_linear_vjp(to_np(x), w_host, a, b, s, to_np(dy), ids)
    want32 = want_dx.astype(np.float32)
    rel = {}
    for planes in (1, 2):
        dx = B.w8a8_lora_linear_input_grad(dy, wb, lb, to_dev(ids), planes=planes, enabled=True)
        S.check_status()
        rel[planes] = O.relative_l2(to_np(dx).astype(np.float32), want32)
    assert rel[2] < 4e-3, rel          # bf16 rounding of dx dominates; the task's bar is 1e-2
    assert rel[1] < 1e-2, rel          # one plane: the int8 step of the cotangent shows
    assert rel[2] <= rel[1]
    d_a, d_b, d_s = B.lora_parameter_grads(x, dy, to_dev(a), to_dev(b), to_dev(s), to_dev(ids))
    assert O.relative_l2(to_np(d_a), want_da) < 1e-4
    assert O.relative_l2(to_np(d_b), want_db) < 1e-4
    assert O.relative_l2(to_np(d_s), want_ds) < 1e-4


def test_input_gradient_without_lora_or_ids(S, B):
    m, k, n = 200, 384, 640
    w_host, w_packed = big_weight(S, k, n, 29)
    dy = device_normal((m, n), 31, 0.1)
    wb = B.pack_weight_backward(w_packed)
    dx = B.w8a8_lora_linear_input_grad(dy, wb, None, None, enabled=True)
    S.check_status()
    want = to_np(dy).astype(np.float32) @ O.dequantize_frozen_weight(w_host).T
    assert O.relative_l2(to_np(dx).astype(np.float32), want) < 4e-3


def test_autograd_function_matches_oracle_vjp(S, B):
    m, k, n, rank, na = 160, 256, 512, 8, 2
    w_host, w_packed = big_weight(S, k, n, 37)
    (a, b, s), _ = big_lora(S, na, k, rank, n, 41, 16.0)
    ids = uniform_ids(m, na, 43)
    x = device_normal((m, k), 47, 1.0).requires_grad_(True)
    ta, tb = to_dev(a).requires_grad_(True), to_dev(b).requires_grad_(True)
    ts = to_dev(s).requires_grad_(True)
    dy = device_normal((m, n), 53, 0.05)
    wb = B.pack_weight_backward(w_packed)
    y = B.w8a8_lora_linear_trainable(x, w_packed, wb, ta, tb, ts, to_dev(ids))
    y.backward(dy)
    S.check_status()
    # forward value is the inference operator's
    np.testing.assert_array_equal(to_np(y), to_np(S.w8a8_lora_linear(x.detach(), w_packed, ta.detach(), tb.detach(),
                                                                    ts.detach(), to_dev(ids), enabled=True)))
    want_dx, want_da, want_db, want_ds = O.quantized_lora_linear_vjp(to_np(x), w_host, a, b, s, to_np(dy), ids)
    assert O.relative_l2(to_np(x.grad).astype(np.float32), want_dx.astype(np.float32)) < 4e-3
    assert O.relative_l2(to_np(ta.grad).astype(np.float32), want_da) < 4e-3   # gradients are cast to the parameter dtype
    assert O.relative_l2(to_np(tb.grad).astype(np.float32), want_db) < 4e-3
    assert O.relative_l2(to_np(ts.grad), want_ds) < 1e-4


def test_input_gradient_at_the_c5_down_shape_sampled_rows(S, B):
    # full launch size of the Qwen3-32B-shaped down projection (M 16384, K 25600, N 5120, 16 adapters of rank 64);
    # every row of dx depends on its own row of dy only, so a seeded sample of rows goes through the oracle
    from parity_util import sample_rows

    m, k, n, rank, na = 16384, 25600, 5120, 64, 16
    w_host, w_packed = big_weight(S, k, n, 61)
    (a, b, s), _ = big_lora(S, na, k, rank, n, 67, 128.0)
    ids = uniform_ids(m, na, 71)
    dy = device_normal((m, n), 73, 0.02)
    wb = B.pack_weight_backward(w_packed)
    lb = B.pack_lora_backward(to_dev(a), to_dev(b), to_dev(s), wb)
    dx = B.w8a8_lora_linear_input_grad(dy, wb, lb, to_dev(ids), enabled=True)
    S.check_status()
    rows = sample_rows(m, 96, 79)
    dy_rows = to_np(dy[torch.from_numpy(rows).cuda()])
    x_dummy = np.zeros((len(rows), k), dtype=dy_rows.dtype)          # dx does not depend on x
    want, _, _, _ = O.quantized_lora_linear_vjp(x_dummy, w_host, a, b, s, dy_rows, ids[rows])
    got = to_np(dx[torch.from_numpy(rows).cuda()]).astype(np.float32)
    rel = O.relative_l2(got, want.astype(np.float32))
    assert rel < 4e-3, rel
