"""The workspace-free W8A8 LoRA linear (skyrl_w8a8_lora_forward_noalloc_sm100_v1).

Some callers of the library cannot allocate device memory where they call it
(an XLA custom-call handler without a scratch result; a serving process whose
memory pool owns the whole device).  For them one entry point keeps its scratch
in a fixed 32 MiB array inside the library.  This test drives that entry point
through the C ABI and requires its output to equal, bit for bit, the output of
the workspace-taking entry point on the same inputs -- twice in a row with
different shapes, because the array keeps the previous call's contents.
It runs last so that a failure here cannot hide the result of any other test.
"""

import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _args(lib_mod, x, w, lora, ids, out, status, workspace=None):
    a = lib_mod.LinearArgs()
    a.struct_size = C.sizeof(lib_mod.LinearArgs)
    a.epilogue = lib_mod.EPI_LINEAR
    a.m, a.n, a.k = x.shape[0], w.padded_out_features, w.in_features
    a.rank, a.num_adapters = lora.rank, lora.num_adapters
    a.x, a.x_row_stride = x.data_ptr(), x.stride(0)
    a.wq, a.sw = w.wq.data_ptr(), w.sw.data_ptr()
    a.lora_a_packed, a.lora_b_packed = lora.a.data_ptr(), lora.b.data_ptr()
    a.lora_scaling = lora.scaling.data_ptr()
    a.lora_b_rows, a.lora_b_rows_rank = lora.b_rows.data_ptr(), lora.b_rows.shape[2]
    a.adapter_ids = ids.data_ptr()
    a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
    a.status = status.data_ptr()
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


def _case(S, seed, m, k, n, rank, adapters):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    wq = torch.randint(-127, 128, (n, k), generator=gen, device="cuda", dtype=torch.int8)
    sw = (torch.rand((n,), generator=gen, device="cuda") * 1e-3 + 1e-4).to(torch.bfloat16).float()
    a = (torch.randn((adapters, k, rank), generator=gen, device="cuda") / k ** 0.5).to(torch.bfloat16)
    b = (torch.randn((adapters, rank, n), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    s = torch.full((adapters,), 2.0, device="cuda")
    ids = torch.randint(0, adapters, (m,), generator=gen, device="cuda", dtype=torch.int32)
    return x, S.pack_weight_nk(wq, sw), S.pack_lora(a, b, s, in_features=k, padded_out_features=n), ids


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    import skyrl_tx_rocm_b200 as S
    from skyrl_tx_rocm_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    # second case is smaller than the first: stale scratch of call 1 lies behind call 2's regions
    for seed, (m, k, n, rank, adapters) in enumerate([(300, 1024, 512, 16, 4), (70, 256, 288, 8, 3)]):
        x, w, lora, ids = _case(S, seed, m, k, n, rank, adapters)
        want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        nbytes = lib.skyrl_w8a8_linear_workspace_bytes(m, n, k, adapters)
        assert 0 < nbytes < _lib.NOALLOC_SCRATCH_BYTES
        ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device="cuda")
        ws = ws[(-ws.data_ptr()) % 1024:][:nbytes]
        _lib.check(lib.skyrl_w8a8_lora_forward_sm100_v1(C.byref(_args(_lib, x, w, lora, ids, want, status, ws)), stream),
                   "reference entry point")
        _lib.check(lib.skyrl_w8a8_lora_forward_noalloc_sm100_v1(C.byref(_args(_lib, x, w, lora, ids, got, status)), stream),
                   "noalloc entry point")
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_noalloc_entry_point_rejects_oversized_requests():
    import skyrl_tx_rocm_b200 as S
    from skyrl_tx_rocm_b200 import _lib

    lib = _lib.load()
    m, k, n = 8192, 4096, 64          # needs about 3 * m * k = 100 MB of scratch
    x = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    w = S.pack_weight_nk(torch.zeros((n, k), dtype=torch.int8, device="cuda"), torch.ones(n, device="cuda"))
    a8 = torch.zeros((1, k, 8), dtype=torch.bfloat16, device="cuda")
    b8 = torch.zeros((1, 8, n), dtype=torch.bfloat16, device="cuda")
    lora = S.pack_lora(a8, b8, torch.ones(1, device="cuda"), in_features=k, padded_out_features=n)
    ids = torch.zeros(m, dtype=torch.int32, device="cuda")
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = lib.skyrl_w8a8_lora_forward_noalloc_sm100_v1(C.byref(_args(_lib, x, w, lora, ids, out, status)),
                                                      torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    msg = lib.skyrl_w8a8_last_error().decode()
    assert "needs" in msg and "built-in array" in msg
