"""The C-ABI library builds, loads and exports every symbol the header declares (no GPU needed)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "skyrl_w8a8_sm100.h"


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(skyrl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for required in (
        "skyrl_w8a8_lora_forward_sm100_v1", "skyrl_w8a8_mlp_block_sm100_v1", "skyrl_w8a8_gemm_sm100_v1",
        "skyrl_rms_quant_sm100_v1", "skyrl_lora_a_proj_sm100_v1", "skyrl_lora_route_sm100_v1",
    ):
        assert required in names


def test_library_loads_and_exports_every_declared_symbol():
    from skyrl_tx_rocm_b200 import _lib

    if not _lib.LIB_PATH.exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location("skyrl_build", ROOT / "skyrl-tx-rocm_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_library()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    declared = _declared_symbols()
    assert declared, "no symbols parsed from the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(declared) == set(_lib.SYMBOLS), "ctypes binding and header disagree"
    loaded = _lib.load()
    assert loaded.skyrl_w8a8_abi_version() == 1


def test_header_is_plain_c_and_size_queries_run_without_a_gpu():
    # csrc/abi_check.c includes the public header as C11 (-Wall -Wextra -Werror -pedantic, so the
    # _Static_assert layout checks are evaluated by a C compiler) and calls the size queries
    import subprocess

    from skyrl_tx_rocm_b200 import _lib

    exe = _lib.LIB_PATH.parent / "abi_check"
    assert exe.exists(), "build.py did not produce the C-ABI check"
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "abi=1" in res.stdout and "rc=-1" in res.stdout


def test_header_asserts_struct_layouts():
    text = HEADER.read_text()
    for name in ("SkyrlW8A8GemmArgs", "SkyrlW8A8LinearArgs", "SkyrlW8A8MlpArgs"):
        assert f"SKYRL_ABI_ASSERT(sizeof({name})" in text and f"offsetof({name}," in text


def test_struct_sizes_are_stable():
    from skyrl_tx_rocm_b200 import _lib

    # Natural alignment, no packing: these sizes are part of ABI v1 and are
    # checked against struct_size by every entry point.
    assert ctypes.sizeof(_lib.GemmArgs) == 32 + 11 * 8 + 2 * 8 + 8 + 8 + 8 * 8 + 8 + 8 + 8 + 4 * 8 + 2 * 8 == 288
    assert ctypes.sizeof(_lib.LinearArgs) == 32 + 3 * 8 + 8 + 7 * 8 + 8 + 8 + 8 + 8 + 8 + 8 + 2 * 8 + 16 == 200
    assert ctypes.sizeof(_lib.MlpArgs) == 32 + 18 * 8 + 4 * 8 + 8 + 16 + 16 + 8 * 8 + 3 * 8 == 336


def test_disabled_by_default_and_exact_bool():
    import torch

    import skyrl_tx_rocm_b200 as S

    x = torch.zeros((2, 16), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="disabled by default"):
        S.w8a8_lora_linear(x, None, None)
    with pytest.raises(TypeError, match="exact bool"):
        S.w8a8_lora_linear(x, None, None, enabled=1)
    with pytest.raises(RuntimeError, match="disabled by default"):
        S.w8a8_mlp_block(x, None, None, None, None, None)


def test_no_cpu_fallback():
    import torch

    import skyrl_tx_rocm_b200 as S

    w = S.quantize_frozen_weight(torch.randn(16, 32))
    assert w.codes.dtype == torch.int8 and w.scales.shape == (1, 32) and w.group_size == 16
    with pytest.raises(S.SkyrlKernelError, match="CUDA"):
        S.pack_weight(w)


def test_weight_quantiser_matches_oracle_bitwise():
    # the product's offline quantiser (ops.quantize_frozen_weight, here on CPU tensors) against the oracle's
    # restatement of quantized_lora.py:128-171: int8 codes from the fp32 scale, stored scale rounded to bf16
    import ml_dtypes
    import numpy as np
    import torch

    import skyrl_tx_rocm_b200 as S
    from oracle import w8a8_oracle as O

    rng = np.random.default_rng(0)
    for k, n, group in ((256, 96, None), (130, 48, 64), (64, 17, 32)):
        w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        w[:, 2] = 0.0                       # zero column: scale 1.0, codes 0
        w[1, 4] = 0.3                       # one element sets the column's absmax
        wb = w.astype(ml_dtypes.bfloat16)
        t = torch.from_numpy(wb.view(np.uint16).copy()).view(torch.bfloat16)
        got = S.quantize_frozen_weight(t, group_size=group)
        want = O.quantize_frozen_weight(wb, group_size=group if group is not None else k + (k % 2))
        np.testing.assert_array_equal(got.codes.numpy(), want.codes)
        np.testing.assert_array_equal(got.scales.view(torch.uint16).numpy(), want.scales.view(np.uint16))
        assert (got.padded_in_features, got.group_size) == (want.padded_in_features, want.group_size)
        assert int(np.abs(got.codes.numpy()[:, 2]).max()) == 0 and float(got.scales[0, 2]) == 1.0
