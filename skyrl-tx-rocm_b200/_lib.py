"""ctypes binding of the C-ABI library (include/skyrl_w8a8_sm100.h).

The library is loaded once and kept alive for the life of the process, like the
reference keeps its typed-FFI library handle
(skyrl/tx/kernels/rocm/gdn_ffi_smoke.py:323,349-353).  There is no fallback: if
the library is missing, every operator raises.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libskyrl_w8a8_sm100.so"

EPI_LINEAR, EPI_SWIGLU, EPI_RESIDUAL, EPI_ACC_I32, EPI_PARTIAL_F32 = 0, 1, 2, 3, 4
NOALLOC_SCRATCH_BYTES = 32 << 20
MLP_REUSE_ROUTING = 1
MLP_INPUT_PREPARED = 2
MLP_FINALIZE_SORTED = 4
MLP_NO_ROW_AMAX = 8
MLP_KEEP_NORMALIZED = 16
TP_EXCHANGE_SINGLE_KERNEL = 1
TP_EXCHANGE_MULTIMEM = 2
TP_EXCHANGE_PROFILE = 4
TP_EXCHANGE_WIDE = 8
MLP_FUSED_ROWS = 32
LINEAR_FUSED_ROWS = 1
GEMM_VARIANT_AUTO, GEMM_VARIANT_SINGLE, GEMM_VARIANT_TWO_TILES, GEMM_VARIANT_CTA_PAIR = 0, 1, 2, 3
FLAGS_GEMM_VARIANT_SHIFT = 8
LORA_RANK_PAD = 64
Z_PARTS = 6            # bf16 parts per row of the LoRA-A projection: 2 adapter slots x (hi, mid, lo)
TILE_ROWS = 128
WEIGHT_KBLOCK = 128

ERROR_NAMES = {
    -1: "invalid argument", -2: "launch failure", -3: "unsupported", -4: "workspace", -5: "driver entry point",
}
STATUS_NAMES = {
    101: "bounded wait ran out in the TMA producer", 102: "bounded wait ran out in the MMA issuer",
    103: "bounded wait ran out in the epilogue", 104: "bounded wait ran out in the LoRA step",
    105: "bounded wait for another rank's flag ran out",
    190: "self-test wait ran out (expected)", 201: "adapter id outside [0, num_adapters)", 202: "tile list overflow", 203: "scattered partial-sum row without an owner",
}


class GemmArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("epilogue", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("rank", C.c_int32), ("num_adapters", C.c_int32), ("max_tiles", C.c_int32),
        ("xq", C.c_void_p), ("sx", C.c_void_p), ("wq", C.c_void_p), ("sw", C.c_void_p),
        ("z_parts", C.c_void_p), ("lora_b_packed", C.c_void_p),
        ("tiles", C.c_void_p), ("num_tiles", C.c_void_p), ("out_row_map", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("out_row_stride", C.c_int64), ("residual_row_stride", C.c_int64), ("status", C.c_void_p),
        ("split_k_slabs", C.c_int32), ("cta_limit", C.c_int32),
        ("scatter_bases", C.c_void_p * 8), ("scatter_row0", C.c_int32), ("scatter_rows", C.c_int32),
        ("row_amax", C.c_void_p), ("sched", C.c_void_p),
        ("z_rows", C.c_void_p), ("row_adapter_ids", C.c_void_p), ("lora_b_rows", C.c_void_p),
        ("lora_b_rows_rank", C.c_int32), ("variant", C.c_int32),
        ("prefetch", C.c_void_p),
        ("prefetch_bytes", C.c_int64),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("epilogue", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("rank", C.c_int32), ("num_adapters", C.c_int32), ("flags", C.c_uint32),
        ("x", C.c_void_p), ("x_row_stride", C.c_int64), ("rms_delta", C.c_void_p),
        ("rms_eps", C.c_float), ("reserved1", C.c_int32),
        ("wq", C.c_void_p), ("sw", C.c_void_p), ("lora_a_packed", C.c_void_p), ("lora_b_packed", C.c_void_p),
        ("lora_scaling", C.c_void_p), ("adapter_ids", C.c_void_p), ("residual", C.c_void_p),
        ("residual_row_stride", C.c_int64), ("out", C.c_void_p), ("out_row_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("timing_events", C.c_void_p * 2),
        ("lora_b_rows", C.c_void_p), ("lora_b_rows_rank", C.c_int32), ("reserved2", C.c_int32),
    ]


class MlpArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("m", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32),
        ("rank", C.c_int32), ("num_adapters", C.c_int32), ("down_epilogue", C.c_int32), ("rms_eps", C.c_float),
        ("x", C.c_void_p), ("rms_delta", C.c_void_p), ("residual", C.c_void_p),
        ("gu_wq", C.c_void_p), ("gu_sw", C.c_void_p), ("gu_a_packed", C.c_void_p), ("gu_b_packed", C.c_void_p),
        ("gu_scaling", C.c_void_p),
        ("dn_wq", C.c_void_p), ("dn_sw", C.c_void_p), ("dn_a_packed", C.c_void_p), ("dn_b_packed", C.c_void_p),
        ("dn_scaling", C.c_void_p),
        ("adapter_ids", C.c_void_p), ("out", C.c_void_p), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("status", C.c_void_p), ("timing_events", C.c_void_p * 4),
        ("flags", C.c_uint32), ("b_rows_rank", C.c_int32), ("gu_b_rows", C.c_void_p), ("dn_b_rows", C.c_void_p),
        ("num_chunks", C.c_int32), ("chunk_index", C.c_int32), ("gemm_cta_limit", C.c_int32), ("tp_scatter_rows", C.c_int32),
        ("tp_scatter_bases", C.c_void_p * 8),
        ("prefetch_next", C.c_void_p),
        ("prefetch_next_bytes", C.c_int64),
        ("prefetch_down_bytes", C.c_int64),
    ]


class TpExchangeArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("tp", C.c_int32), ("row_begin", C.c_int32), ("row_count", C.c_int32),
        ("wait_value", C.c_int32), ("signal_value", C.c_int32), ("grid_ctas", C.c_int32), ("flags", C.c_uint32),
        ("partials", C.c_void_p * 8), ("wait_flags", C.c_void_p), ("peer_workspaces", C.c_void_p * 8),
        ("signal_flags", C.c_void_p * 8), ("out", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares
SYMBOLS = {
    "skyrl_w8a8_abi_version": (C.c_int, []),
    "skyrl_w8a8_last_error": (C.c_char_p, []),
    "skyrl_w8a8_bounded_wait_selftest_sm100_v1": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "skyrl_lora_route_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_rms_quant_sm100_v1": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_float, C.c_void_p, C.c_int32,
                                           C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skyrl_w8a8_grad_quant_sm100_v1": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skyrl_lora_a_proj_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                             C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                             C.c_void_p, C.c_void_p]),
    "skyrl_group_sum_cast_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                                C.c_int64, C.c_void_p]),
    "skyrl_w8a8_gemm_sm100_v1": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "skyrl_w8a8_gemm_k_splits": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "skyrl_w8a8_linear_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "skyrl_w8a8_lora_forward_sm100_v1": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "skyrl_w8a8_lora_forward_noalloc_sm100_v1": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "skyrl_rms_gate_up_w8a8_lora_swiglu_sm100_v1": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "skyrl_down_w8a8_lora_residual_sm100_v1": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "skyrl_w8a8_mlp_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "skyrl_w8a8_mlp_block_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.c_void_p]),
    "skyrl_w8a8_mlp_tp_finalize_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.c_void_p, C.c_void_p, C.c_int32,
                                                      C.c_int32, C.c_void_p]),
    "skyrl_w8a8_mlp_tp_finalize_slabs_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.POINTER(C.c_void_p), C.c_int32,
                                                            C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "skyrl_w8a8_mlp_tp_prepare_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.c_int32, C.c_int32, C.c_void_p]),
    "skyrl_w8a8_mlp_workspace_regions": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                   C.POINTER(C.c_size_t)]),
    "skyrl_w8a8_mlp_tp_exchange_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.POINTER(MlpArgs), C.POINTER(TpExchangeArgs),
                                                      C.c_void_p]),
    "skyrl_w8a8_tp_signal_sm100_v1": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p]),
    "skyrl_w8a8_tp_wait_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_w8a8_mlp_workspace_stage_regions": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                         C.POINTER(C.c_size_t)]),
    "skyrl_w8a8_mlp_tp_unsort_sm100_v1": (C.c_int, [C.POINTER(MlpArgs), C.c_void_p, C.c_void_p, C.c_void_p]),
    "skyrl_pack_weight_kn_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_pack_weight_nk_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_pack_lora_a_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_pack_lora_b_rows_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "skyrl_pack_lora_b_sm100_v1": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
}

_lock = threading.Lock()
_lib = None


class SkyrlKernelError(RuntimeError):
    """The C-ABI library rejected a call or failed to enqueue it."""


def load():
    """Return the loaded library; raises if it was not built (no fallback path)."""
    global _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise SkyrlKernelError(
                    f"{LIB_PATH} is missing: build it with `python skyrl-tx-rocm_b200/build.py` "
                    "(the W8A8 operators have no CPU or eager fallback)"
                )
            lib = C.CDLL(str(LIB_PATH))
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            if lib.skyrl_w8a8_abi_version() != 1:
                raise SkyrlKernelError("C-ABI version mismatch")
            _lib = lib
        return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().skyrl_w8a8_last_error().decode("utf-8", "replace")
        exc = ValueError if rc == -1 else SkyrlKernelError
        raise exc(f"{what}: {ERROR_NAMES.get(rc, rc)}: {msg}")
