"""Python operator surface of the B200 W8A8 multi-LoRA MLP kernels.

Mirrors the operators the reference's model layers call (names, positional
order, `enabled=` discipline and error types), generalised to W8A8 with
per-token adapters:

* `w8a8_lora_linear`, `w8a8_frozen_linear` ... skyrl/tx/kernels/rocm/w8a8_lora.py:827-920
* `w8a8_rms_gate_up_lora_swiglu` ............ skyrl/tx/kernels/rocm/bf16_rms_gate_up_lora_swiglu_contiguous.py:698-757
* `w8a8_down_lora_residual` ................. skyrl/tx/kernels/rocm/bf16_lora_residual.py:507-566
* `w8a8_mlp_block` .......................... Qwen3_5MLP.forward_with_post_attention_rms, skyrl/tx/models/qwen3_5.py:786-826
* `GroupQuantizedWeight`, `quantize_frozen_weight` ... skyrl/tx/kernels/quantized_lora.py:20-41,128-171

torch is used for device memory and streams only; all arithmetic of the path
runs in the hand-written CUDA library behind the C ABI
(include/skyrl_w8a8_sm100.h).  There is no CPU or eager fallback.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._cache import IdentityCache
from ._lib import (GEMM_VARIANT_AUTO, GEMM_VARIANT_CTA_PAIR, GEMM_VARIANT_SINGLE, GEMM_VARIANT_TWO_TILES,  # noqa: F401
                   EPI_ACC_I32, EPI_LINEAR, EPI_PARTIAL_F32, EPI_RESIDUAL, EPI_SWIGLU, LORA_RANK_PAD, TILE_ROWS, Z_PARTS,
                   WEIGHT_KBLOCK, SkyrlKernelError)

__all__ = (
    "GroupQuantizedWeight", "PackedW8Weight", "PackedLoRA", "SkyrlKernelError",
    "quantize_frozen_weight", "pack_signed_int4", "unpack_signed_int4", "pack_weight", "pack_weight_nk", "pack_lora",
    "prepare_routing", "rms_quant",
    "w8a8_lora_linear", "w8a8_frozen_linear", "w8a8_int32_accumulator", "w8a8_lora_linear_f32",
    "w8a8_rms_gate_up_lora_swiglu", "w8a8_down_lora_residual", "w8a8_mlp_block", "w8a8_mlp_tp_finalize",
    "w8a8_mlp_tp_finalize_slabs", "w8a8_mlp_tp_unsort", "w8a8_mlp_workspace_regions", "w8a8_mlp_stage_regions",
    "w8a8_mlp_tp_exchange", "tp_signal", "tp_wait", "use_workspace",
    "chunk_rows",
    "EPI_LINEAR", "EPI_SWIGLU", "EPI_RESIDUAL", "EPI_ACC_I32", "EPI_PARTIAL_F32",
    "GEMM_VARIANT_AUTO", "GEMM_VARIANT_SINGLE", "GEMM_VARIANT_TWO_TILES", "GEMM_VARIANT_CTA_PAIR",
    "check_status", "bounded_wait_selftest", "RMS_EPS",
)

RMS_EPS = 1e-6
MAX_LORA_RANK = LORA_RANK_PAD


# --------------------------------------------------------------------------- #
# storage
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class GroupQuantizedWeight:
    """The reference's storage contract (quantized_lora.py:20-41): int8 codes
    [Kpad, N], scales [Kpad / group_size, N]."""

    codes: torch.Tensor
    scales: torch.Tensor
    original_in_features: int
    padded_in_features: int
    bits: int
    group_size: int


@dataclass(frozen=True)
class PackedW8Weight:
    """Device format of a per-output-channel W8 weight: int8 [ceil(K / 128), Npad, 128]
    (K-block-major: for one block of 128 K values the rows of all output channels are
    contiguous), fp32 scales [Npad]; `out_features` <= Npad (Npad % 32 == 0)."""

    wq: torch.Tensor
    sw: torch.Tensor
    in_features: int
    out_features: int
    group_size: int = 0  # 0: one scale per output channel; > 0: sw is [K / group_size, Npad] (compatibility path)

    @property
    def padded_out_features(self) -> int:
        return self.wq.shape[1]


@dataclass(frozen=True)
class PackedLoRA:
    """Device format of the LoRA tables of one projection: A as bf16
    [A, 64, K], B as bf16 [A, Npad, 64] (tensor-core path) and as dense bf16
    [A, Npad, rr] with rr = rank rounded up to 8 (small-batch path), scaling fp32 [A]."""

    a: torch.Tensor
    b: torch.Tensor
    scaling: torch.Tensor
    rank: int
    num_adapters: int
    b_rows: torch.Tensor | None = None


def _validate_exact_bool(name: str, value) -> None:
    if type(value) is not bool:
        raise TypeError(f"{name} must be an exact bool")


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise SkyrlKernelError(f"{name} must live on a CUDA device: the W8A8 operators have no CPU path")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def pack_signed_int4(values: torch.Tensor) -> torch.Tensor:
    """Pairs along axis zero -> low / high two's-complement nibbles of one byte (quantized_lora.py:94-107)."""
    if values.ndim < 1 or values.shape[0] == 0 or values.shape[0] % 2:
        raise ValueError("signed INT4 packing requires an even, nonempty axis zero")
    if values.dtype not in (torch.int8, torch.int16, torch.int32, torch.int64):
        raise TypeError(f"signed INT4 values must be integral, got {values.dtype}")
    low = (values[0::2].to(torch.int16) & 0xF).to(torch.uint8)
    high = (values[1::2].to(torch.int16) & 0xF).to(torch.uint8)
    return low | (high << 4)


def unpack_signed_int4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of `pack_signed_int4` (quantized_lora.py:110-125): int8 values in [-8, 7]."""
    if packed.ndim < 1 or packed.shape[0] == 0:
        raise ValueError("signed INT4 input must have a nonempty axis zero")
    if packed.dtype != torch.uint8:
        raise TypeError(f"packed signed INT4 values must be uint8, got {packed.dtype}")
    low = (packed & 0xF).to(torch.int16)
    high = (packed >> 4).to(torch.int16)
    low = torch.where(low >= 8, low - 16, low).to(torch.int8)
    high = torch.where(high >= 8, high - 16, high).to(torch.int8)
    return torch.stack((low, high), dim=1).reshape(packed.shape[0] * 2, *packed.shape[1:])


def quantize_frozen_weight(weight: torch.Tensor, *, bits: int = 8, group_size: int | None = None,
                           scale_dtype: torch.dtype = torch.bfloat16) -> GroupQuantizedWeight:
    """Offline symmetric quantiser of a [K, N] weight (quantized_lora.py:128-171), W8 or W4.

    `group_size=None` means one group over all of K (per-output-channel), the
    scheme every benchmark configuration uses.  Codes are computed with the
    fp32 scale; the stored scale is cast to `scale_dtype` afterwards.  W4 codes
    (range [-7, 7]) are packed two to a byte along K, as the reference stores them.
    """
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    qmax_int = (1 << (bits - 1)) - 1
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [K, N], got {tuple(weight.shape)}")
    if not weight.is_floating_point():
        raise TypeError(f"weight must be floating point, got {weight.dtype}")
    k, n = weight.shape
    if group_size is None:
        group_size = k + (k % 2)
    if group_size <= 0 or group_size % 2:
        raise ValueError(f"group_size must be a positive even integer, got {group_size}")
    kpad = (k + group_size - 1) // group_size * group_size
    w32 = torch.zeros((kpad, n), dtype=torch.float32, device=weight.device)
    w32[:k] = weight.to(torch.float32)
    grouped = w32.view(-1, group_size, n)
    amax = grouped.abs().amax(dim=1)
    # a TENSOR divisor: dividing by a Python scalar is evaluated as a multiplication by the rounded reciprocal,
    # which differs from the reference's fp32 quotient amax / 127 in the last bit for some values
    qmax = torch.full((), float(qmax_int), dtype=torch.float32, device=weight.device)
    scales = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    codes = torch.clamp(torch.round(grouped / scales[:, None, :]), -qmax_int, qmax_int).to(torch.int8)
    codes = codes.view(kpad, n).contiguous()
    if bits == 4:
        codes = pack_signed_int4(codes)
    return GroupQuantizedWeight(codes, scales.to(scale_dtype), k, kpad, bits, group_size)


def pack_weight(weight: GroupQuantizedWeight) -> PackedW8Weight:
    """[K, N] codes + [groups, N] scales -> the packed device format.

    W4 weights (quantized_lora.py:94-125: two codes per byte) are expanded to int8 codes here, once, at
    load time: sm_100 has no int4 tensor-core kind, so the W4 arithmetic runs on the same int8 kernels
    (exactly: the codes are the same integers), at W8 memory cost on the device."""
    if weight.bits == 4:
        if weight.codes.ndim != 2 or weight.codes.dtype != torch.uint8:
            raise TypeError("W4 codes must be a rank-two UINT8 array of packed nibbles")
        codes8 = unpack_signed_int4(weight.codes)[: weight.padded_in_features].contiguous()
        weight = GroupQuantizedWeight(codes8, weight.scales, weight.original_in_features, weight.padded_in_features, 8,
                                      weight.group_size)
    if weight.bits != 8:
        raise ValueError(f"the B200 path takes W8 or W4 codes, got W{weight.bits}")
    if weight.codes.ndim != 2 or weight.codes.dtype != torch.int8:
        raise TypeError("W8 codes must be a rank-two INT8 array")
    if weight.scales.ndim != 2 or not weight.scales.is_floating_point():
        raise TypeError("W8 scales must be a rank-two floating-point array")
    grouped = weight.group_size != weight.padded_in_features
    if weight.padded_in_features % weight.group_size or weight.scales.shape[0] != weight.padded_in_features // weight.group_size:
        raise ValueError(f"scale shape {tuple(weight.scales.shape)} does not match K={weight.padded_in_features}, "
                         f"group_size={weight.group_size}")
    if grouped and weight.group_size % 16:
        raise ValueError(f"grouped weights need group_size to be a multiple of 16, got {weight.group_size}")
    _require_cuda(weight.codes, "weight.codes")
    kpad, n = weight.codes.shape
    k = kpad
    if k % 16:
        k = (kpad + 15) // 16 * 16
    npad = (n + 31) // 32 * 32
    codes = weight.codes
    if k != kpad or npad != n:
        padded = torch.zeros((k, npad), dtype=torch.int8, device=codes.device)
        padded[:kpad, :n] = codes
        codes = padded
    codes = codes.contiguous()
    wq = torch.empty(((k + WEIGHT_KBLOCK - 1) // WEIGHT_KBLOCK, npad, WEIGHT_KBLOCK), dtype=torch.int8,
                     device=codes.device)
    lib = _lib.load()
    _lib.check(lib.skyrl_pack_weight_kn_sm100_v1(_ptr(codes), k, npad, _ptr(wq), _stream()), "pack_weight")
    if grouped:
        if k != kpad:
            raise ValueError("grouped weights need K to be a multiple of 16")
        sw = torch.zeros((weight.scales.shape[0], npad), dtype=torch.float32, device=codes.device)
        sw[:, :n] = weight.scales.to(torch.float32)
        return PackedW8Weight(wq, sw, k, n, weight.group_size)
    sw = torch.zeros((npad,), dtype=torch.float32, device=codes.device)
    sw[:n] = weight.scales[0].to(torch.float32)
    return PackedW8Weight(wq, sw, k, n)


def pack_weight_nk(codes_nk: torch.Tensor, scales: torch.Tensor) -> PackedW8Weight:
    """int8 [N, K] codes (K contiguous, the [out, in] order checkpoints use) + per-output-channel
    scales [N] -> the packed device format.  N must be a multiple of 32 and K of 16."""
    _require_cuda(codes_nk, "codes_nk")
    if codes_nk.ndim != 2 or codes_nk.dtype != torch.int8:
        raise TypeError("W8 codes must be a rank-two INT8 array")
    n, k = codes_nk.shape
    if n % 32 or k % 16:
        raise ValueError(f"pack_weight_nk needs N % 32 == 0 and K % 16 == 0, got N={n}, K={k}")
    if scales.shape != (n,):
        raise ValueError(f"scales must have shape ({n},), got {tuple(scales.shape)}")
    codes_nk = codes_nk.contiguous()
    wq = torch.empty(((k + WEIGHT_KBLOCK - 1) // WEIGHT_KBLOCK, n, WEIGHT_KBLOCK), dtype=torch.int8,
                     device=codes_nk.device)
    lib = _lib.load()
    _lib.check(lib.skyrl_pack_weight_nk_sm100_v1(_ptr(codes_nk), n, k, _ptr(wq), _stream()), "pack_weight_nk")
    return PackedW8Weight(wq, scales.to(torch.float32).contiguous(), k, n)


def pack_lora(lora_a: torch.Tensor, lora_b: torch.Tensor, lora_scaling, *, in_features: int | None = None,
              padded_out_features: int | None = None) -> PackedLoRA:
    """LoRA tables in the reference layout (A [A, K, r], B [A, r, N], scaling [A];
    2-D A/B + scalar = one adapter: lora.py:259-268) -> device format."""
    if isinstance(lora_a, PackedLoRA):
        return lora_a
    _require_cuda(lora_a, "lora_a")
    _require_cuda(lora_b, "lora_b")
    if lora_a.dtype != torch.bfloat16 or lora_b.dtype != torch.bfloat16:
        raise TypeError("LoRA A and B must both be BF16")
    if lora_a.ndim == 2 and lora_b.ndim == 2:
        lora_a, lora_b = lora_a[None], lora_b[None]
    if lora_a.ndim != 3 or lora_b.ndim != 3:
        raise ValueError("lora_a and lora_b must both be rank-two or both rank-three")
    na, k, r = lora_a.shape
    if lora_b.shape[0] != na or lora_b.shape[1] != r:
        raise ValueError(f"incompatible LoRA shapes: A={tuple(lora_a.shape)}, B={tuple(lora_b.shape)}")
    n = lora_b.shape[2]
    if r > MAX_LORA_RANK:
        raise ValueError(f"LoRA rank must not exceed {MAX_LORA_RANK}, got {r}")
    scaling = torch.as_tensor(lora_scaling, dtype=torch.float32, device=lora_a.device).reshape(-1)
    if scaling.numel() != na:
        raise ValueError(f"lora_scaling must have {na} entries, got {scaling.numel()}")
    kp = in_features if in_features is not None else (k + 15) // 16 * 16
    npad = padded_out_features if padded_out_features is not None else (n + 31) // 32 * 32
    if kp < k or npad < n:
        raise ValueError("packed LoRA dimensions must not be smaller than the logical ones")
    a_src, b_src = lora_a.contiguous(), lora_b.contiguous()
    if kp != k:
        a_src = torch.zeros((na, kp, r), dtype=torch.bfloat16, device=lora_a.device)
        a_src[:, :k] = lora_a
    if npad != n:
        b_src = torch.zeros((na, r, npad), dtype=torch.bfloat16, device=lora_a.device)
        b_src[:, :, :n] = lora_b
    a_packed = torch.empty((na, LORA_RANK_PAD, kp), dtype=torch.bfloat16, device=lora_a.device)
    b_packed = torch.empty((na, npad, LORA_RANK_PAD), dtype=torch.bfloat16, device=lora_a.device)
    lib = _lib.load()
    _lib.check(lib.skyrl_pack_lora_a_sm100_v1(_ptr(a_src), na, kp, r, _ptr(a_packed), _stream()), "pack_lora_a")
    _lib.check(lib.skyrl_pack_lora_b_sm100_v1(_ptr(b_src), na, r, npad, _ptr(b_packed), _stream()), "pack_lora_b")
    rr = (r + 7) // 8 * 8
    b_rows = torch.empty((na, npad, rr), dtype=torch.bfloat16, device=lora_a.device)
    _lib.check(lib.skyrl_pack_lora_b_rows_sm100_v1(_ptr(b_src), na, r, npad, _ptr(b_rows), _stream()), "pack_lora_b_rows")
    return PackedLoRA(a_packed, b_packed, scaling.contiguous(), r, na, b_rows)


# --------------------------------------------------------------------------- #
# per-device scratch (torch owns the memory; the C ABI never allocates)
# --------------------------------------------------------------------------- #
_workspaces: dict[int, torch.Tensor] = {}
_pinned_workspaces: set[int] = set()
_status: dict[int, torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None or ws.numel() < nbytes + 1024:
        if idx in _pinned_workspaces:
            raise SkyrlKernelError(f"the workspace registered with use_workspace() has {ws.numel()} bytes, this call needs "
                                   f"{nbytes + 1024}; register a larger one or release it with use_workspace(None)")
        ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    off = (-ws.data_ptr()) % 1024
    return ws[off: off + nbytes]


def use_workspace(buffer: torch.Tensor | None, device=None) -> None:
    """Make the operators of `buffer`'s device carve their scratch from `buffer` (uint8, CUDA) instead of a
    tensor of their own: a tensor-parallel stack registers a piece of peer-mapped (symmetric) memory here so
    that other ranks can store the rows they prepared straight into this rank's workspace.  The operators
    raise if a call needs more than the buffer holds.  `None` releases the registration."""
    if buffer is None:
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        _pinned_workspaces.discard(idx)
        _workspaces.pop(idx, None)
        return
    _require_cuda(buffer, "buffer")
    if buffer.dtype != torch.uint8 or buffer.ndim != 1 or not buffer.is_contiguous():
        raise TypeError("the workspace must be a contiguous one-dimensional uint8 tensor")
    idx = buffer.device.index if buffer.device.index is not None else torch.cuda.current_device()
    _workspaces[idx] = buffer
    _pinned_workspaces.add(idx)


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _status.get(idx)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=device)
        _status[idx] = st
    return st


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel recorded a failure (bounded wait ran
    out, adapter id out of range).  The operators themselves never synchronise."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _status_word(device)
    code = int(st[0].item())
    if code != 0:
        st.zero_()
        raise SkyrlKernelError(f"device status {code}: {_lib.STATUS_NAMES.get(code, 'unknown')}")


def bounded_wait_selftest(limit_ms: float = 50.0, device=None) -> None:
    """Launch the library's failure-detection self-test: one CTA waits `limit_ms` on a barrier nothing
    arrives at, gives up and records status 190.  The next `check_status()` raises for it; the device
    stays usable."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = _status_word(device)
    _lib.check(_lib.load().skyrl_w8a8_bounded_wait_selftest_sm100_v1(st.data_ptr(), int(limit_ms * 1e6), _stream()),
               "bounded_wait_selftest")


# --------------------------------------------------------------------------- #
# validation shared by the operators
# --------------------------------------------------------------------------- #
def _check_x(x: torch.Tensor, k_logical: int) -> torch.Tensor:
    _require_cuda(x, "x")
    if x.ndim < 2 or x.numel() == 0:
        raise ValueError(f"x must have a nonempty row domain and final K axis, got {tuple(x.shape)}")
    if x.dtype != torch.bfloat16:
        raise TypeError(f"x must be BF16, got {x.dtype}")
    if x.shape[-1] != k_logical:
        raise ValueError(f"x K={x.shape[-1]} does not match W8 K={k_logical}")
    return x.reshape(-1, x.shape[-1])


def _pad_cols(x2: torch.Tensor, k: int) -> torch.Tensor:
    if x2.shape[1] == k and x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0:
        return x2
    out = torch.zeros((x2.shape[0], k), dtype=x2.dtype, device=x2.device)
    out[:, : x2.shape[1]] = x2
    return out


def _check_ids(adapter_ids, m: int, lora: PackedLoRA | None):
    if adapter_ids is None:
        if lora is not None and lora.num_adapters != 1:
            raise ValueError("adapter_ids is required when the LoRA tables hold more than one adapter")
        return None
    _require_cuda(adapter_ids, "adapter_ids")
    if adapter_ids.dtype != torch.int32:
        raise TypeError(f"adapter_ids must be INT32, got {adapter_ids.dtype}")
    if adapter_ids.shape != (m,):
        raise ValueError(f"adapter_ids must have shape ({m},), got {tuple(adapter_ids.shape)}")
    return adapter_ids.contiguous()


# Conversions of the reference's own argument types (GroupQuantizedWeight, [A, K, r] / [A, r, N] LoRA tables) to
# the device format happen once per tensor version, not per call: the reference's design asks for a load-time
# canonical weight (rocm/QUANTIZED_FFI.md:69-74), and a LoRA table changes only at an optimizer step.
_pack_cache = IdentityCache()


def _weight_of(weight) -> PackedW8Weight:
    if isinstance(weight, PackedW8Weight):
        return weight
    if isinstance(weight, GroupQuantizedWeight):
        return _pack_cache.get((weight.codes, weight.scales), (weight.group_size, weight.padded_in_features),
                               lambda: pack_weight(weight))
    raise TypeError("weight must be a GroupQuantizedWeight or a PackedW8Weight")


def _lora_of(weight: PackedW8Weight, lora_a, lora_b, lora_scaling) -> PackedLoRA:
    if isinstance(lora_a, PackedLoRA):
        lora = lora_a
    else:
        a_k = lora_a.shape[-2]
        if a_k not in (weight.in_features,) and not (a_k <= weight.in_features < a_k + 16):
            raise ValueError(f"lora_a K={a_k} does not match W8 K={weight.in_features}")
        if lora_b.shape[-1] != weight.out_features:
            raise ValueError(f"LoRA output N={lora_b.shape[-1]} does not match weight N={weight.out_features}")
        sources = (lora_a, lora_b) + ((lora_scaling,) if isinstance(lora_scaling, torch.Tensor) else ())
        extra = (weight.in_features, weight.padded_out_features,
                 None if isinstance(lora_scaling, torch.Tensor) else float(lora_scaling))
        lora = _pack_cache.get(sources, extra, lambda: pack_lora(lora_a, lora_b, lora_scaling, in_features=weight.in_features,
                                                                 padded_out_features=weight.padded_out_features))
    if lora.a.shape[2] != weight.in_features or lora.b.shape[1] != weight.padded_out_features:
        raise ValueError("packed LoRA tables do not match the packed weight")
    return lora


def _run_linear_grouped(x2, weight: PackedW8Weight, lora: PackedLoRA | None, ids):
    """Compatibility path for group_size < K: one single-group GEMM per K group into fp32 slabs, then the
    ordered group sum, the LoRA term (accumulated by the last group's GEMM) and the single bf16 cast
    (quantized_lora.py:242-254, 298-304).  Correct for every group size; not tuned."""
    lib = _lib.load()
    m, k, npad, g_size = x2.shape[0], weight.in_features, weight.padded_out_features, weight.group_size
    groups = k // g_size
    x2 = _pad_cols(x2, k)
    dev = x2.device
    na = lora.num_adapters if lora is not None else 1
    st = _status_word(dev)
    perm, tiles, num = prepare_routing(ids, m, na)
    row_map = perm if ids is not None else None
    max_tiles = tiles.shape[0]
    z_parts = None
    if lora is not None:
        if ids is not None:
            _, _, xs = rms_quant(x2, row_map=perm, want_normalized=True)  # rows gathered into sorted order
        else:
            xs = x2.contiguous()
        z_parts = torch.empty((m, Z_PARTS, LORA_RANK_PAD), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.skyrl_lora_a_proj_sm100_v1(_ptr(xs), m, k, _ptr(lora.a), _ptr(lora.scaling), na, lora.rank,
                                                  _ptr(tiles), _ptr(num), max_tiles, _ptr(z_parts), _ptr(st),
                                                  _stream()), "lora_a_proj")
    slabs = torch.empty((groups, m, npad), dtype=torch.float32, device=dev)
    sliceable = g_size % _lib.WEIGHT_KBLOCK == 0  # whole K blocks of the packed weight per group
    for j in range(groups):
        xq_j, sx_j, _ = rms_quant(x2[:, j * g_size:(j + 1) * g_size], row_map=row_map)
        a = _lib.GemmArgs()
        a.struct_size = C.sizeof(_lib.GemmArgs)
        a.epilogue = EPI_PARTIAL_F32
        a.m, a.n = m, npad
        if sliceable:
            a.k = g_size
            xq = xq_j
            a.wq = weight.wq.data_ptr() + j * (g_size // _lib.WEIGHT_KBLOCK) * npad * _lib.WEIGHT_KBLOCK
        else:
            # a group that is not a whole number of 128-wide K blocks: full-K pass with the codes of the
            # other groups zeroed, which contributes exactly nothing to the int32 accumulator
            a.k = k
            xq = torch.zeros((m, k), dtype=torch.int8, device=dev)
            xq[:, j * g_size:(j + 1) * g_size] = xq_j
            a.wq = weight.wq.data_ptr()
        a.xq, a.sx, a.sw = xq.data_ptr(), sx_j.data_ptr(), weight.sw[j].data_ptr()
        last = j == groups - 1
        a.rank = lora.rank if (lora is not None and last) else 0
        a.num_adapters = na
        a.max_tiles = max_tiles
        if a.rank:
            a.z_parts, a.lora_b_packed = z_parts.data_ptr(), lora.b.data_ptr()
        a.tiles, a.num_tiles = tiles.data_ptr(), num.data_ptr()
        a.out, a.out_row_stride = slabs[j].data_ptr(), npad
        a.status = st.data_ptr()
        _lib.check(lib.skyrl_w8a8_gemm_sm100_v1(C.byref(a), _stream()), "w8a8_gemm (group)")
    out = torch.empty((m, npad), dtype=torch.bfloat16, device=dev)
    _lib.check(lib.skyrl_group_sum_cast_sm100_v1(_ptr(slabs), groups, m, npad, _ptr(row_map), _ptr(out), npad,
                                                 _stream()), "group_sum_cast")
    return out


def _run_linear(x2, weight: PackedW8Weight, lora: PackedLoRA | None, ids, epilogue, *, rms_delta=None, eps=RMS_EPS,
                residual=None, out=None, timing_events=None, fused_rows=False, gemm_variant=0):
    if weight.group_size:
        if epilogue != EPI_LINEAR or rms_delta is not None or residual is not None:
            raise SkyrlKernelError("grouped weights (group_size < K) are served by w8a8_lora_linear and "
                                   "w8a8_frozen_linear only; the fused operators take per-output-channel scales")
        return _run_linear_grouped(x2, weight, lora, ids)
    lib = _lib.load()
    m = x2.shape[0]
    k, npad = weight.in_features, weight.padded_out_features
    x2 = _pad_cols(x2, k)
    dev = x2.device
    if epilogue == EPI_SWIGLU:
        out_cols, out_dtype = npad // 2, torch.bfloat16
    elif epilogue == EPI_ACC_I32:
        out_cols, out_dtype = npad, torch.int32
    elif epilogue == EPI_PARTIAL_F32:
        out_cols, out_dtype = npad, torch.float32
    else:
        out_cols, out_dtype = npad, torch.bfloat16
    if out is None:
        out = torch.empty((m, out_cols), dtype=out_dtype, device=dev)
    na = lora.num_adapters if lora is not None else 1
    nbytes = lib.skyrl_w8a8_linear_workspace_bytes(m, npad, k, na)
    ws = _workspace(dev, nbytes)
    st = _status_word(dev)
    a = _lib.LinearArgs()
    a.struct_size = C.sizeof(_lib.LinearArgs)
    a.epilogue = epilogue
    a.m, a.n, a.k = m, npad, k
    a.rank = lora.rank if lora is not None else 0
    a.num_adapters = na
    a.flags = (_lib.LINEAR_FUSED_ROWS if fused_rows else 0) | (int(gemm_variant) << _lib.FLAGS_GEMM_VARIANT_SHIFT)
    a.x = x2.data_ptr()
    a.x_row_stride = x2.stride(0)
    a.rms_delta = rms_delta.data_ptr() if rms_delta is not None else None
    a.rms_eps = float(eps)
    a.wq = weight.wq.data_ptr()
    a.sw = weight.sw.data_ptr()
    if lora is not None:
        a.lora_a_packed = lora.a.data_ptr()
        a.lora_b_packed = lora.b.data_ptr()
        a.lora_scaling = lora.scaling.data_ptr()
        if lora.b_rows is not None:
            a.lora_b_rows, a.lora_b_rows_rank = lora.b_rows.data_ptr(), lora.b_rows.shape[2]
    a.adapter_ids = ids.data_ptr() if ids is not None else None
    if residual is not None:
        a.residual = residual.data_ptr()
        a.residual_row_stride = residual.stride(0)
    a.out = out.data_ptr()
    a.out_row_stride = out.stride(0)
    a.workspace = ws.data_ptr()
    a.workspace_bytes = nbytes
    a.status = st.data_ptr()
    if timing_events is not None:
        a.timing_events[0], a.timing_events[1] = timing_events[0].cuda_event, timing_events[1].cuda_event
    # every fused variant has its own exported target (one symbol per operator, as a custom-call layer binds them)
    if epilogue == EPI_SWIGLU:
        _lib.check(lib.skyrl_rms_gate_up_w8a8_lora_swiglu_sm100_v1(C.byref(a), _stream()), "rms_gate_up_w8a8_lora_swiglu")
    elif epilogue == EPI_RESIDUAL:
        _lib.check(lib.skyrl_down_w8a8_lora_residual_sm100_v1(C.byref(a), _stream()), "down_w8a8_lora_residual")
    else:
        _lib.check(lib.skyrl_w8a8_lora_forward_sm100_v1(C.byref(a), _stream()), "w8a8_lora_forward")
    return out


def _pad_delta(rms_delta, k_logical: int, k: int):
    _require_cuda(rms_delta, "rms_delta")
    if rms_delta.dtype != torch.bfloat16 or rms_delta.shape != (k_logical,):
        raise TypeError(f"rms_delta must be BF16 with shape ({k_logical},)")
    if k == k_logical:
        return rms_delta.contiguous()
    raise ValueError("RMSNorm fusion needs K to be a multiple of 16")


# --------------------------------------------------------------------------- #
# operators
# --------------------------------------------------------------------------- #
def w8a8_frozen_linear(x, weight, *, enabled: bool = False, interpret: bool = False, block_m: int = 128,
                       block_n: int = 256, row_superblock: int = 0):
    """Frozen W8A8 base only (w8a8_lora.py:827-867).  Tile-size keywords are
    accepted for signature compatibility and ignored."""
    _validate_exact_bool("enabled", enabled)
    _validate_exact_bool("interpret", interpret)
    if not enabled:
        raise RuntimeError("the W8A8 frozen-linear kernel is disabled by default")
    w = _weight_of(weight)
    k_logical = weight.original_in_features if isinstance(weight, GroupQuantizedWeight) else w.in_features
    x2 = _check_x(x, k_logical)
    y = _run_linear(x2, w, None, None, EPI_LINEAR)
    return y[:, : w.out_features].reshape(*x.shape[:-1], w.out_features)


def w8a8_lora_linear(x, weight, lora_a, lora_b=None, lora_scaling=None, adapter_ids=None, *, enabled: bool = False,
                     interpret: bool = False, block_m: int = 128, block_n: int = 256, row_superblock: int = 0,
                     timing_events=None, fused_rows: bool = False, gemm_variant: int = 0):
    """y = bf16(dequant(xq wq^T) + s (x A) B) (w8a8_lora.py:870-920).

    `lora_a` [K, r] / `lora_b` [r, N] / scalar scaling select one adapter as in
    the reference; [A, K, r] / [A, r, N] / [A] with `adapter_ids` int32 [M]
    select an adapter per token row.  A `PackedLoRA` may be passed as `lora_a`.
    """
    _validate_exact_bool("enabled", enabled)
    _validate_exact_bool("interpret", interpret)
    if not enabled:
        raise RuntimeError("the W8A8 LoRA kernel is disabled by default")
    w = _weight_of(weight)
    k_logical = weight.original_in_features if isinstance(weight, GroupQuantizedWeight) else w.in_features
    x2 = _check_x(x, k_logical)
    lora = _lora_of(w, lora_a, lora_b, lora_scaling)
    ids = _check_ids(adapter_ids, x2.shape[0], lora)
    y = _run_linear(x2, w, lora, ids, EPI_LINEAR, timing_events=timing_events, fused_rows=fused_rows, gemm_variant=gemm_variant)
    return y[:, : w.out_features].reshape(*x.shape[:-1], w.out_features)


def w8a8_lora_linear_f32(x, weight, lora_a=None, lora_b=None, lora_scaling=None, adapter_ids=None, *,
                         enabled: bool = False, gemm_variant: int = 0):
    """The fp32 value of `w8a8_lora_linear` BEFORE its single bf16 cast, (f32(acc) * sx) * sw + s (x A) B
    (quantized_lora.py:248-252, 301-303), in token order.  Parity evidence: where a bf16 output differs from
    the reference's by one unit in the last place, this value shows whether the exact result sat on a
    rounding boundary.  `lora_a=None` gives the frozen base."""
    _validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 pre-cast probe is disabled by default")
    w = _weight_of(weight)
    k_logical = weight.original_in_features if isinstance(weight, GroupQuantizedWeight) else w.in_features
    x2 = _check_x(x, k_logical)
    lora = _lora_of(w, lora_a, lora_b, lora_scaling) if lora_a is not None else None
    ids = _check_ids(adapter_ids, x2.shape[0], lora)
    y = _run_linear(x2, w, lora, ids, EPI_PARTIAL_F32, gemm_variant=gemm_variant)
    return y[:, : w.out_features]


def w8a8_int32_accumulator(x, weight, *, enabled: bool = False, gemm_variant: int = 0):
    """Raw int32 accumulator xq @ wq^T and the activation codes' scales, for
    bit-exact parity checks (quantized_lora.py:242-247)."""
    _validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 accumulator probe is disabled by default")
    w = _weight_of(weight)
    x2 = _check_x(x, w.in_features if not isinstance(weight, GroupQuantizedWeight) else weight.original_in_features)
    acc = _run_linear(x2, w, None, None, EPI_ACC_I32, gemm_variant=gemm_variant)
    return acc[:, : w.out_features]


def w8a8_rms_gate_up_lora_swiglu(x, rms_delta, frozen_weight, lora_a, lora_b=None, lora_scaling=None,
                                 adapter_ids=None, *, enabled: bool = False, eps: float = RMS_EPS, timing_events=None,
                                 gemm_variant: int = 0):
    """h = swiglu(W8A8-LoRA gate_up(rmsnorm(x))) with interleaved (gate, up)
    columns; never materialises the [M, 2I] projection
    (bf16_rms_gate_up_lora_swiglu_contiguous.py:698-757).  `rms_delta=None`
    skips the normalisation."""
    _validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 RMS+gate/up+SwiGLU kernel is disabled by default")
    w = _weight_of(frozen_weight)
    if w.out_features % 2:
        raise ValueError("gate_up needs an even number of physical output columns")
    k_logical = frozen_weight.original_in_features if isinstance(frozen_weight, GroupQuantizedWeight) else w.in_features
    x2 = _check_x(x, k_logical)
    lora = _lora_of(w, lora_a, lora_b, lora_scaling) if lora_a is not None else None
    ids = _check_ids(adapter_ids, x2.shape[0], lora)
    delta = _pad_delta(rms_delta, k_logical, w.in_features) if rms_delta is not None else None
    h = _run_linear(x2, w, lora, ids, EPI_SWIGLU, rms_delta=delta, eps=eps, timing_events=timing_events,
                    gemm_variant=gemm_variant)
    inter = w.out_features // 2
    return h[:, :inter].reshape(*x.shape[:-1], inter)


def w8a8_down_lora_residual(x, frozen_weight, lora_a, lora_b=None, lora_scaling=None, residual=None,
                            adapter_ids=None, *, enabled: bool = False, timing_events=None, gemm_variant: int = 0):
    """out = residual + W8A8-LoRA down(x) (bf16_lora_residual.py:507-566)."""
    _validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 down+residual kernel is disabled by default")
    w = _weight_of(frozen_weight)
    k_logical = frozen_weight.original_in_features if isinstance(frozen_weight, GroupQuantizedWeight) else w.in_features
    x2 = _check_x(x, k_logical)
    lora = _lora_of(w, lora_a, lora_b, lora_scaling) if lora_a is not None else None
    ids = _check_ids(adapter_ids, x2.shape[0], lora)
    if residual is None:
        y = _run_linear(x2, w, lora, ids, EPI_LINEAR)
    else:
        _require_cuda(residual, "residual")
        if residual.dtype != torch.bfloat16:
            raise TypeError(f"residual must be BF16, got {residual.dtype}")
        r2 = residual.reshape(-1, residual.shape[-1])
        if r2.shape != (x2.shape[0], w.out_features):
            raise ValueError(f"residual must have shape ({x2.shape[0]}, {w.out_features}), got {tuple(r2.shape)}")
        r2 = _pad_cols(r2, w.padded_out_features)
        y = _run_linear(x2, w, lora, ids, EPI_RESIDUAL, residual=r2, timing_events=timing_events,
                        gemm_variant=gemm_variant)
    return y[:, : w.out_features].reshape(*x.shape[:-1], w.out_features)


def w8a8_mlp_block(x, rms_delta, gate_up_weight: PackedW8Weight, gate_up_lora: PackedLoRA | None,
                   down_weight: PackedW8Weight, down_lora: PackedLoRA | None, adapter_ids=None, *, residual=None,
                   enabled: bool = False, eps: float = RMS_EPS, out=None, down_epilogue: int = EPI_RESIDUAL,
                   timing_events=None, return_call: bool = False, reuse_routing: bool = False, chunk=None,
                   gemm_cta_limit: int = 0, input_prepared: bool = False, prepare_rows=None, scatter=None,
                   row_amax_from_epilogue: bool = True, keep_normalized: bool = False, build_only: bool = False,
                   fused_rows: bool = False, gemm_variant: int = 0, prefetch_next: PackedW8Weight | None = None,
                   prefetch_bytes: int = 0):
    """One MLP block, out = residual + down(swiglu(gate_up(rmsnorm(x)))), with
    the adapter routing computed once and h kept on the device in sorted row
    order (qwen3_5.py:786-826).  Takes packed weights and tables only.

    Sequence-parallel callers split the call: `prepare_rows=(row_begin, row_count)`
    runs only the stage in front of the gate_up GEMM (RMSNorm, codes, scales,
    LoRA-A projection) for those sorted rows and returns the call handle;
    `input_prepared=True` runs the rest on a workspace whose regions
    (`w8a8_mlp_workspace_regions`) already hold that stage's results.
    `scatter=(rows_per_owner, [address of owner 0's slab, ...])` makes the down
    GEMM store each owner's rows of the fp32 partial sums straight into that
    owner's slab (device addresses, possibly peer mappings) instead of `out`.
    `row_amax_from_epilogue=False` makes the quantiser of h find the row absmax itself (a cross-check:
    both forms give identical bits); `fused_rows=True` makes small batches (at most 128 rows) finish each
    projection in the GEMM's own epilogue instead of a second row-wise kernel (same bits, one launch fewer;
    slower on B200 at decode shapes, so not the default).  `build_only=True` validates and returns the call handle without
    enqueuing anything (the handle of the NEXT block is an argument of `w8a8_mlp_tp_exchange`).
    `prefetch_bytes > 0` (small batches only) makes each GEMM ask up to that many leading bytes of the NEXT
    GEMM's weights into L2 once its own loads are out — the down weights behind gate_up, and behind down the
    gate_up weights of `prefetch_next` (the following block) — so that HBM keeps delivering during the
    row-wise kernels between two GEMMs; it changes no value."""
    _validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 MLP block is disabled by default")
    if not isinstance(gate_up_weight, PackedW8Weight) or not isinstance(down_weight, PackedW8Weight):
        raise TypeError("w8a8_mlp_block takes PackedW8Weight weights")
    hidden, two_i = gate_up_weight.in_features, gate_up_weight.padded_out_features
    inter = two_i // 2
    if gate_up_weight.out_features != two_i or down_weight.out_features != down_weight.padded_out_features:
        raise ValueError("w8a8_mlp_block needs feature sizes that are multiples of 32")
    if down_weight.in_features != inter or down_weight.out_features != hidden:
        raise ValueError("down weight does not match gate_up weight")
    x2 = _check_x(x, hidden)
    x2 = _pad_cols(x2, hidden)
    m = x2.shape[0]
    if (gate_up_lora is None) != (down_lora is None):
        raise ValueError("give LoRA tables for both projections or for neither")
    ids = _check_ids(adapter_ids, m, gate_up_lora)
    delta = _pad_delta(rms_delta, hidden, hidden) if rms_delta is not None else None
    lib = _lib.load()
    dev = x2.device
    na = gate_up_lora.num_adapters if gate_up_lora is not None else 1
    nbytes = lib.skyrl_w8a8_mlp_workspace_bytes(m, hidden, inter, na)
    ws = _workspace(dev, nbytes)
    st = _status_word(dev)
    if out is None:
        out = torch.empty((m, hidden), dtype=torch.float32 if down_epilogue == EPI_PARTIAL_F32 else torch.bfloat16,
                          device=dev)
    a = _lib.MlpArgs()
    a.struct_size = C.sizeof(_lib.MlpArgs)
    a.m, a.hidden, a.inter = m, hidden, inter
    a.rank = gate_up_lora.rank if gate_up_lora is not None else 0
    a.num_adapters = na
    a.down_epilogue = down_epilogue
    a.rms_eps = float(eps)
    a.x = x2.data_ptr()
    a.rms_delta = delta.data_ptr() if delta is not None else None
    r2 = None
    if residual is not None:
        r2 = _pad_cols(residual.reshape(-1, residual.shape[-1]), hidden)
        a.residual = r2.data_ptr()
    a.gu_wq, a.gu_sw = gate_up_weight.wq.data_ptr(), gate_up_weight.sw.data_ptr()
    a.dn_wq, a.dn_sw = down_weight.wq.data_ptr(), down_weight.sw.data_ptr()
    if gate_up_lora is not None:
        if gate_up_lora.rank != down_lora.rank or gate_up_lora.num_adapters != down_lora.num_adapters:
            raise ValueError("gate_up and down LoRA tables must share rank and adapter count")
        a.gu_a_packed, a.gu_b_packed = gate_up_lora.a.data_ptr(), gate_up_lora.b.data_ptr()
        a.gu_scaling = gate_up_lora.scaling.data_ptr()
        a.dn_a_packed, a.dn_b_packed = down_lora.a.data_ptr(), down_lora.b.data_ptr()
        a.dn_scaling = down_lora.scaling.data_ptr()
        if gate_up_lora.b_rows is not None and down_lora.b_rows is not None:
            a.gu_b_rows, a.dn_b_rows = gate_up_lora.b_rows.data_ptr(), down_lora.b_rows.data_ptr()
            a.b_rows_rank = gate_up_lora.b_rows.shape[2]
    a.adapter_ids = ids.data_ptr() if ids is not None else None
    a.out = out.data_ptr()
    a.workspace = ws.data_ptr()
    a.workspace_bytes = nbytes
    a.status = st.data_ptr()
    if timing_events is not None:
        for i, ev in enumerate(timing_events):
            a.timing_events[i] = ev.cuda_event
    if reuse_routing:
        a.flags |= _lib.MLP_REUSE_ROUTING
    if input_prepared:
        a.flags |= _lib.MLP_INPUT_PREPARED
    if not row_amax_from_epilogue:
        a.flags |= _lib.MLP_NO_ROW_AMAX
    if keep_normalized:
        a.flags |= _lib.MLP_KEEP_NORMALIZED
    if fused_rows:
        a.flags |= _lib.MLP_FUSED_ROWS
    a.flags |= int(gemm_variant) << _lib.FLAGS_GEMM_VARIANT_SHIFT
    if chunk is not None:
        a.chunk_index, a.num_chunks = int(chunk[0]), int(chunk[1])
    a.gemm_cta_limit = int(gemm_cta_limit)
    if prefetch_bytes > 0:
        a.prefetch_down_bytes = int(prefetch_bytes) // 16 * 16
        if prefetch_next is not None:
            a.prefetch_next = prefetch_next.wq.data_ptr()
            a.prefetch_next_bytes = min(int(prefetch_bytes), prefetch_next.wq.numel()) // 16 * 16
    if scatter is not None:
        a.tp_scatter_rows = int(scatter[0])
        if len(scatter[1]) > 8:
            raise ValueError("at most 8 scatter owners")
        for i, addr in enumerate(scatter[1]):
            a.tp_scatter_bases[i] = int(addr)
    if build_only:
        return out, (a, x2, delta, ids, r2)
    if prepare_rows is not None:
        _lib.check(lib.skyrl_w8a8_mlp_tp_prepare_sm100_v1(C.byref(a), int(prepare_rows[0]), int(prepare_rows[1]),
                                                        _stream()), "w8a8_mlp_tp_prepare")
        return out, (a, x2, delta, ids, r2)
    _lib.check(lib.skyrl_w8a8_mlp_block_sm100_v1(C.byref(a), _stream()), "w8a8_mlp_block")
    if return_call:
        # keeps the argument block (and through it the workspace layout) for the tensor-parallel finalize
        return out, (a, x2, delta, ids, r2)
    return out.reshape(*x.shape[:-1], hidden) if out.shape[0] == m else out


def chunk_rows(m: int, num_chunks: int) -> int:
    """Rows per chunk of a chunked MLP block call: ceil(m / num_chunks) rounded up to the 128-row tile."""
    per = (m + num_chunks - 1) // num_chunks
    return (per + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS


def w8a8_mlp_tp_finalize(call, reduced: torch.Tensor, out: torch.Tensor, row_begin: int = 0,
                         row_count: int | None = None, *, sorted_out: bool = False):
    """Second half of a row-parallel block: out[perm[i]] = bf16(bf16(reduced[i]) + residual[perm[i]]).

    `call` is the handle returned by `w8a8_mlp_block(..., down_epilogue=EPI_PARTIAL_F32, return_call=True)`;
    `reduced` is the reduced fp32 [M, H] partial-sum buffer in adapter-sorted row order.  With
    `sorted_out` row i goes to out[i] instead (a later `w8a8_mlp_tp_unsort` restores token order)."""
    a = call[0]
    lib = _lib.load()
    if row_count is None:
        row_count = a.m - row_begin
    flags = a.flags
    a.flags = (flags | _lib.MLP_FINALIZE_SORTED) if sorted_out else (flags & ~_lib.MLP_FINALIZE_SORTED)
    try:
        _lib.check(lib.skyrl_w8a8_mlp_tp_finalize_sm100_v1(C.byref(a), _ptr(reduced), _ptr(out), row_begin, row_count,
                                                         _stream()), "w8a8_mlp_tp_finalize")
    finally:
        a.flags = flags
    return out


def w8a8_mlp_tp_finalize_slabs(call, slab_addresses, out: torch.Tensor, row_begin: int, row_count: int, *,
                               sorted_out: bool = False):
    """Finalize rows whose partial sums were scattered to this rank and not yet added: slab s (a device
    address) holds rank s's fp32 sums of sorted rows [row_begin, row_begin + row_count); the slabs are added
    in ascending s, then as `w8a8_mlp_tp_finalize`."""
    a = call[0]
    lib = _lib.load()
    ptrs = (C.c_void_p * len(slab_addresses))(*[int(p) for p in slab_addresses])
    flags = a.flags
    a.flags = (flags | _lib.MLP_FINALIZE_SORTED) if sorted_out else (flags & ~_lib.MLP_FINALIZE_SORTED)
    try:
        _lib.check(lib.skyrl_w8a8_mlp_tp_finalize_slabs_sm100_v1(C.byref(a), ptrs, len(slab_addresses), _ptr(out),
                                                               row_begin, row_count, _stream()),
                   "w8a8_mlp_tp_finalize_slabs")
    finally:
        a.flags = flags
    return out


def w8a8_mlp_tp_exchange(call, next_call, out: torch.Tensor, *, tp: int, row_begin: int, row_count: int, partials,
                         wait_flags=None, wait_value: int = 0, peer_workspaces=None, signal_flags=None,
                         signal_value: int = 0, sorted_out: bool = False, grid_ctas: int = 0, single_kernel: bool = False,
                         multimem: bool = False, profile: bool = False, wide: bool = False):
    """Fused exchange between two blocks of a sequence-parallel stack (one kernel per rank and row chunk).

    `call` is the handle of the `w8a8_mlp_block(..., down_epilogue=EPI_PARTIAL_F32, return_call=True)` call that
    produced this rank's partial sums, `next_call` the handle of the next block's call on the same chunk
    (`build_only=True`; None behind the last block).  `partials` lists every rank's partial-sum buffer as a
    device address (own buffer and peer mappings), `peer_workspaces` every rank's workspace base address,
    `wait_flags` an int32 tensor of `tp` words in this rank's memory that the ranks raise to `wait_value` when
    their partial sums are complete, `signal_flags` one flag address per rank that this call sets to
    `signal_value` once the rows it prepared have been stored everywhere.  `single_kernel=True` selects the
    one-kernel form (same bits; the default is a streaming sum kernel followed by the row-wise quantiser).
    `multimem=True`: `partials[0]` is the multicast address of a symmetric buffer holding every rank's partial
    sums; the sum is then formed inside NVSwitch (agrees with the other forms to fp32 rounding)."""
    a = call[0]
    lib = _lib.load()
    x = _lib.TpExchangeArgs()
    x.struct_size = C.sizeof(_lib.TpExchangeArgs)
    x.tp, x.row_begin, x.row_count = int(tp), int(row_begin), int(row_count)
    x.wait_value, x.signal_value, x.grid_ctas = int(wait_value), int(signal_value), int(grid_ctas)
    x.flags = (_lib.TP_EXCHANGE_SINGLE_KERNEL if single_kernel else 0) | (_lib.TP_EXCHANGE_MULTIMEM if multimem else 0) | (_lib.TP_EXCHANGE_PROFILE if profile else 0) | (_lib.TP_EXCHANGE_WIDE if wide else 0)
    if len(partials) != (1 if multimem else tp):
        raise ValueError(f"{1 if multimem else tp} partial-sum buffers wanted, got {len(partials)}")
    for s_, addr in enumerate(partials):
        x.partials[s_] = int(addr)
    x.wait_flags = wait_flags.data_ptr() if wait_flags is not None else None
    if next_call is not None:
        if peer_workspaces is None or len(peer_workspaces) != tp:
            raise ValueError(f"{tp} workspace addresses wanted for the next block")
        for r, addr in enumerate(peer_workspaces):
            x.peer_workspaces[r] = int(addr)
    if signal_flags is not None:
        for r, addr in enumerate(signal_flags):
            x.signal_flags[r] = int(addr) if addr else None
    x.out = out.data_ptr()
    flags = a.flags
    a.flags = (flags | _lib.MLP_FINALIZE_SORTED) if sorted_out else (flags & ~_lib.MLP_FINALIZE_SORTED)
    try:
        _lib.check(lib.skyrl_w8a8_mlp_tp_exchange_sm100_v1(C.byref(a), C.byref(next_call[0]) if next_call is not None else None,
                                                         C.byref(x), _stream()), "w8a8_mlp_tp_exchange")
    finally:
        a.flags = flags
    return out


def tp_signal(flag_addresses, value: int) -> None:
    """After the work enqueued so far on the current stream: set the flag words at `flag_addresses` (device
    addresses, possibly in other ranks' memory; None entries are skipped) to `value`."""
    ptrs = (C.c_void_p * len(flag_addresses))(*[int(p) if p else None for p in flag_addresses])
    _lib.check(_lib.load().skyrl_w8a8_tp_signal_sm100_v1(ptrs, len(flag_addresses), int(value), _stream()), "tp_signal")


def tp_wait(flags: torch.Tensor, count: int, value: int) -> None:
    """Hold the current stream until `count` int32 flag words of `flags` (this rank's memory) have reached
    `value`; bounded (status 105 after 2 s, reported by `check_status`)."""
    st = _status_word(flags.device)
    _lib.check(_lib.load().skyrl_w8a8_tp_wait_sm100_v1(flags.data_ptr(), int(count), int(value), st.data_ptr(), _stream()),
               "tp_wait")


def w8a8_mlp_tp_unsort(call, sorted_rows: torch.Tensor, out: torch.Tensor):
    """out[perm[i]] = sorted_rows[i]: bf16 [M, H] rows from adapter-sorted back to token order."""
    _lib.check(_lib.load().skyrl_w8a8_mlp_tp_unsort_sm100_v1(C.byref(call[0]), _ptr(sorted_rows), _ptr(out), _stream()),
               "w8a8_mlp_tp_unsort")
    return out


def w8a8_mlp_workspace_regions(m: int, hidden: int, inter: int, num_adapters: int, device):
    """Views of the workspace regions a sequence-parallel gather moves, indexed by sorted row:
    (codes int8 [m, hidden], scales fp32 [m], LoRA-A parts bf16 [m, 384])."""
    lib = _lib.load()
    na = max(int(num_adapters), 1)
    ws = _workspace(device, lib.skyrl_w8a8_mlp_workspace_bytes(m, hidden, inter, na))
    off = (C.c_size_t * 3)()
    _lib.check(lib.skyrl_w8a8_mlp_workspace_regions(m, hidden, inter, na, off), "w8a8_mlp_workspace_regions")
    xq = ws[off[0]: off[0] + m * hidden].view(torch.int8).view(m, hidden)
    sx = ws[off[1]: off[1] + 4 * m].view(torch.float32)
    z = ws[off[2]: off[2] + m * Z_PARTS * LORA_RANK_PAD * 2].view(torch.bfloat16).view(m, Z_PARTS * LORA_RANK_PAD)
    return xq, sx, z


def w8a8_mlp_stage_regions(m: int, hidden: int, inter: int, num_adapters: int, device):
    """Views of what the last `w8a8_mlp_block` call of these sizes left in the workspace, for stage-by-stage
    checks: (perm int32 [m], h bf16 [m, inter], codes of h int8 [m, inter], scales of h fp32 [m],
    rmsnorm(x) bf16 [m, hidden]).  h, its codes and the normalised rows are in the GEMM's row order:
    adapter-sorted (row i = token perm[i]) for m > 128 with adapter ids, token order otherwise (small
    batches store the normalised rows only when the block ran with `keep_normalized=True`)."""
    lib = _lib.load()
    na = max(int(num_adapters), 1)
    ws = _workspace(device, lib.skyrl_w8a8_mlp_workspace_bytes(m, hidden, inter, na))
    off = (C.c_size_t * 5)()
    _lib.check(lib.skyrl_w8a8_mlp_workspace_stage_regions(m, hidden, inter, na, off), "w8a8_mlp_workspace_stage_regions")
    perm = ws[off[0]: off[0] + 4 * m].view(torch.int32)
    h = ws[off[1]: off[1] + 2 * m * inter].view(torch.bfloat16).view(m, inter)
    hq = ws[off[2]: off[2] + m * inter].view(torch.int8).view(m, inter)
    sh = ws[off[3]: off[3] + 4 * m].view(torch.float32)
    xn = ws[off[4]: off[4] + 2 * m * hidden].view(torch.bfloat16).view(m, hidden)
    return perm, h, hq, sh, xn


# --------------------------------------------------------------------------- #
# stage-level entry points (used by the parity tests)
# --------------------------------------------------------------------------- #
def prepare_routing(adapter_ids, m: int, num_adapters: int):
    """Device statement of prepare_routing (layers/util.py:66-87): returns
    (perm int32 [m], tiles int32 [T, 4], num_tiles int32 [1])."""
    lib = _lib.load()
    dev = adapter_ids.device if adapter_ids is not None else torch.device("cuda", torch.cuda.current_device())
    max_tiles = (m + TILE_ROWS - 1) // TILE_ROWS + max(num_adapters, 1)
    perm = torch.empty(m, dtype=torch.int32, device=dev)
    tiles = torch.zeros((max_tiles, 4), dtype=torch.int32, device=dev)
    num = torch.zeros(4, dtype=torch.int32, device=dev)
    st = _status_word(dev)
    _lib.check(lib.skyrl_lora_route_sm100_v1(_ptr(adapter_ids), m, num_adapters, _ptr(perm), _ptr(tiles), _ptr(num),
                                             max_tiles, _ptr(st), _stream()), "lora_route")
    return perm, tiles, num


def rms_quant(x, rms_delta=None, *, eps: float = RMS_EPS, row_map=None, want_normalized: bool = False):
    """RMSNorm (optional) + per-token int8 quantisation: returns (codes int8
    [M, K], scales fp32 [M], normalised bf16 [M, K] or None)."""
    lib = _lib.load()
    _require_cuda(x, "x")
    m, k = x.shape
    xq = torch.empty((m, k), dtype=torch.int8, device=x.device)
    sx = torch.empty((m,), dtype=torch.float32, device=x.device)
    xn = torch.empty((m, k), dtype=torch.bfloat16, device=x.device) if want_normalized else None
    _lib.check(lib.skyrl_rms_quant_sm100_v1(_ptr(x), x.stride(0), _ptr(rms_delta), float(eps), _ptr(row_map), m, k,
                                            _ptr(xq), _ptr(sx), _ptr(xn), _stream()), "rms_quant")
    return xq, sx, xn
