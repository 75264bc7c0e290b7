"""Load -> quantise -> pack pipeline of the MLP weights, with an in-memory and an on-disk cache.

What the reference does when it builds the model, restated for this library's device format:

* checkpoints store `gate_proj`, `up_proj` and `down_proj` as `[out, in]` matrices; the model fuses gate and
  up into ONE projection whose physical output columns interleave them, (gate0, up0, gate1, up1, ...)
  (`_fuse_checkpoint_arrays_numpy` with group sizes (1, 1), skyrl/tx/utils/models.py:159-215, called from
  `load_safetensors`, :329-340; the runtime twin is `FusedLoRALinear.fuse`, skyrl/tx/layers/lora.py:318-336);
* the frozen matrices are quantised once, per output channel, by `quantize_frozen_weight`
  (skyrl/tx/kernels/quantized_lora.py:128-171);
* a native kernel wants its weight in ONE canonical device layout prepared at load time, not re-derived per
  call (rocm/QUANTIZED_FFI.md:69-74).

The canonical layout here is `PackedW8Weight` (int8 `[ceil(K/128), N, 128]`, fp32 scales).  Everything in this
file is pure indexing on whatever device the tensors live on, except `pack_weight`, which runs the library's
pack kernel for CUDA tensors; `pack_weight_host` / `unpack_weight` are its host statements (the same bytes),
used for the cache file and for the pack-unpack identity test.
"""

from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass

import torch

from . import ops
from ._cache import IdentityCache  # noqa: F401  (re-exported: the memo the operators use for per-call conversions)
from ._lib import WEIGHT_KBLOCK

FORMAT_VERSION = 1


# --------------------------------------------------------------------------- #
# fuse / split of gate and up (checkpoint <-> model layout)
# --------------------------------------------------------------------------- #
def fuse_gate_up(gate_kn: torch.Tensor, up_kn: torch.Tensor) -> torch.Tensor:
    """[K, I] gate and [K, I] up -> [K, 2I] with interleaved columns (gate0, up0, gate1, up1, ...): the
    reference's fused layout for group sizes (1, 1) (skyrl/tx/utils/models.py:159-215)."""
    if gate_kn.shape != up_kn.shape or gate_kn.ndim < 1:
        raise ValueError(f"gate and up must have the same shape, got {tuple(gate_kn.shape)} and {tuple(up_kn.shape)}")
    return torch.stack((gate_kn, up_kn), dim=-1).reshape(*gate_kn.shape[:-1], 2 * gate_kn.shape[-1])


def split_gate_up(fused_kn: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of `fuse_gate_up` (FusedLoRALinear.split, skyrl/tx/layers/lora.py:338-351)."""
    if fused_kn.shape[-1] % 2:
        raise ValueError("a fused gate/up projection has an even number of columns")
    return fused_kn[..., 0::2], fused_kn[..., 1::2]


# --------------------------------------------------------------------------- #
# host statements of the packed layout
# --------------------------------------------------------------------------- #
def pack_weight_host(codes_kn: torch.Tensor) -> torch.Tensor:
    """int8 [K, N] -> int8 [ceil(K / 128), N, 128] (K zero-padded to the block), by indexing only: byte for byte
    what skyrl_pack_weight_kn_sm100_v1 writes."""
    if codes_kn.ndim != 2 or codes_kn.dtype != torch.int8:
        raise TypeError("W8 codes must be a rank-two INT8 array")
    k, n = codes_kn.shape
    kb = (k + WEIGHT_KBLOCK - 1) // WEIGHT_KBLOCK
    padded = torch.zeros((kb * WEIGHT_KBLOCK, n), dtype=torch.int8, device=codes_kn.device)
    padded[:k] = codes_kn
    return padded.view(kb, WEIGHT_KBLOCK, n).permute(0, 2, 1).contiguous()


def unpack_weight(packed: ops.PackedW8Weight) -> ops.GroupQuantizedWeight:
    """The reference's storage (codes int8 [K, N], scales bf16 [groups, N]) back from the device format.
    pack(unpack(w)) == w and unpack(pack(q)) == q for every weight the operators accept."""
    kb, npad, blk = packed.wq.shape
    codes = packed.wq.permute(0, 2, 1).reshape(kb * blk, npad)[: packed.in_features, : packed.out_features].contiguous()
    sw = packed.sw if packed.group_size else packed.sw[None]
    scales = sw[:, : packed.out_features].to(torch.bfloat16).contiguous()
    group = packed.group_size or packed.in_features
    return ops.GroupQuantizedWeight(codes, scales, packed.in_features, packed.in_features, 8, group)


# --------------------------------------------------------------------------- #
# packed MLP weights + caches
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class PackedMLPWeights:
    """The frozen weights of one MLP block in device format (gate_up interleaved, down)."""

    gate_up: ops.PackedW8Weight
    down: ops.PackedW8Weight

    @property
    def hidden_size(self) -> int:
        return self.gate_up.in_features

    @property
    def intermediate_size(self) -> int:
        return self.gate_up.out_features // 2


def quantize_and_pack_mlp(gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor, *,
                          tp: int = 1, rank: int = 0) -> PackedMLPWeights:
    """Checkpoint matrices (`[out, in]`: gate/up `[I, H]`, down `[H, I]`, on a CUDA device) -> packed W8 weights
    of tensor-parallel rank `rank` of `tp`.

    gate_up is sharded on (gate, up) PAIRS of output columns and down on input features, as the reference's
    sharding specs do (skyrl/tx/models/qwen3_5.py:633,644); the down shard is quantised over its own K slice
    (the reference's group format with group_size = I / tp)."""
    from .tp import shard_bounds

    if gate_proj.shape != up_proj.shape or gate_proj.ndim != 2:
        raise ValueError("gate_proj and up_proj must be [I, H] matrices of the same shape")
    inter, hidden = gate_proj.shape
    if down_proj.shape != (hidden, inter):
        raise ValueError(f"down_proj must be [{hidden}, {inter}], got {tuple(down_proj.shape)}")
    lo, hi = shard_bounds(inter, tp, rank)
    fused_kn = fuse_gate_up(gate_proj[lo:hi].t(), up_proj[lo:hi].t())            # [H, 2 I/tp]
    down_kn = down_proj[:, lo:hi].t().contiguous()                                # [I/tp, H]
    gate_up = ops.pack_weight(ops.quantize_frozen_weight(fused_kn.contiguous()))
    down = ops.pack_weight(ops.quantize_frozen_weight(down_kn))
    return PackedMLPWeights(gate_up, down)


def tensor_digest(*tensors: torch.Tensor) -> str:
    """Content key of source tensors for the on-disk cache (SHA-256 of shapes, dtypes and bytes)."""
    h = hashlib.sha256()
    h.update(f"skyrl-w8-pack-v{FORMAT_VERSION}".encode())
    for t in tensors:
        c = t.detach().contiguous().cpu()
        h.update(f"{tuple(c.shape)}:{c.dtype}".encode())
        h.update(c.view(torch.uint8).numpy().tobytes() if c.dtype != torch.bfloat16 else c.view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def save_packed_weight(path: str | os.PathLike, packed: ops.PackedW8Weight) -> None:
    """Write the reference storage of a packed weight (codes [K, N] + bf16 scales + meta): the device layout
    is reproduced from it exactly by `load_packed_weight`, on any device."""
    q = unpack_weight(packed)
    meta = {"format": FORMAT_VERSION, "in_features": packed.in_features, "out_features": packed.out_features,
            "group_size": packed.group_size, "padded_out_features": packed.padded_out_features}
    tmp = f"{os.fspath(path)}.tmp{os.getpid()}"
    torch.save({"meta": json.dumps(meta), "codes": q.codes.cpu(), "scales": q.scales.cpu().view(torch.int16)}, tmp)
    os.replace(tmp, path)   # readers never see a half-written file


def load_packed_weight(path: str | os.PathLike, device=None) -> ops.PackedW8Weight:
    blob = torch.load(path, map_location="cpu", weights_only=True)
    meta = json.loads(blob["meta"])
    if meta.get("format") != FORMAT_VERSION:
        raise ValueError(f"{path}: packed-weight format {meta.get('format')} is not {FORMAT_VERSION}")
    codes, scales = blob["codes"], blob["scales"].view(torch.bfloat16)
    k, n = meta["in_features"], meta["out_features"]
    npad = meta["padded_out_features"]
    group = meta["group_size"] or k
    if device is not None and torch.device(device).type == "cuda":
        gq = ops.GroupQuantizedWeight(codes.to(device), scales.to(device), k, k, 8, group)
        return ops.pack_weight(gq)
    padded = torch.zeros((codes.shape[0], npad), dtype=torch.int8)
    padded[:, :n] = codes
    sw = torch.zeros((scales.shape[0], npad), dtype=torch.float32)
    sw[:, :n] = scales.float()
    return ops.PackedW8Weight(pack_weight_host(padded), sw if meta["group_size"] else sw[0], k, n, meta["group_size"])


class PackedWeightCache:
    """On-disk cache of packed weights keyed by the content of their source tensors: quantising and packing a
    checkpoint happens once per (weights, sharding), later loads read the int8 codes back."""

    def __init__(self, directory: str | os.PathLike):
        self.directory = os.fspath(directory)
        os.makedirs(self.directory, exist_ok=True)
        self.hits = 0
        self.misses = 0

    def path(self, key: str) -> str:
        return os.path.join(self.directory, f"{key}.w8pack")

    def get_or_build(self, key: str, build, device=None) -> ops.PackedW8Weight:
        p = self.path(key)
        if os.path.exists(p):
            self.hits += 1
            return load_packed_weight(p, device)
        self.misses += 1
        packed = build()
        save_packed_weight(p, packed)
        return packed

    def mlp(self, gate_proj, up_proj, down_proj, *, tp: int = 1, rank: int = 0) -> PackedMLPWeights:
        key = tensor_digest(gate_proj, up_proj, down_proj)
        built: dict = {}

        def build(which):
            if not built:
                w = quantize_and_pack_mlp(gate_proj, up_proj, down_proj, tp=tp, rank=rank)
                built.update(gate_up=w.gate_up, down=w.down)
            return built[which]

        dev = gate_proj.device
        return PackedMLPWeights(self.get_or_build(f"{key}-gate_up-tp{tp}r{rank}", lambda: build("gate_up"), dev),
                                self.get_or_build(f"{key}-down-tp{tp}r{rank}", lambda: build("down"), dev))
