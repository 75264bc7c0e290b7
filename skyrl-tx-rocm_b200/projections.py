"""The other LoRA-bearing projections of a decoder layer on the W8A8 kernels.

The MLP is not the only place the reference applies `base + LoRA`: the attention block's fused `qkv_proj`
(components q / k / v interleaved per key-value group) and its `o_proj` are the same `LoRALinear` /
`FusedLoRALinear` layers (skyrl/tx/models/qwen3_5.py:326-350; call sites :365 and :384), as are the linear
attention block's `in_proj_*` / `out_proj` (:548-601).  They take the same operator, `w8a8_lora_linear`, and
the same split of fused columns (`FusedLoRALinear.split`, skyrl/tx/layers/lora.py:338-351).
"""

from __future__ import annotations

import torch

from . import ops


def fuse_components(arrays, group_sizes) -> torch.Tensor:
    """Interleave per-component arrays (last axis) into the fused layout: for every group g the columns
    [component 0's group g | component 1's group g | ...] (FusedLoRALinear.fuse, skyrl/tx/layers/lora.py:324-336;
    the checkpoint-side twin is _fuse_checkpoint_arrays_numpy, skyrl/tx/utils/models.py:159-193)."""
    arrays = list(arrays)
    if len(arrays) != len(group_sizes) or not arrays:
        raise ValueError(f"expected one nonempty array per group size, got {len(arrays)} and {len(group_sizes)}")
    if any(g <= 0 for g in group_sizes):
        raise ValueError(f"group sizes must all be positive, got {tuple(group_sizes)}")
    batch = arrays[0].shape[:-1]
    if arrays[0].shape[-1] % group_sizes[0]:
        raise ValueError(f"last dim {arrays[0].shape[-1]} is not divisible by first group size {group_sizes[0]}")
    groups = arrays[0].shape[-1] // group_sizes[0]
    parts = []
    for arr, g in zip(arrays, group_sizes):
        if arr.shape[:-1] != batch or arr.shape[-1] != groups * g:
            raise ValueError(f"array of shape {tuple(arr.shape)} does not hold {groups} groups of {g}")
        parts.append(arr.reshape(*batch, groups, g))
    return torch.cat(parts, dim=-1).reshape(*batch, -1)


def split_components(fused: torch.Tensor, group_sizes) -> tuple[torch.Tensor, ...]:
    """Inverse of `fuse_components` (FusedLoRALinear.split, skyrl/tx/layers/lora.py:338-351)."""
    total, gs = fused.shape[-1], sum(group_sizes)
    if total % gs:
        raise ValueError(f"last dim {total} not divisible by sum(group_sizes)={gs}")
    groups = total // gs
    view = fused.reshape(*fused.shape[:-1], groups, gs)
    out, off = [], 0
    for g in group_sizes:
        out.append(view[..., off:off + g].reshape(*fused.shape[:-1], groups * g))
        off += g
    return tuple(out)


class LoRALinearW8:
    """`LoRALinear.__call__(x, adapter_indices)` (skyrl/tx/layers/lora.py:270-272) on a W8 (or W4) frozen weight:
    y = bf16(dequant(xq wq^T) + s[a] (x A[a]) B[a]) per token."""

    def __init__(self, weight, lora: ops.PackedLoRA | None = None, *, enabled: bool = False):
        if type(enabled) is not bool:
            raise TypeError("enabled must be an exact bool")
        self.weight = ops._weight_of(weight) if enabled and not isinstance(weight, ops.PackedW8Weight) else weight
        self.lora = lora
        self.enabled = enabled

    def _token_ids(self, x, adapter_indices):
        if adapter_indices is None:
            return None
        tokens = x.numel() // x.shape[-1]
        if adapter_indices.numel() == tokens:
            return adapter_indices.reshape(-1).contiguous()
        if x.ndim >= 3 and adapter_indices.shape == (x.shape[0],):
            return adapter_indices.repeat_interleave(tokens // x.shape[0]).contiguous()
        raise ValueError(f"adapter_indices of shape {tuple(adapter_indices.shape)} match neither sequences nor tokens")

    def __call__(self, x, adapter_indices=None):
        if not self.enabled:
            raise RuntimeError("the W8A8 LoRA projection is disabled by default")
        ids = self._token_ids(x, adapter_indices)
        if self.lora is None:
            return ops.w8a8_frozen_linear(x, self.weight, enabled=True)
        return ops.w8a8_lora_linear(x, self.weight, self.lora, adapter_ids=ids, enabled=True)


class FusedLoRALinearW8(LoRALinearW8):
    """`FusedLoRALinear.__call__` (skyrl/tx/layers/lora.py:313-316): one projection, split into its components.
    For attention: components (q, k, v) with group sizes (q_per_kv * 2 * head_dim, head_dim, head_dim)
    (skyrl/tx/models/qwen3_5.py:326-338)."""

    def __init__(self, weight, lora=None, *, components, group_sizes, enabled: bool = False):
        super().__init__(weight, lora, enabled=enabled)
        if len(components) != len(group_sizes):
            raise ValueError("one group size per component")
        self.components = tuple(components)
        self.group_sizes = tuple(int(g) for g in group_sizes)

    def __call__(self, x, adapter_indices=None):
        return split_components(super().__call__(x, adapter_indices), self.group_sizes)
