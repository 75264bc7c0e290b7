"""Model wiring: an MLP module shaped like the reference's `Qwen3_5MLP` / `Qwen3MLP` that routes to the
W8A8 multi-LoRA kernels.

The reference's module owns a fused `gate_up_proj` and a `down_proj`, is called by the decoder layer either as
`mlp(norm(x), adapter_indices=..., residual=...)` or as `mlp.forward_with_post_attention_rms(x, norm,
adapter_indices=..., residual=...)`, and chooses a fused kernel through selector predicates that fall back to
the plain path whenever a geometry is not qualified (skyrl/tx/models/qwen3_5.py:605-826, decoder call
:882-896; Qwen3: skyrl/tx/models/qwen3.py:100-131, :297-303).  The flag that arms a fused path lives in the
backend configuration and is validated there (skyrl/backends/jax.py:126-204).

Here the same three pieces exist for the W8A8 path:

* `W8A8BackendConfig`    the flag and its validation (mesh / rank / adapter limits),
* selector predicates    `_can_use_w8a8_mlp_block`, `_can_use_w8a8_rms_gate_up_swiglu`,
                         `_can_use_w8a8_down_residual`, each a pure function of shapes, dtypes and the flag,
* `Qwen3_5MLP`           `forward_with_post_attention_rms` / `__call__` that pick, in this order: the whole
                         block in one call (`ops.w8a8_mlp_block`), the two fused halves
                         (`ops.w8a8_rms_gate_up_lora_swiglu` + `ops.w8a8_down_lora_residual`), or those halves
                         behind a separate norm pass; with a tensor-parallel group, this rank's shard of the
                         block and one all-reduce (`tp.TensorParallelMLP`).

Unlike the reference's prototypes the predicates accept any batch, any rank up to 64, any number of adapters
and a tensor-parallel group; what they still reject (odd feature sizes, wrong dtypes, a missing norm weight)
falls back to the next path, and a disabled flag raises like every operator of this library.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops
from .weights import PackedMLPWeights


@dataclass(frozen=True)
class W8A8BackendConfig:
    """Backend switches of the W8A8 path (the counterpart of the reference's `qwen35_*` options)."""

    w8a8_mlp: bool = False                # arm the fused W8A8 MLP path at all
    max_lora_adapters: int = 1
    max_lora_rank: int = 8
    tensor_parallel_size: int = 1
    rms_norm_eps: float = 1e-6

    def __post_init__(self):
        if type(self.w8a8_mlp) is not bool:
            raise TypeError("w8a8_mlp must be an exact bool")
        if self.max_lora_rank < 0 or self.max_lora_rank > ops.MAX_LORA_RANK:
            raise ValueError(f"w8a8_mlp supports LoRA ranks up to {ops.MAX_LORA_RANK}, got {self.max_lora_rank}")
        if self.max_lora_adapters < 0 or self.max_lora_adapters > 4096:
            raise ValueError(f"w8a8_mlp supports up to 4096 adapters, got {self.max_lora_adapters}")
        if self.tensor_parallel_size < 1 or self.tensor_parallel_size > 8:
            raise ValueError(f"w8a8_mlp is qualified for 1 to 8 tensor-parallel ranks, got {self.tensor_parallel_size}")


def _is_device_tensor(t) -> bool:
    return isinstance(t, torch.Tensor) and t.is_cuda


class RMSNormWeights:
    """What the MLP needs of the layer norm in front of it: the (1 + delta) weight and eps
    (Qwen3_5RMSNorm, skyrl/tx/models/qwen3_5.py:259-278)."""

    def __init__(self, weight: torch.Tensor, eps: float = 1e-6):
        self.weight = weight
        self.eps = eps


class Qwen3_5MLP:
    """RMSNorm -> gate_up (W8A8 + LoRA) -> SwiGLU -> down (W8A8 + LoRA) (+ residual)."""

    def __init__(self, config: W8A8BackendConfig, weights: PackedMLPWeights, gate_up_lora: ops.PackedLoRA | None,
                 down_lora: ops.PackedLoRA | None, *, tp_group=None):
        if (gate_up_lora is None) != (down_lora is None):
            raise ValueError("give LoRA tables for both projections or for neither")
        if gate_up_lora is not None and gate_up_lora.rank > config.max_lora_rank:
            raise ValueError(f"LoRA rank {gate_up_lora.rank} exceeds max_lora_rank={config.max_lora_rank}")
        if gate_up_lora is not None and gate_up_lora.num_adapters > max(config.max_lora_adapters, 1):
            raise ValueError(f"{gate_up_lora.num_adapters} adapters exceed max_lora_adapters={config.max_lora_adapters}")
        self.config = config
        self.weights = weights
        self.gate_up_lora = gate_up_lora
        self.down_lora = down_lora
        self.tp_group = tp_group
        self.last_path = None    # name of the path the last call took (tests and logs read it)

    # ------------------------------------------------------------------ selector predicates
    def _common(self, x, adapter_indices) -> bool:
        w = self.weights
        return bool(
            self.config.w8a8_mlp
            and _is_device_tensor(x) and x.dtype == torch.bfloat16
            and x.ndim >= 2 and x.numel() > 0 and x.shape[-1] == w.hidden_size
            and w.hidden_size % 32 == 0 and w.intermediate_size % 16 == 0
            and (adapter_indices is None or (adapter_indices.dtype == torch.int32 and _is_device_tensor(adapter_indices)))
            and (self.gate_up_lora is None or adapter_indices is not None or self.gate_up_lora.num_adapters == 1)
        )

    def _can_use_w8a8_mlp_block(self, x, rms_delta, rms_eps, adapter_indices, residual) -> bool:
        return bool(
            self._common(x, adapter_indices)
            and self.config.tensor_parallel_size == 1
            and (rms_delta is None or (rms_delta.dtype == torch.bfloat16 and rms_delta.shape == (self.weights.hidden_size,)))
            and (rms_delta is None or rms_eps == self.config.rms_norm_eps)
            and residual is not None and residual.dtype == torch.bfloat16 and residual.shape == x.shape
        )

    def _can_use_w8a8_rms_gate_up_swiglu(self, x, rms_delta, rms_eps, adapter_indices) -> bool:
        return bool(
            self._common(x, adapter_indices)
            and self.config.tensor_parallel_size == 1
            and rms_delta is not None and rms_delta.dtype == torch.bfloat16
            and rms_delta.shape == (self.weights.hidden_size,)
        )

    def _can_use_w8a8_down_residual(self, product, residual, adapter_indices) -> bool:
        w = self.weights
        return bool(
            self.config.w8a8_mlp and self.config.tensor_parallel_size == 1
            and residual is not None and residual.dtype == torch.bfloat16
            and product.dtype == torch.bfloat16 and product.shape[-1] == w.intermediate_size
            and residual.shape == (*product.shape[:-1], w.hidden_size)
        )

    # ------------------------------------------------------------------ helpers
    def _token_ids(self, x, adapter_indices):
        """Per-sequence adapter ids [B] -> per-token ids [B * T] (LoRAMixin.apply_lora repeats the index over
        the sequence: skyrl/tx/layers/lora.py:131-140); per-token ids pass through."""
        if adapter_indices is None:
            return None
        tokens = x.numel() // x.shape[-1]
        if adapter_indices.numel() == tokens:
            return adapter_indices.reshape(-1).contiguous()
        if x.ndim >= 3 and adapter_indices.shape == (x.shape[0],):
            return adapter_indices.repeat_interleave(tokens // x.shape[0]).contiguous()
        raise ValueError(f"adapter_indices of shape {tuple(adapter_indices.shape)} match neither {x.shape[0]} sequences "
                         f"nor {tokens} tokens")

    def _require_armed(self):
        if not self.config.w8a8_mlp:
            raise RuntimeError("the W8A8 MLP path is disabled by default")

    # ------------------------------------------------------------------ forward
    def forward_with_post_attention_rms(self, x, rms_norm: RMSNormWeights, adapter_indices=None, *, residual=None):
        """`residual + mlp(norm(x))` with the norm fused into the front half when the geometry allows
        (Qwen3_5MLP.forward_with_post_attention_rms, skyrl/tx/models/qwen3_5.py:786-826)."""
        self._require_armed()
        delta = rms_norm.weight
        ids = self._token_ids(x, adapter_indices)
        w = self.weights
        if self._can_use_w8a8_mlp_block(x, delta, rms_norm.eps, ids, residual):
            self.last_path = "w8a8_mlp_block"
            out = ops.w8a8_mlp_block(x.reshape(-1, w.hidden_size), delta, w.gate_up, self.gate_up_lora, w.down,
                                     self.down_lora, ids, residual=residual.reshape(-1, w.hidden_size), enabled=True,
                                     eps=rms_norm.eps)
            return out.reshape(x.shape)
        if self.config.tensor_parallel_size > 1:
            return self._tensor_parallel(x, delta, rms_norm.eps, ids, residual)
        if self._can_use_w8a8_rms_gate_up_swiglu(x, delta, rms_norm.eps, ids):
            self.last_path = "w8a8_rms_gate_up_swiglu+down"
            product = ops.w8a8_rms_gate_up_lora_swiglu(x, delta, w.gate_up, self.gate_up_lora, adapter_ids=ids,
                                                       enabled=True, eps=rms_norm.eps)
            return self._apply_down(product, residual, ids)
        return self(rms_norm_reference(x, delta, rms_norm.eps), adapter_indices=adapter_indices, residual=residual)

    def __call__(self, x, adapter_indices=None, *, residual=None):
        """`x` is already normalised (Qwen3_5MLP.__call__, qwen3_5.py:817-826; Qwen3MLP.__call__, qwen3.py:128-131)."""
        self._require_armed()
        ids = self._token_ids(x, adapter_indices)
        w = self.weights
        if self._can_use_w8a8_mlp_block(x, None, self.config.rms_norm_eps, ids, residual):
            self.last_path = "w8a8_mlp_block(no norm)"
            out = ops.w8a8_mlp_block(x.reshape(-1, w.hidden_size), None, w.gate_up, self.gate_up_lora, w.down,
                                     self.down_lora, ids, residual=residual.reshape(-1, w.hidden_size), enabled=True)
            return out.reshape(x.shape)
        if self.config.tensor_parallel_size > 1:
            return self._tensor_parallel(x, None, self.config.rms_norm_eps, ids, residual)
        self.last_path = "w8a8_gate_up_swiglu+down"
        product = ops.w8a8_rms_gate_up_lora_swiglu(x, None, w.gate_up, self.gate_up_lora, adapter_ids=ids, enabled=True)
        return self._apply_down(product, residual, ids)

    def _tensor_parallel(self, x, delta, eps, ids, residual):
        """This rank's shard of the block: partial sums, one all-reduce over the group, finalize
        (the ("tp", "fsdp") sharding of down_proj, skyrl/tx/models/qwen3_5.py:644)."""
        from .tp import TensorParallelMLP

        w = self.weights
        self.last_path = "tensor_parallel_block"
        block = TensorParallelMLP(delta, w.gate_up, self.gate_up_lora, w.down, self.down_lora, group=self.tp_group, eps=eps)
        x2 = x.reshape(-1, w.hidden_size)
        if residual is None:
            # the row-parallel finalize adds a residual; without one the block's own input is subtracted again
            out = block.forward(x2, ids, residual=torch.zeros_like(x2))
        else:
            out = block.forward(x2, ids, residual=residual.reshape(-1, w.hidden_size))
        return out.reshape(x.shape)

    def _apply_down(self, product, residual, ids):
        """Down projection, fused with the residual add when one is given (Qwen3_5MLP._apply_down,
        skyrl/tx/models/qwen3_5.py:760-784)."""
        w = self.weights
        if self._can_use_w8a8_down_residual(product, residual, ids):
            return ops.w8a8_down_lora_residual(product, w.down, self.down_lora, residual=residual, adapter_ids=ids,
                                               enabled=True)
        out = ops.w8a8_down_lora_residual(product, w.down, self.down_lora, adapter_ids=ids, enabled=True)
        return out if residual is None else residual + out


def rms_norm_reference(x: torch.Tensor, delta: torch.Tensor, eps: float) -> torch.Tensor:
    """The unfused norm of the fallback path: `ops.rms_quant` returns the normalised rows the kernels use
    (Qwen3_5RMSNorm.__call__, skyrl/tx/models/qwen3_5.py:269-278)."""
    x2 = x.reshape(-1, x.shape[-1])
    return ops.rms_quant(x2.contiguous(), delta, eps=eps, want_normalized=True)[2].reshape(x.shape)


class Qwen3MLP(Qwen3_5MLP):
    """The Qwen3 form: same projections, called on normalised input without a residual
    (skyrl/tx/models/qwen3.py:100-131); the decoder adds the residual itself (:297-303)."""

    def __call__(self, x, adapter_indices=None):  # noqa: D102 - signature of the reference module
        return super().__call__(x, adapter_indices=adapter_indices, residual=None)
