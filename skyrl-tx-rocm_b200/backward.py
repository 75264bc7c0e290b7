"""Backward pass of the W8A8 LoRA linear (straight-through estimator).

The reference defines the operator as a `jax.custom_vjp` whose backward treats both quantisers as the
identity and the frozen base as its dequantised weight (`_quantized_lora_linear_bwd`,
skyrl/tx/kernels/quantized_lora.py:337-394):

    R  = s * (dy @ B^T)
    dx = dy @ deq(W)^T + R @ A^T          (dominant: an [M, N] x [N, K] contraction)
    dA = x^T @ R,   dB = s * (x @ A)^T @ dy,   ds = sum(dy * ((x @ A) @ B))

Here the dominant contraction runs on the same tcgen05 int8 kernels as the forward: the weight's
per-output-channel scale moves to the cotangent, g = dy * sw, each row of g is split into two int8 planes
(`skyrl_w8a8_grad_quant_sm100_v1`), and the GEMM runs once per plane over a TRANSPOSED packed copy of the
codes (unit weight scales) into fp32 slabs.  dx therefore equals the fp32 product to about 2^-15 relative
(two planes) — far inside bf16's own rounding — at the cost of one bf16 GEMM, and `R @ A^T` rides the LoRA
slice of the last plane's launch exactly as `s (x A) B` does in the forward.  The rank-r reductions dA, dB and
ds are two orders of magnitude smaller and use library matmuls over the adapter-sorted rows (bf16 tensor-core
products with fp32 results; the small fp32 factors are split into two bf16 terms).

`W8A8LoRALinearFunction` ties forward and backward together for `torch.autograd`, the counterpart of the
reference's `quantized_lora_linear.defvjp(...)` (quantized_lora.py:397).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib, ops
from .ops import EPI_PARTIAL_F32, LORA_RANK_PAD, Z_PARTS, PackedLoRA, PackedW8Weight


@dataclass(frozen=True)
class PackedW8Backward:
    """What the input gradient needs from a frozen weight: the codes packed with N as the contraction
    dimension and the forward scales as a column vector.  Built once per weight at load time."""

    wq_t: PackedW8Weight     # in_features = padded N of the forward weight, out_features = K, scales 1
    col_scale: torch.Tensor  # fp32 [padded N]: the forward weight's per-output-channel scales
    in_features: int         # K of the forward weight
    out_features: int        # N of the forward weight


def pack_weight_backward(weight) -> PackedW8Backward:
    """Forward weight (reference storage or packed) -> its backward companion."""
    w = ops._weight_of(weight)
    if w.group_size:
        raise ops.SkyrlKernelError("the backward path takes per-output-channel scales (one group over K)")
    k, npad = w.in_features, w.padded_out_features
    if k % 32:
        raise ValueError(f"the input gradient needs K to be a multiple of 32, got {k}")
    kb, _, blk = w.wq.shape
    codes_kn = w.wq.permute(0, 2, 1).reshape(kb * blk, npad)[:k].contiguous()   # [K, padded N]: rows = outputs of W^T
    ones = torch.ones((k,), dtype=torch.float32, device=w.wq.device)
    return PackedW8Backward(ops.pack_weight_nk(codes_kn, ones), w.sw.contiguous(), k, w.out_features)


def pack_lora_backward(lora_a: torch.Tensor, lora_b: torch.Tensor, lora_scaling, weight_bwd: PackedW8Backward) -> PackedLoRA:
    """LoRA tables of the transposed operator: "A" = B^T [A, N, r], "B" = A^T [A, r, K], same scaling, so that
    s (dy B^T) A^T is the forward LoRA expression of the transposed weight."""
    if lora_a.ndim == 2:
        lora_a, lora_b = lora_a[None], lora_b[None]
    return ops.pack_lora(lora_b.transpose(1, 2).contiguous(), lora_a.transpose(1, 2).contiguous(), lora_scaling,
                         in_features=weight_bwd.wq_t.in_features,
                         padded_out_features=weight_bwd.wq_t.padded_out_features)


def w8a8_lora_linear_input_grad(dy: torch.Tensor, weight_bwd: PackedW8Backward, lora_bwd: PackedLoRA | None = None,
                                adapter_ids=None, *, planes: int = 2, enabled: bool = False) -> torch.Tensor:
    """dx = dy @ deq(W)^T + s (dy @ B^T) @ A^T as bf16 [..., K] (quantized_lora.py:364-372)."""
    ops._validate_exact_bool("enabled", enabled)
    if not enabled:
        raise RuntimeError("the W8A8 backward kernel is disabled by default")
    if planes not in (1, 2):
        raise ValueError("planes must be 1 or 2")
    lib = _lib.load()
    wt = weight_bwd.wq_t
    n_logical, npad, k = weight_bwd.out_features, wt.in_features, wt.out_features
    dy2 = ops._pad_cols(ops._check_x(dy, n_logical), npad)
    m, dev = dy2.shape[0], dy2.device
    na = lora_bwd.num_adapters if lora_bwd is not None else 1
    ids = ops._check_ids(adapter_ids, m, lora_bwd)
    st = ops._status_word(dev)
    perm, tiles, num = ops.prepare_routing(ids, m, na)
    row_map = perm if ids is not None else None
    max_tiles = tiles.shape[0]

    q = torch.empty((planes, m, npad), dtype=torch.int8, device=dev)
    s = torch.empty((planes, m), dtype=torch.float32, device=dev)
    second = planes == 2
    _lib.check(lib.skyrl_w8a8_grad_quant_sm100_v1(
        ops._ptr(dy2), dy2.stride(0), ops._ptr(weight_bwd.col_scale), ops._ptr(row_map), m, npad, ops._ptr(q[0]),
        ops._ptr(s[0]), ops._ptr(q[1]) if second else None, ops._ptr(s[1]) if second else None, ops._stream()),
        "grad_quant")

    z_parts = None
    if lora_bwd is not None:
        if ids is not None:
            _, _, ys = ops.rms_quant(dy2, row_map=perm, want_normalized=True)   # dy rows in adapter-sorted order
        else:
            ys = dy2.contiguous()
        z_parts = torch.empty((m, Z_PARTS, LORA_RANK_PAD), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.skyrl_lora_a_proj_sm100_v1(ops._ptr(ys), m, npad, ops._ptr(lora_bwd.a), ops._ptr(lora_bwd.scaling),
                                                  na, lora_bwd.rank, ops._ptr(tiles), ops._ptr(num), max_tiles,
                                                  ops._ptr(z_parts), ops._ptr(st), ops._stream()), "lora_a_proj (backward)")

    slabs = torch.empty((planes, m, k), dtype=torch.float32, device=dev)
    for p in range(planes):
        a = _lib.GemmArgs()
        a.struct_size = C.sizeof(_lib.GemmArgs)
        a.epilogue = EPI_PARTIAL_F32
        a.m, a.n, a.k = m, k, npad
        a.xq, a.sx, a.sw = q[p].data_ptr(), s[p].data_ptr(), wt.sw.data_ptr()
        a.wq = wt.wq.data_ptr()
        last = p == planes - 1
        a.rank = lora_bwd.rank if (lora_bwd is not None and last) else 0
        a.num_adapters = na
        a.max_tiles = max_tiles
        if a.rank:
            a.z_parts, a.lora_b_packed = z_parts.data_ptr(), lora_bwd.b.data_ptr()
        a.tiles, a.num_tiles = tiles.data_ptr(), num.data_ptr()
        a.out, a.out_row_stride = slabs[p].data_ptr(), k
        a.status = st.data_ptr()
        _lib.check(lib.skyrl_w8a8_gemm_sm100_v1(C.byref(a), ops._stream()), "w8a8_gemm (input gradient)")
    dx = torch.empty((m, k), dtype=torch.bfloat16, device=dev)
    _lib.check(lib.skyrl_group_sum_cast_sm100_v1(ops._ptr(slabs), planes, m, k, ops._ptr(row_map), ops._ptr(dx), k,
                                                 ops._stream()), "group_sum_cast (input gradient)")
    return dx.reshape(*dy.shape[:-1], k)


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 result of a @ b.  bf16 operands on a CUDA device multiply on the tensor cores (products of bf16 pairs are
    exact in the fp32 accumulator) without an fp32 copy of either operand; anything else takes the plain fp32 path."""
    if a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16:
        return torch.mm(a, b, out_dtype=torch.float32)
    return a.float() @ b.float()


def _split_bf16(t: torch.Tensor):
    """fp32 -> (hi, lo) bf16 with hi + lo == t to 2^-17 relative: keeps a small fp32 factor exact enough for a bf16
    tensor-core matmul against a large bf16 operand."""
    hi = t.to(torch.bfloat16)
    return hi, (t - hi.float()).to(torch.bfloat16)


def lora_parameter_grads(x: torch.Tensor, dy: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor, lora_scaling,
                         adapter_ids=None):
    """(dA [A, K, r], dB [A, r, N], ds [A]) in fp32 (quantized_lora.py:374-389), rows grouped by adapter.

    Library matmuls.  Each gradient is a rank-r reduction over the rows: U = x A and R' = dy B^T are [M, r]; then
    dA = x^T (s R'), dB = s U^T dy and ds = sum(U * R') (the reference's sum(dy * (U B)) with the contraction over N
    done first).  On a CUDA device the large operands x and dy stay bf16: the small fp32 factors are split into two
    bf16 terms, so every product runs on the tensor cores with fp32 accumulation."""
    squeeze = lora_a.ndim == 2
    if squeeze:
        lora_a, lora_b = lora_a[None], lora_b[None]
    na, k, r = lora_a.shape
    n = lora_b.shape[2]
    x2 = x.reshape(-1, k)
    dy2 = dy.reshape(-1, n)
    m = x2.shape[0]
    scaling = torch.as_tensor(lora_scaling, dtype=torch.float32, device=x.device).reshape(-1)
    d_a = torch.zeros((na, k, r), dtype=torch.float32, device=x.device)
    d_b = torch.zeros((na, r, n), dtype=torch.float32, device=x.device)
    d_s = torch.zeros((na,), dtype=torch.float32, device=x.device)
    if adapter_ids is None:
        xs, gs, counts = x2, dy2, [m] + [0] * (na - 1)
    else:
        ids = adapter_ids.reshape(-1).to(torch.int64)
        order = torch.argsort(ids, stable=True)
        counts = torch.bincount(ids, minlength=na).tolist()
        xs, gs = x2[order], dy2[order]            # one gather; the adapters' rows are then contiguous slices
    fast = xs.is_cuda and xs.dtype == torch.bfloat16 and gs.dtype == torch.bfloat16
    start = 0
    for a, count in enumerate(counts):
        if count == 0:
            continue
        xa, ga = xs[start:start + count], gs[start:start + count]
        start += count
        inter = _mm_f32(xa, lora_a[a])                       # U  [Ma, r]
        low_unscaled = _mm_f32(ga, lora_b[a].t())            # R' [Ma, r]
        low = low_unscaled * scaling[a]
        if fast:
            low_hi, low_lo = _split_bf16(low)
            int_hi, int_lo = _split_bf16(inter)
            xat, gat = xa.t(), ga
            d_a[a] = _mm_f32(xat, low_hi) + _mm_f32(xat, low_lo)
            d_b[a] = (_mm_f32(int_hi.t(), gat) + _mm_f32(int_lo.t(), gat)) * scaling[a]
        else:
            d_a[a] = xa.float().t() @ low
            d_b[a] = (inter.t() @ ga.float()) * scaling[a]
        d_s[a] = (inter * low_unscaled).sum()
    if squeeze:
        return d_a[0], d_b[0], d_s[0]
    return d_a, d_b, d_s


class W8A8LoRALinearFunction(torch.autograd.Function):
    """y = w8a8_lora_linear(x, W, A, B, s, ids) with the reference's straight-through backward
    (quantized_lora.py:317-397).  The frozen weight receives no gradient."""

    @staticmethod
    def forward(ctx, x, lora_a, lora_b, lora_scaling, weight, weight_bwd, adapter_ids):
        ctx.save_for_backward(x, lora_a, lora_b, lora_scaling, adapter_ids if adapter_ids is not None else torch.empty(0))
        ctx.weight_bwd = weight_bwd
        ctx.has_ids = adapter_ids is not None
        return ops.w8a8_lora_linear(x, weight, lora_a, lora_b, lora_scaling, adapter_ids, enabled=True)

    @staticmethod
    def backward(ctx, dy):
        x, lora_a, lora_b, lora_scaling, ids = ctx.saved_tensors
        ids = ids if ctx.has_ids else None
        dy = dy.contiguous()
        lora_bwd = pack_lora_backward(lora_a.detach(), lora_b.detach(), lora_scaling.detach(), ctx.weight_bwd)
        dx = w8a8_lora_linear_input_grad(dy, ctx.weight_bwd, lora_bwd, ids, enabled=True) if ctx.needs_input_grad[0] else None
        d_a, d_b, d_s = lora_parameter_grads(x.detach(), dy, lora_a.detach(), lora_b.detach(), lora_scaling.detach(), ids)
        return (dx, d_a.to(lora_a.dtype), d_b.to(lora_b.dtype), d_s.reshape(lora_scaling.shape).to(lora_scaling.dtype),
                None, None, None)


def w8a8_lora_linear_trainable(x, weight, weight_bwd: PackedW8Backward, lora_a, lora_b, lora_scaling, adapter_ids=None):
    """Differentiable form of `ops.w8a8_lora_linear` (x, A, B and the scaling receive gradients)."""
    scaling = lora_scaling if isinstance(lora_scaling, torch.Tensor) else torch.as_tensor(
        lora_scaling, dtype=torch.float32, device=x.device)
    return W8A8LoRALinearFunction.apply(x, lora_a, lora_b, scaling, weight, weight_bwd, adapter_ids)
