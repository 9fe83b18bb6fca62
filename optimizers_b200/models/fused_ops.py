"""Fused building blocks of the example transformer models.

Each function has two implementations with the same mathematics: plain PyTorch (CPU, unsupported
shapes, or ``set_fused_ops(False)``) and this package's CUDA kernels (``ops/csrc/model_kernels.cu``)
around library GEMMs.

``lm_head_cross_entropy(x, weight, targets)``
    mean cross-entropy of ``x @ weight.T`` against ``targets`` without ever materialising fp32
    logits.  The logits are computed in the autocast dtype into a buffer whose row pitch is padded
    to a multiple of 64 elements, so the three GEMMs (logits, dx, dweight) run on aligned operands
    whatever the vocabulary size (an odd size such as 50257 otherwise forces the GEMM library onto
    its slowest unaligned kernels); one kernel then reads each row once, emits the loss and
    overwrites the row with ``softmax - onehot`` for the backward GEMMs.

``linear``
    ``F.linear`` whose backward computes the bias gradient with a column-sum kernel that reads the
    incoming gradient once with 8-byte accesses (the generic reduction runs at a fraction of the
    memory bandwidth for this shape).

``layer_norm`` / ``rms_norm``
    fp32 statistics, output directly in the autocast dtype (what the following linear layer
    consumes), backward with a two-stage dgamma / dbeta reduction.

No reference counterpart (the reference's examples use stock torch modules).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

_ENABLED = True
_EXT = None
launch_count = 0  # kernels of this module launched so far (benchmarks report the difference)


def set_fused_ops(enabled: bool) -> None:
    """Globally switch the CUDA implementations on or off (off: plain PyTorch everywhere)."""
    global _ENABLED
    _ENABLED = bool(enabled)


def _ext():
    global _EXT
    if _EXT is None:
        from optimizers_b200.ops import build

        _EXT = build.load()
    return _EXT


def _count() -> None:
    global launch_count
    launch_count += 1


def _native(x: Tensor) -> bool:
    return _ENABLED and x.is_cuda and torch.cuda.get_device_capability(x.device)[0] == 10


def _compute_dtype(x: Tensor) -> torch.dtype:
    if x.is_cuda and torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    return x.dtype


# --------------------------------------------------------------------------------------------------
# LM head + cross-entropy
# --------------------------------------------------------------------------------------------------
class _LMHeadXent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, targets: Tensor, ignore_index: int):  # type: ignore[override]
        ext = _ext()
        V, C = weight.shape
        ld = (V + 63) // 64 * 64
        xb = x.to(torch.bfloat16)
        wb = torch.empty(ld, C, dtype=torch.bfloat16, device=x.device)
        wb[:V].copy_(weight)
        wb[V:].zero_()
        logits = torch.mm(xb, wb.t())  # [T, ld]; the padding columns are exact zeros
        targets = targets.contiguous()
        loss_rows = ext.xent_fwd_bwd(logits, V, targets, ignore_index)  # logits now hold softmax - onehot
        _count()
        valid = (targets != ignore_index).sum().clamp_(min=1).to(torch.float32)
        ctx.save_for_backward(xb, wb, logits, valid)
        ctx.V = V
        ctx.x_dtype = x.dtype
        ctx.w_dtype = weight.dtype
        return loss_rows.sum() / valid

    @staticmethod
    def backward(ctx, grad_out: Tensor):  # type: ignore[override]
        xb, wb, dlogits, valid = ctx.saved_tensors
        scale = (grad_out / valid).to(torch.float32)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = (torch.mm(dlogits, wb) * scale).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = (torch.mm(dlogits.t(), xb)[: ctx.V] * scale).to(ctx.w_dtype)
        return dx, dw, None, None


def lm_head_cross_entropy(x: Tensor, weight: Tensor, targets: Tensor, ignore_index: int = -100) -> Tensor:
    """Mean cross-entropy of the logits ``x @ weight.T`` ([T, C] x [V, C]) against ``targets`` [T]."""
    x2 = x.reshape(-1, x.shape[-1])
    t = targets.reshape(-1)
    if _native(x2) and _compute_dtype(x2) == torch.bfloat16 and weight.shape[1] % 8 == 0:
        return _LMHeadXent.apply(x2, weight, t, ignore_index)
    logits = F.linear(x2, weight)
    return F.cross_entropy(logits.float(), t, ignore_index=ignore_index)


# --------------------------------------------------------------------------------------------------
# LayerNorm / RMSNorm
# --------------------------------------------------------------------------------------------------
class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, gamma: Tensor, beta: Tensor | None, eps: float, rms: bool, out_dtype: torch.dtype):  # type: ignore[override]
        ext = _ext()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        g32 = gamma.float().contiguous()
        b32 = None if beta is None else beta.float().contiguous()
        y, mean, rstd = ext.norm_fwd(x2, g32, b32, eps, rms, out_dtype == torch.bfloat16)
        _count()
        ctx.save_for_backward(x2, g32, mean, rstd)
        ctx.rms = rms
        ctx.shape = shape
        ctx.param_dtypes = (gamma.dtype, None if beta is None else beta.dtype)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x2, g32, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape)
        if dy2.dtype not in (torch.float32, torch.bfloat16):
            dy2 = dy2.float()
        dx, partial = _ext().norm_bwd(dy2.contiguous(), x2, g32, mean, rstd, ctx.rms)
        _count()
        sums = partial.sum(0)
        gd, bd = ctx.param_dtypes
        dgamma = sums[0].to(gd) if ctx.needs_input_grad[1] else None
        dbeta = sums[1].to(bd) if (bd is not None and ctx.needs_input_grad[2]) else None
        return dx.view(ctx.shape), dgamma, dbeta, None, None, None


def _norm_native_ok(x: Tensor) -> bool:
    return (
        _native(x) and x.dtype in (torch.float32, torch.bfloat16) and x.numel() > 0
        and _ext().norm_supported(x.shape[-1])
    )


def _norm_out_dtype(x: Tensor) -> torch.dtype:
    cd = _compute_dtype(x)
    return torch.bfloat16 if cd == torch.bfloat16 else torch.float32 if x.dtype == torch.float32 else x.dtype


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor, eps: float = 1e-5) -> Tensor:
    """LayerNorm over the last dim.  Under bf16 autocast the result is bf16 (the normalisation
    itself runs in fp32 on the unrounded input, as autocast's fp32 layer_norm followed by the next
    layer's input cast does)."""
    if _norm_native_ok(x):
        return _Norm.apply(x, weight, bias, eps, False, _norm_out_dtype(x))
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """RMSNorm over the last dim: ``x / sqrt(mean(x^2) + eps) * weight`` with fp32 statistics."""
    if _norm_native_ok(x):
        return _Norm.apply(x, weight, None, eps, True, _norm_out_dtype(x))
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


# --------------------------------------------------------------------------------------------------
# Linear with a fast bias gradient
# --------------------------------------------------------------------------------------------------
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor, dtype: torch.dtype):  # type: ignore[override]
        xb, wb = x.to(dtype), weight.to(dtype)
        ctx.save_for_backward(xb, wb)
        ctx.dtypes = (x.dtype, weight.dtype, bias.dtype)
        return F.linear(xb, wb, bias.to(dtype))

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        xb, wb = ctx.saved_tensors
        xd, wd, bd = ctx.dtypes
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.mm(dy2, wb).view(xb.shape).to(xd)
        if ctx.needs_input_grad[1]:
            dw = torch.mm(dy2.t(), xb.reshape(-1, xb.shape[-1])).to(wd)
        if ctx.needs_input_grad[2]:
            db = _ext().colsum(dy2).to(bd)
            _count()
        return dx, dw, db, None


def linear(x: Tensor, weight: Tensor, bias: Tensor | None) -> Tensor:
    """``F.linear`` in the autocast dtype; on the GPU the bias gradient comes from a dedicated kernel."""
    cd = _compute_dtype(x)
    if (
        bias is not None and _native(x) and cd in (torch.float32, torch.bfloat16) and weight.shape[0] % 4 == 0
        and torch.is_grad_enabled()
    ):
        return _Linear.apply(x, weight, bias, cd)
    return F.linear(x, weight, bias)
