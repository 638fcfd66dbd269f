"""LayerNorm on the hand-written row-in-registers kernels (``csrc/cuda/ln_kernels.cu``).

``layer_norm(x, weight, bias, eps)`` has the contract of ``torch.nn.functional.layer_norm`` over the
last dimension.  bf16 CUDA activations whose row length is a multiple of 8 and at most 2048 take the
kernels; everything else (CPU, fp32, longer rows) takes PyTorch's implementation.  The reference has
no normalisation code of its own; this is what the GPT-2 model of this library calls.
"""
import os
import weakref

import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()

# BLUEFOG_B200_LN_RESIDUAL=0: the two gradients of a block input are added by autograd (one more pass per LayerNorm)
FUSE_RESIDUAL_GRADIENT = os.environ.get("BLUEFOG_B200_LN_RESIDUAL", "1") != "0"


def _eligible(x, weight, bias):
    return (x.is_cuda and x.dtype == torch.bfloat16 and _b.native is not None and weight is not None
            and bias is not None and weight.dtype == bias.dtype
            and weight.dtype in (torch.float32, torch.bfloat16)
            and x.shape[-1] % 8 == 0 and 8 <= x.shape[-1] <= 2048 and x.numel() > 0)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x = x.contiguous()
        y, mean, rstd = _b.native.ln_forward(x, weight, bias, eps)
        ctx.save_for_backward(x, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dx, sums = _b.native.ln_backward(dy.contiguous(), x, weight, mean, rstd)
        sums = sums.to(weight.dtype)                  # [dgamma, dbeta], one conversion for both
        return dx, sums[0], sums[1], None


# Column sums that left a backward kernel together with a gradient: data_ptr of the gradient -> (weak reference to
# it, fp32 sums).  The backward pass of the linear layer that receives that gradient takes its bias gradient from
# here instead of reading the gradient once more.  An entry is only honoured while the tensor it was made for is
# alive, so an address that the allocator hands out again cannot match.
_column_sums = {}
column_sum_hits = 0          # how many bias gradients were served from _column_sums (tests read this)


def _offer_column_sums(grad, sums):
    for key in [k for k, (ref, _) in _column_sums.items() if ref() is None]:
        del _column_sums[key]
    _column_sums[grad.data_ptr()] = (weakref.ref(grad), sums)


def take_column_sums(dy):
    """Column sums of the 2-D gradient ``dy`` (fp32, or already converted to the gradient's dtype) if the kernel that
    produced it summed them on its way, else None."""
    global column_sum_hits
    entry = _column_sums.pop(dy.data_ptr(), None) if _column_sums else None
    if entry is None:
        return None
    made_for = entry[0]()
    if made_for is None or made_for.numel() != dy.numel() or made_for.shape[-1] != dy.shape[-1]:
        return None
    column_sum_hits += 1
    return entry[1]


class _LayerNormResidualFn(torch.autograd.Function):
    """(LayerNorm(x), x): the second result is the residual branch.  Its backward pass forms LN'(dy) + d_residual in the
    LayerNorm kernel (no addition pass of its own) and sums the columns of the total for the layer in front of it."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x = x.contiguous()
        y, mean, rstd = _b.native.ln_forward(x, weight, bias, eps)
        ctx.save_for_backward(x, weight, mean, rstd)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x, weight, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        if dres is None:
            dx, sums = _b.native.ln_backward(dy.contiguous(), x, weight, mean, rstd)
            sums = sums.to(weight.dtype)
            return dx, sums[0], sums[1], None
        dx, sums = _b.native.ln_backward(dy.contiguous(), x, weight, mean, rstd, dres.contiguous())
        if weight.dtype == dx.dtype:
            sums = sums.to(weight.dtype)              # the bias gradient wants the activation dtype: one conversion for all three
        _offer_column_sums(dx, sums[2])
        return dx, sums[0].to(weight.dtype), sums[1].to(weight.dtype), None


def layer_norm_residual(x, weight, bias, eps=1e-5):
    """``(layer_norm(x), x)`` for the pattern ``x + f(layer_norm(x))`` of a pre-norm transformer block: feed the second
    result to the addition.  Both gradients then meet inside the LayerNorm backward kernel."""
    if _eligible(x, weight, bias) and x.requires_grad and torch.is_grad_enabled() and FUSE_RESIDUAL_GRADIENT:
        return _LayerNormResidualFn.apply(x, weight, bias, eps)
    return layer_norm(x, weight, bias, eps), x


def layer_norm(x, weight, bias, eps=1e-5):
    if _eligible(x, weight, bias):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


class LayerNorm(torch.nn.LayerNorm):
    """``torch.nn.LayerNorm`` over the last dimension that routes bf16 CUDA inputs to the kernels."""

    def forward(self, x):
        if len(self.normalized_shape) == 1:
            return layer_norm(x, self.weight, self.bias, self.eps)
        return super().forward(x)

    def with_residual(self, x):
        """``(self(x), x)``; see ``layer_norm_residual``."""
        if len(self.normalized_shape) == 1:
            return layer_norm_residual(x, self.weight, self.bias, self.eps)
        return super().forward(x), x
