"""LayerNorm on the hand-written row-in-registers kernels (``csrc/cuda/ln_kernels.cu``).

``layer_norm(x, weight, bias, eps)`` has the contract of ``torch.nn.functional.layer_norm`` over the
last dimension.  bf16 CUDA activations whose row length is a multiple of 8 and at most 2048 take the
kernels; everything else (CPU, fp32, longer rows) takes PyTorch's implementation.  The reference has
no normalisation code of its own; this is what the GPT-2 model of this library calls.
"""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


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
        dx, dgamma, dbeta = _b.native.ln_backward(dy.contiguous(), x, weight, mean, rstd)
        return dx, dgamma.to(weight.dtype), dbeta.to(weight.dtype), None


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
