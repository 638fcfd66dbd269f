"""Fused training-mode BatchNorm + ReLU (+ residual add) for NHWC bf16 activations.

``bn_act(x, bn, relu=True, residual=None)`` computes ``relu(batch_norm(x) + residual)`` with two
streaming kernels forward and two backward (bluefog_b200/csrc/cuda/bn_kernels.cu) instead of
the separate normalisation, add and ReLU passes; it falls back to PyTorch for eval mode and
for tensors the kernels do not cover (not CUDA, not bf16, not channels_last).
"""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


class _BnActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, beta, running_mean, running_var, eps, momentum, relu):
        y, mean, rstd = _b.native.bn_forward(x, residual, gamma, beta, running_mean, running_var, eps, momentum, relu)
        ctx.save_for_backward(x, y, mean, rstd, gamma)
        ctx.relu = relu
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, mean, rstd, gamma = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx, dres, dgamma, dbeta = _b.native.bn_backward(dy, y, x, mean, rstd, gamma, ctx.relu, ctx.has_res)
        return dx, (dres if ctx.has_res else None), dgamma, dbeta, None, None, None, None, None


def bn_act(x, bn, relu=True, residual=None):
    """``bn`` is an ``nn.BatchNorm2d``-like module (weight, bias, running_mean, running_var, eps, momentum)."""
    use_kernel = (bn.training and x.is_cuda and x.dtype == torch.bfloat16 and bn.weight is not None
                  and _b.native.bn_supported(x)
                  and (residual is None or (residual.dtype == torch.bfloat16 and residual.shape == x.shape)))
    if use_kernel:
        if residual is not None and not residual.is_contiguous(memory_format=torch.channels_last):
            residual = residual.contiguous(memory_format=torch.channels_last)
        if bn.track_running_stats and bn.num_batches_tracked is not None:
            bn.num_batches_tracked.add_(1)
        momentum = 0.1 if bn.momentum is None else bn.momentum
        rm = bn.running_mean if bn.track_running_stats else None
        rv = bn.running_var if bn.track_running_stats else None
        return _BnActFn.apply(x, residual, bn.weight, bn.bias, rm, rv, bn.eps, momentum, relu)
    out = bn(x)
    if residual is not None:
        out = out + residual
    return F.relu(out) if relu else out
