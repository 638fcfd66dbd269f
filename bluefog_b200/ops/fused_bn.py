"""Fused training-mode BatchNorm + ReLU (+ residual add) for NHWC bf16 activations.

``bn_act(x, bn, relu=True, residual=None)`` computes ``relu(batch_norm(x) + residual)`` with two
streaming kernels forward and two backward (bluefog_b200/csrc/cuda/bn_kernels.cu) instead of
the separate normalisation, add and ReLU passes; it falls back to PyTorch for eval mode and
for tensors the kernels do not cover (not CUDA, not bf16, not channels_last).
"""
import os
import weakref

import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


class _Workspace:
    """Zero-initialised scratch for the per-channel sums of all BatchNorm layers of one step.

    ``begin_step`` clears the part used by the previous step with a single memset and hands out
    slices from the start again; layers that run without ``begin_step`` (or do not fit) simply
    allocate their own zeros.  A slice is used at most once per generation, so a second backward
    through the same forward, or two forwards before a backward, fall back to fresh zeros.
    """

    def __init__(self, device, capacity=1 << 20):
        self.buf = torch.zeros(capacity, dtype=torch.float32, device=device)
        self.offset = 0
        self.high_water = 0
        self.generation = 0
        self.active = False

    def begin_step(self):
        if self.high_water:
            self.buf[:self.high_water].zero_()
        self.offset = 0
        self.high_water = 0
        self.generation += 1
        self.active = True

    def take(self, n):
        if not self.active or self.offset + n > self.buf.numel():
            return None, -1
        out = self.buf[self.offset:self.offset + n]
        self.offset += (n + 63) // 64 * 64
        self.high_water = max(self.high_water, self.offset)
        return out, self.generation


_workspaces = {}

# BLUEFOG_B200_PAIR_GRADIENTS=0: the two gradients of a block input are added by autograd as usual
PAIR_GRADIENTS = os.environ.get("BLUEFOG_B200_PAIR_GRADIENTS", "1") != "0"


def begin_step(device):
    """Call once at the start of a training forward pass (the models of this package do)."""
    if _pending_pairs:
        _pending_pairs.clear()
        raise RuntimeError("a gradient pair of split_for_two_uses was never taken by the BatchNorm that produced the "
                           "tensor; use it only on outputs of bn_act")
    if device.type != "cuda":
        return
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = _Workspace(device)
    ws.begin_step()


def _take(device, n):
    ws = _workspaces.get(device.index if device.index is not None else torch.cuda.current_device())
    if ws is None:
        return None, -1, None
    t, gen = ws.take(n)
    return t, gen, ws


def take_sums(device, channels):
    """2*channels zeroed fp32 values for the kernel that produces a BatchNorm input to add the per-channel sum and
    sum of squares of its output to; hand them to ``bn_act(..., stats=)``, which then skips its statistics pass."""
    t, _, _ = _take(device, 2 * channels)
    return t if t is not None else torch.zeros(2 * channels, dtype=torch.float32, device=device)


# Gradient pairs on their way from _SplitFn.backward to the BatchNorm backward that consumes them:
# data_ptr of the first addend -> (weak reference to it, second addend)
_pending_pairs = {}


class _SplitFn(torch.autograd.Function):
    """``x -> (x, x)`` for a tensor with two uses (a residual block reads its input through the first convolution
    and through the shortcut).  Autograd would add the two gradients in a pass of its own (two reads, one write
    of a full activation); here they travel as a pair to the BatchNorm kernels that produced ``x``, which read both
    addends and form the sum in registers."""

    @staticmethod
    def forward(ctx, x):
        return x.view_as(x), x.view_as(x)

    @staticmethod
    def backward(ctx, ga, gb):
        if ga is None or gb is None:
            return ga if gb is None else gb
        if (ga.shape != gb.shape or ga.dtype != torch.bfloat16 or gb.dtype != torch.bfloat16
                or not ga.is_contiguous(memory_format=torch.channels_last)
                or not gb.is_contiguous(memory_format=torch.channels_last)):
            return ga + gb
        _pending_pairs[ga.data_ptr()] = (weakref.ref(ga), gb)
        return ga


def split_for_two_uses(x):
    """Two handles of ``x`` whose gradients reach the producer of ``x`` un-added (see ``_SplitFn``).  Only outputs of
    ``bn_act`` that took the kernel path qualify; any other tensor comes back twice unchanged."""
    if getattr(x, "_bfb_takes_pairs", False) and x.requires_grad and torch.is_grad_enabled():
        return _SplitFn.apply(x)
    return x, x


class _BnActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, beta, running_mean, running_var, eps, momentum, relu, stats):
        # accumulators (several copies for few channels) and a zeroed word for the barrier of the one-launch kernels
        c2 = _b.native.bn_workspace_floats(x.shape[1]) if hasattr(_b.native, "bn_workspace_floats") else 2 * x.shape[1]
        if stats is not None:
            fwd_sums = stats
        else:
            fwd_sums, _, _ = _take(x.device, c2)
        y, mean, rstd, mask = _b.native.bn_forward(x, residual, gamma, beta, running_mean, running_var, eps, momentum,
                                                   relu, fwd_sums, stats is not None)
        # backward needs x, the statistics and one bit per element for the ReLU; not y itself
        ctx.save_for_backward(x, mask, mean, rstd, gamma)
        ctx.relu = relu
        ctx.has_res = residual is not None
        ctx.bwd_sums, ctx.bwd_gen, ctx.ws = _take(x.device, c2)   # reserved now, consumed by backward
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mask, mean, rstd, gamma = ctx.saved_tensors
        dy2 = None
        pair = _pending_pairs.pop(dy.data_ptr(), None)
        if pair is not None:
            if pair[0]() is not dy:
                raise RuntimeError("gradient pair does not belong to this gradient")
            dy2 = pair[1]
        dy = dy.contiguous(memory_format=torch.channels_last)
        sums = None
        if ctx.bwd_sums is not None and ctx.ws.generation == ctx.bwd_gen:
            sums, ctx.bwd_sums = ctx.bwd_sums, None    # a slice is clean only once
        dx, dres, dgamma, dbeta = _b.native.bn_backward(dy, mask, x, mean, rstd, gamma, ctx.relu, ctx.has_res, sums, dy2)
        return dx, (dres if ctx.has_res else None), dgamma, dbeta, None, None, None, None, None, None


def bn_act(x, bn, relu=True, residual=None, count_batches=True, stats=None):
    """``bn`` is an ``nn.BatchNorm2d``-like module (weight, bias, running_mean, running_var, eps, momentum).
    ``stats``: 2*C fp32 values holding sum(x) and sum(x^2) per channel, written by the producer of ``x``
    (see ``take_sums``); ignored where the kernels do not apply."""
    use_kernel = (bn.training and x.is_cuda and x.dtype == torch.bfloat16 and bn.weight is not None
                  and _b.native.bn_supported(x)
                  and (residual is None or (residual.dtype == torch.bfloat16 and residual.shape == x.shape)))
    if use_kernel:
        if residual is not None and not residual.is_contiguous(memory_format=torch.channels_last):
            residual = residual.contiguous(memory_format=torch.channels_last)
        if count_batches and bn.track_running_stats and bn.num_batches_tracked is not None:
            bn.num_batches_tracked.add_(1)
        momentum = 0.1 if bn.momentum is None else bn.momentum
        rm = bn.running_mean if bn.track_running_stats else None
        rv = bn.running_var if bn.track_running_stats else None
        y = _BnActFn.apply(x, residual, bn.weight, bn.bias, rm, rv, bn.eps, momentum, relu, stats)
        y._bfb_takes_pairs = PAIR_GRADIENTS          # its backward accepts the pairs of split_for_two_uses
        return y
    out = bn(x)
    if residual is not None:
        out = out + residual
    return F.relu(out) if relu else out
