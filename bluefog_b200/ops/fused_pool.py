"""3x3 / stride 2 / padding 1 max pooling and global average pooling on NHWC bf16 activations with hand-written
forward and backward kernels (bluefog_b200/csrc/cuda/pool_kernels.cu); anything else goes to PyTorch."""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y, idx = _b.native.maxpool3x3s2_forward(x)
        ctx.save_for_backward(idx)
        ctx.hw = (x.shape[2], x.shape[3])
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        return _b.native.maxpool3x3s2_backward(dy, idx, ctx.hw[0], ctx.hw[1])


def maxpool3x3s2(x: torch.Tensor) -> torch.Tensor:
    if (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last)):
        return _MaxPoolFn.apply(x)
    return F.max_pool2d(x, kernel_size=3, stride=2, padding=1)


class _AvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.hw = (x.shape[2], x.shape[3])
        return _b.native.avgpool_forward(x)

    @staticmethod
    def backward(ctx, dy):
        return _b.native.avgpool_backward(dy.contiguous(), ctx.hw[0], ctx.hw[1])


def global_avgpool(x: torch.Tensor) -> torch.Tensor:
    """``x.mean((2, 3))`` of a [N, C, H, W] activation as [N, C]."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last) and hasattr(_b.native, "avgpool_forward")):
        return _AvgPoolFn.apply(x)
    return torch.flatten(F.adaptive_avg_pool2d(x, (1, 1)), 1)
