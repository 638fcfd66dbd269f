"""3x3 / stride 1 / pad 1 convolution on the tcgen05 implicit-GEMM kernel, with autograd.

``conv3x3(x, weight)`` has the contract of ``F.conv2d(x, weight, padding=1)`` for a
``[Cout, Cin, 3, 3]`` filter.  bf16 channels_last CUDA activations with ``Cin % 64 == 0``,
``Cout % 8 == 0``, ``Cout >= 64`` and ``W <= 128`` take ``csrc/cuda/conv_tcgen05.cu``:

* forward:  the kernel on (x, weight);
* input gradient: the same kernel on (dy, the same filter), reading the filter taps in reverse order
  and the filter tiles as MN-major operands (the channel axes swap roles without a transposed copy)
  — the transposed convolution of a stride-1 "same" convolution is again one;
* filter gradient: reduces over every output pixel of the batch (a split-K problem with two
  pixel-major operands); it is left to the library (``aten::convolution_backward`` with only the
  weight mask set).

Everything else takes ``F.conv2d``.  The reference has no convolution code of its own
(examples/pytorch_benchmark.py:100 uses torchvision on cuDNN).
"""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


def available() -> bool:
    C = _b.native
    return bool(torch.cuda.is_available() and hasattr(C, "conv3x3_nhwc") and C.gemm_supported())


def eligible(x: torch.Tensor, weight: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and tuple(weight.shape[2:]) == (3, 3) and weight.shape[1] == x.shape[1] and available()):
        return False
    n, cin, h, w = x.shape
    cout = weight.shape[0]
    # the input gradient runs the kernel with the roles of Cin and Cout exchanged
    return bool(_b.native.conv3x3_supported(n, h, w, cin, cout) and _b.native.conv3x3_supported(n, h, w, cout, cin))


class _Conv3x3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        x = x.contiguous(memory_format=torch.channels_last)
        wk = weight.contiguous(memory_format=torch.channels_last)          # [Cout, 3, 3, Cin] in memory
        ctx.save_for_backward(x, weight)
        return _b.native.conv3x3_nhwc(x, wk)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # the forward filter [Cout, Cin, 3, 3] is read in place: as an MN-major operand (its reduction
            # channels are the outer dimension here) and with the taps in reverse order (180-degree rotation)
            dx = _b.native.conv3x3_nhwc(dy, weight.contiguous(memory_format=torch.channels_last), True, 1)
        if ctx.needs_input_grad[1]:
            dw = torch.ops.aten.convolution_backward(dy, x, weight, None, (1, 1), (1, 1), (1, 1), False, (0, 0), 1,
                                                     (False, True, False))[1]
        return dx, dw


def conv3x3(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if eligible(x, weight):
        return _Conv3x3Fn.apply(x, weight)
    return F.conv2d(x, weight, padding=1)
