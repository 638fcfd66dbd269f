"""Mean cross-entropy of bf16 logits on the row-per-block kernels (``csrc/cuda/ce_kernels.cu``).

``cross_entropy(logits, targets)`` has the contract of ``F.cross_entropy(logits.float(), targets)`` (mean
reduction, every target a valid class) for a contiguous bf16 CUDA matrix whose row length is a multiple of 8;
the arithmetic is fp32 but no fp32 copy of the logits is made, and the gradient is written directly in bf16.
Anything else takes PyTorch's implementation.  The reference has no loss code of its own.
"""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        loss, lse = _b.native.cross_entropy_forward(logits, targets)
        ctx.save_for_backward(logits, targets, lse)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        logits, targets, lse = ctx.saved_tensors
        g = grad_out.to(torch.float32).reshape(1).contiguous()
        return _b.native.cross_entropy_backward(logits, targets, lse, g), None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    if (logits.is_cuda and logits.dim() == 2 and logits.dtype == torch.bfloat16 and logits.is_contiguous()
            and logits.shape[1] % 8 == 0 and logits.shape[0] > 0 and targets.dtype == torch.int64
            and _b.native is not None and hasattr(_b.native, "cross_entropy_forward")):
        return _CrossEntropyFn.apply(logits, targets.contiguous())
    return F.cross_entropy(logits.float(), targets)
