"""bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), with autograd.

``linear(a, w, bias)`` computes ``a @ w.T + bias`` for row-major bf16 ``a`` [M, K] and
``w`` [N, K] with fp32 accumulation in tensor memory.  The backward pass uses the same
kernel for both products (dA = dY @ W, dW = dY.T @ A).
"""
import torch

from bluefog_b200.common.basics import get_basics

_b = get_basics()


def available() -> bool:
    """True when the tcgen05 GEMM kernel is built into the native module and a GPU is present."""
    C = _b.native
    return bool(torch.cuda.is_available() and hasattr(C, "gemm_bf16_nt") and C.gemm_supported())


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, bias):
        ctx.save_for_backward(a, w)
        ctx.has_bias = bias is not None
        return _b.native.gemm_bf16_nt(a, w, bias, 0)

    @staticmethod
    def backward(ctx, dy):
        a, w = ctx.saved_tensors
        dy = dy.contiguous()
        da = dw = db = None
        if ctx.needs_input_grad[0]:
            # dA[M,K] = dY[M,N] @ W[N,K]  ->  NT form needs W^T [K,N] as the "weight"
            da = _b.native.gemm_bf16_nt(dy, w.t().contiguous(), None, 0)
        if ctx.needs_input_grad[1]:
            # dW[N,K] = dY^T[N,M] @ A[M,K] -> NT form: (dY^T) @ (A^T)^T
            dw = _b.native.gemm_bf16_nt(dy.t().contiguous(), a.t().contiguous(), None, 0)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return da, dw, db


def linear(a: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    """``a @ w.T (+ bias)`` on the tcgen05 kernel; a: [M, K] bf16, w: [N, K] bf16."""
    return _LinearFn.apply(a.contiguous(), w.contiguous(), bias)
