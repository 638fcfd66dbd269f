"""bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), with autograd.

``linear(a, w, bias)`` computes ``a @ w.T + bias`` for row-major bf16 ``a`` [M, K] and
``w`` [N, K] with fp32 accumulation in tensor memory.  The backward pass computes dA = dY @ W on the
same kernel with W read in place as an MN-major operand, and dW = dY.T @ A with both operands read
MN-major (products with too few output tiles for a kernel without split-K go to the library, see
``_LinearFn.backward``).
"""
import torch

from bluefog_b200.common.basics import get_basics
from bluefog_b200.ops import fused_ln

_b = get_basics()


def available() -> bool:
    """True when the tcgen05 GEMM kernel is built into the native module and a GPU is present."""
    C = _b.native
    return bool(torch.cuda.is_available() and hasattr(C, "gemm_bf16_nt") and C.gemm_supported())


def _input_gradient(dy2d: torch.Tensor, w2d: torch.Tensor) -> torch.Tensor:
    """dX[M, K] = dY[M, N] @ W[N, K] on the tcgen05 kernel.  W [N, K] row-major is exactly the [K_red, N_out]
    operand of this product, which the kernel reads in place as an MN-major tile (no transposed copy)."""
    if w2d.shape[1] % 8 == 0 and w2d.shape[0] % 8 == 0:
        return _b.native.gemm_bf16_nn(dy2d, w2d.contiguous())
    return _b.native.gemm_bf16_nt(dy2d, w2d.t().contiguous(), None, 0)


def _nt_ok(m_rows, n_rows, k):
    """The kernel needs a reduction length that is a multiple of 8 (16-byte TMA row pitch)."""
    return k % 8 == 0 and m_rows > 0 and n_rows > 0


# Weight gradients with fewer output tiles (128 x 256) than this leave most SMs idle in a kernel without split-K
_TN_MIN_TILES = 120


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, bias, residual=None):
        ctx.save_for_backward(a, w)
        ctx.has_bias = bias is not None
        # residual: added in the GEMM epilogue (out = a w^T + bias + residual) instead of by a pass of its own
        return _b.native.gemm_bf16_nt(a, w, bias, 0, None, residual)

    @staticmethod
    def backward(ctx, dy):
        a, w = ctx.saved_tensors
        dy = dy.contiguous()
        da = dw = db = None
        if ctx.needs_input_grad[0]:
            # dA[M,K] = dY[M,N] @ W[N,K]: the reduction runs over N, so the kernel's second operand
            # is W^T [K,N]; weights are small, the transpose copy is cheap.
            if _nt_ok(dy.shape[0], w.shape[1], dy.shape[1]):
                da = _input_gradient(dy, w)
            else:
                da = dy @ w
        if ctx.needs_input_grad[1]:
            # dW[N,K] = dY^T @ A reduces over the rows of two activation matrices: both operands are MN-major
            # for that product and the kernels read them in place.
            dw = _weight_gradient(dy, a)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            sums = fused_ln.take_column_sums(dy)                  # summed on the way by the kernel that made dy
            if sums is not None:
                db = sums.to(dy.dtype)
            elif dy.shape[1] % 8 == 0 and hasattr(_b.native, "column_sum"):
                db = _b.native.column_sum(dy).to(dy.dtype)       # fp32 sums of the bf16 gradient in one pass
            else:
                db = dy.sum(0, dtype=torch.float32).to(dy.dtype)
        return da, dw, db, (dy if ctx.needs_input_grad[3] else None)


def linear(a: torch.Tensor, w: torch.Tensor, bias=None, residual=None) -> torch.Tensor:
    """``a @ w.T (+ bias) (+ residual)`` on the tcgen05 kernel; a: [M, K] bf16, w: [N, K] bf16, residual: [M, N] bf16
    (added in the epilogue when N is a multiple of 8)."""
    if a.shape[-1] % 8 != 0:
        y = torch.nn.functional.linear(a, w, bias)
        return y if residual is None else y + residual
    if residual is not None and (w.shape[0] % 8 != 0 or residual.dtype != torch.bfloat16):
        return _LinearFn.apply(a.contiguous(), w.contiguous(), bias) + residual
    return _LinearFn.apply(a.contiguous(), w.contiguous(), bias, None if residual is None else residual.contiguous())


class _Conv1x1Fn(torch.autograd.Function):
    """Stride-1 1x1 convolution of channels_last activations: forward and input gradient are the GEMMs
    [N*H*W, Cin] x [Cin, Cout] and [N*H*W, Cout] x [Cout, Cin] on the tcgen05 kernel; the filter
    gradient (a reduction over all pixels) is the split-K kernel of ``csrc/cuda/conv_tcgen05.cu``."""

    @staticmethod
    def forward(ctx, x, weight, col_stats=None):
        n, c, h, w = x.shape
        cout = weight.shape[0]
        ctx.save_for_backward(x, weight)
        a = x.permute(0, 2, 3, 1).reshape(n * h * w, c)                  # a view of NHWC memory
        y = _b.native.gemm_bf16_nt(a, weight.reshape(cout, c), None, 0, col_stats)
        return y.view(n, h, w, cout).permute(0, 3, 1, 2)                   # channels_last [N, Cout, H, W]

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        n, c, h, w = x.shape
        cout = weight.shape[0]
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            d2 = dy.permute(0, 2, 3, 1).reshape(n * h * w, cout)
            dx = _input_gradient(d2, weight.reshape(cout, c)).view(n, h, w, c).permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            C = _b.native
            if (hasattr(C, "conv_wgrad") and c % 64 == 0 and cout % 8 == 0
                    and C.conv_wgrad_supported(n, h, w, c, cout, 1)):
                # a reduction over all pixels into a handful of tiles: the split-K kernel with both operands pixel-major
                dw = C.conv_wgrad(dy, x, [0], [0], [0], 1, 1, False).view(cout, 1, 1, c).permute(0, 3, 1, 2)
            else:
                dw = torch.ops.aten.convolution_backward(dy, x, weight, None, (1, 1), (0, 0), (1, 1), False, (0, 0), 1,
                                                         (False, True, False))[1]
        return dx, dw, None


class _Conv1x1ForkFn(torch.autograd.Function):
    """``(conv1x1(x, w), x)``: the first convolution of a residual block together with the block's shortcut.  In the
    backward pass the gradient that arrives through the shortcut is added inside the epilogue of the input-gradient
    GEMM (fp32, before rounding), instead of autograd adding two full activation tensors in a pass of its own."""

    @staticmethod
    def forward(ctx, x, weight, col_stats=None):
        n, c, h, w = x.shape
        cout = weight.shape[0]
        ctx.save_for_backward(x, weight)
        a = x.permute(0, 2, 3, 1).reshape(n * h * w, c)
        y = _b.native.gemm_bf16_nt(a, weight.reshape(cout, c), None, 0, col_stats)
        return y.view(n, h, w, cout).permute(0, 3, 1, 2), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dshortcut):
        x, weight = ctx.saved_tensors
        n, c, h, w = x.shape
        cout = weight.shape[0]
        C = _b.native
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            d2 = dy.permute(0, 2, 3, 1).reshape(n * h * w, cout)
            add = None
            if dshortcut is not None:
                add = dshortcut.contiguous(memory_format=torch.channels_last).permute(0, 2, 3, 1).reshape(n * h * w, c)
            dx = C.gemm_bf16_nn(d2, weight.reshape(cout, c).contiguous(), add).view(n, h, w, c).permute(0, 3, 1, 2)
        if ctx.needs_input_grad[1]:
            dw = C.conv_wgrad(dy, x, [0], [0], [0], 1, 1, False).view(cout, 1, 1, c).permute(0, 3, 1, 2)
        return dx, dw, None


def conv1x1_fork_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    C = _b.native
    if not (conv1x1_supported(x, weight) and hasattr(C, "conv_wgrad")):
        return False
    n, c, h, w = x.shape
    return bool(c % 64 == 0 and weight.shape[0] % 8 == 0 and C.conv_wgrad_supported(n, h, w, c, weight.shape[0], 1))


def conv1x1_fork(x: torch.Tensor, weight: torch.Tensor, col_stats=None):
    """Returns ``(conv1x1(x, weight), shortcut)`` where ``shortcut`` equals ``x``; use ``shortcut`` for the residual
    connection of the block (see ``_Conv1x1ForkFn``).  Only where ``conv1x1_fork_supported``."""
    return _Conv1x1ForkFn.apply(x, weight, col_stats)


def conv1x1_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``conv1x1`` runs this input on the tcgen05 GEMM."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 4
            and x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0 and x.numel() > 0
            and x.is_contiguous(memory_format=torch.channels_last) and available())


def conv1x1(x: torch.Tensor, weight: torch.Tensor, col_stats=None) -> torch.Tensor:
    """``F.conv2d(x, weight)`` for a [Cout, Cin, 1, 1] filter and stride 1.  bf16 channels_last CUDA
    activations with Cin % 8 == 0 and Cout % 8 == 0 take the tcgen05 GEMM, the rest the library.
    ``col_stats`` (2*Cout fp32 values, only where ``conv1x1_supported``): the GEMM epilogue adds the
    per-channel sum and sum of squares of the output, the batch statistics of a following BatchNorm."""
    if conv1x1_supported(x, weight):
        return _Conv1x1Fn.apply(x, weight, col_stats)
    if col_stats is not None:
        raise ValueError("conv1x1: col_stats needs the tcgen05 path (see conv1x1_supported)")
    return torch.nn.functional.conv2d(x, weight)


class _MlpGeluFn(torch.autograd.Function):
    """y = gelu_tanh(a W1^T + b1) W2^T + b2 with both GELU passes inside GEMM epilogues: the first product
    stores its pre-activation next to the activated matrix, and the input gradient of the second product is
    multiplied by GELU'(pre-activation) before it is written."""

    @staticmethod
    def forward(ctx, a, w1, b1, w2, b2, residual=None):
        g, u = _b.native.gemm_bf16_nt_gelu(a, w1, b1)
        y = _b.native.gemm_bf16_nt(g, w2, b2, 0, None, residual)        # residual joins in the epilogue
        ctx.save_for_backward(a, w1, w2, u, g)
        ctx.has_bias = (b1 is not None, b2 is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        a, w1, w2, u, g = ctx.saved_tensors
        dy = dy.contiguous()
        C = _b.native
        du = C.gemm_bf16_nn_gelu_grad(dy, w2, u)                  # (dY W2) * GELU'(u)
        dw2 = _weight_gradient(dy, g)
        db2 = None
        if ctx.has_bias[1]:
            sums = fused_ln.take_column_sums(dy)
            db2 = (sums if sums is not None else C.column_sum(dy)).to(dy.dtype)
        da = _input_gradient(du, w1) if ctx.needs_input_grad[0] else None
        dw1 = _weight_gradient(du, a)
        db1 = C.column_sum(du).to(du.dtype) if ctx.has_bias[0] else None
        return da, dw1, db1, dw2, db2, (dy if ctx.needs_input_grad[5] else None)


# Rows up to which a weight gradient with few output tiles takes the split-K kernel of the convolution filter
# gradients.  With GPT-2 medium's 8192 rows that kernel needs 31 us for 1024 x 1024 and 67 us for 1024 x 3072
# against 15 and 36 us of the library's split-K product, which cost the step 1.9 ms; those go to the library.
_SPLITK_MAX_ROWS = 4096


def _weight_gradient(dy: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """dW[N, K] = dY[M, N]^T @ A[M, K].  Products with many output tiles take the TN kernel (one CTA per tile walks
    the whole reduction); products with few tiles and a reduction of at most ``_SPLITK_MAX_ROWS`` rows take the
    split-K kernel of the convolution filter gradients, which sees the rows as M images of one pixel; the rest is
    the library's."""
    n_out, k_in = dy.shape[1], a.shape[1]
    tiles = ((n_out + 127) // 128) * ((k_in + 255) // 256)
    C = _b.native
    if n_out % 8 == 0 and k_in % 8 == 0 and tiles >= _TN_MIN_TILES:
        return C.gemm_bf16_tn(dy, a)
    m = dy.shape[0]
    if (m <= _SPLITK_MAX_ROWS and hasattr(C, "conv_wgrad") and n_out % 8 == 0 and k_in % 64 == 0
            and dy.is_contiguous() and a.is_contiguous() and C.conv_wgrad_supported(m, 1, 1, k_in, n_out, 1)):
        return C.conv_wgrad(dy.view(m, n_out, 1, 1), a.view(m, k_in, 1, 1), [0], [0], [0], 1, 1, False).view(n_out, k_in)
    return dy.t() @ a


def mlp_gelu(a: torch.Tensor, w1: torch.Tensor, b1, w2: torch.Tensor, b2, residual=None) -> torch.Tensor:
    """``F.linear(F.gelu(F.linear(a, w1, b1), approximate="tanh"), w2, b2) (+ residual)`` for a bf16 CUDA matrix ``a``
    [M, K] on the tcgen05 kernels with the GELU (and the residual add) folded into the GEMM epilogues; other inputs
    take PyTorch's ops."""
    ok = (a.is_cuda and a.dim() == 2 and all(t.dtype == torch.bfloat16 for t in (a, w1, w2))
          and a.shape[1] % 8 == 0 and w1.shape[0] % 8 == 0 and w2.shape[0] % 8 == 0 and a.numel() > 0
          and (b1 is None or b1.dtype == torch.bfloat16) and (b2 is None or b2.dtype == torch.bfloat16)
          and available() and hasattr(_b.native, "gemm_bf16_nt_gelu"))
    if ok and (residual is None or (residual.dtype == torch.bfloat16 and residual.shape == (a.shape[0], w2.shape[0]))):
        return _MlpGeluFn.apply(a.contiguous(), w1.contiguous(), b1, w2.contiguous(), b2,
                                None if residual is None else residual.contiguous())
    h = torch.nn.functional.gelu(torch.nn.functional.linear(a, w1, b1), approximate="tanh")
    y = torch.nn.functional.linear(h, w2, b2)
    return y if residual is None else y + residual
