"""Convolutions on the tcgen05 implicit-GEMM kernels, with autograd.

``conv2d(x, weight, stride, padding)`` has the contract of ``F.conv2d`` for bf16 channels_last CUDA
activations, a square ``[Cout, Cin, R, R]`` filter with ``R*R <= 16`` taps, stride 1 or 2, and channel counts
that are multiples of 64.  All three products run on ``csrc/cuda/conv_tcgen05.cu``:

* forward: one implicit GEMM over the filter taps (strided reads for stride 2);
* input gradient: stride 1 - the same kernel on (dy, the same filter) with mirrored taps and the filter read in
  place as an MN-major operand (the channel axes swap roles without a transposed copy); stride 2 - one launch per
  parity class of the input position, each over the taps that reach that class, stored with stride 2;
* filter gradient: the split-K kernel that reduces over pixel patches with both operands position-major.

Stride-1 1x1 convolutions are plain GEMMs and take ``ops.gemm.conv1x1`` (the persistent GEMM) for the forward
pass and the input gradient; their filter gradient takes the split-K kernel of this module.
``stem_conv`` is the 7x7 / stride 2 stem evaluated as a 4x4 convolution over a space-to-depth image.

Everything else takes ``F.conv2d``.  The reference has no convolution code of its own
(examples/pytorch_benchmark.py:100 uses torchvision on cuDNN).
"""
import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()


def available() -> bool:
    C = _b.native
    return bool(torch.cuda.is_available() and hasattr(C, "conv_igemm") and C.gemm_supported())


def _out_size(n, k, stride, pad):
    return (n + 2 * pad - k) // stride + 1


def eligible(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, padding: int = 1) -> bool:
    """Whether ``conv2d`` runs forward, input gradient and filter gradient of this call on the tcgen05 kernels."""
    if not (x.is_cuda and x.dim() == 4 and weight.dim() == 4 and x.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16 and weight.shape[1] == x.shape[1] and weight.shape[2] == weight.shape[3]
            and stride in (1, 2) and available()):
        return False
    n, cin, h, w = x.shape
    cout, k = weight.shape[0], weight.shape[2]
    if k * k > 16 or cin % 64 or cout % 64 or padding < 0 or padding > k // 2:
        return False
    ho, wo = _out_size(h, k, stride, padding), _out_size(w, k, stride, padding)
    if ho < 1 or wo < 1:
        return False
    C = _b.native
    ok = C.conv_igemm_supported(n, ho, wo, cin, cout, stride) and C.conv_wgrad_supported(n, ho, wo, cin, cout, stride)
    if stride == 1:
        return bool(ok and C.conv_igemm_supported(n, h, w, cout, cin, 1))
    return bool(ok and C.conv_igemm_supported(n, (h + 1) // 2, (w + 1) // 2, cout, cin, 1))


def _forward_taps(k, pad):
    dh = [r - pad for r in range(k) for _ in range(k)]
    dw = [s - pad for _ in range(k) for s in range(k)]
    return dh, dw, list(range(k * k))


def filter_gradient(dy, x, k, stride, pad, stem_view=False):
    """dW [Cout, Cin, k, k] (channels_last memory) of a convolution with output gradient ``dy`` and input ``x``."""
    dh, dw, wt = _forward_taps(k, pad)
    g = _b.native.conv_wgrad(dy, x, dh, dw, wt, k * k, stride, stem_view)          # [Cout, k*k, Cin]
    return g.view(g.shape[0], k, k, g.shape[2]).permute(0, 3, 1, 2)


def forward_product(x, wk, stride, pad):
    """y = conv(x, w) for channels_last ``x`` and the filter in channels_last memory ``wk`` [Cout, Cin, k, k]."""
    n, cin, h, w = x.shape
    cout, k = wk.shape[0], wk.shape[2]
    ho, wo = _out_size(h, k, stride, pad), _out_size(w, k, stride, pad)
    y = torch.empty((n, cout, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    dh, dw, wt = _forward_taps(k, pad)
    return _b.native.conv_igemm(x, wk, y, ho, wo, dh, dw, wt, k * k, stride, 0)


def input_gradient(dy, wk, x_shape, stride, pad):
    """dX of a convolution with output gradient ``dy``.  The forward filter [Cout, k, k, Cin] is read in place as an
    MN-major operand: its reduction channels (Cout) are the outer dimension here."""
    C = _b.native
    n, cin, h, w = x_shape
    k = wk.shape[2]
    if stride == 1:
        dx = torch.empty(x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        dh = [pad - r for r in range(k) for _ in range(k)]
        dw = [pad - s for _ in range(k) for s in range(k)]
        return C.conv_igemm(dy, wk, dx, h, w, dh, dw, list(range(k * k)), k * k, 1, 1)
    # input position (2a + ph, 2b + pw) is reached by the taps with (ph + pad - r) and (pw + pad - s) even
    classes = []
    for ph in range(2):
        for pw in range(2):
            taps = [(r, s) for r in range(k) for s in range(k) if (ph + pad - r) % 2 == 0 and (pw + pad - s) % 2 == 0]
            classes.append((ph, pw, taps))
    covered = all(taps for _, _, taps in classes)      # a 1x1 filter reaches only the even positions
    dx = torch.empty(x_shape, dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
    if not covered:
        dx.zero_()
    for ph, pw, taps in classes:
        ha, wa = (h - ph + 1) // 2, (w - pw + 1) // 2
        if not taps or ha == 0 or wa == 0:
            continue
        C.conv_igemm(dy, wk, dx, ha, wa, [(ph + pad - r) // 2 for r, _ in taps], [(pw + pad - s) // 2 for _, s in taps],
                     [r * k + s for r, s in taps], k * k, 1, 1, 2, ph, pw)
    return dx


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, stride, pad):
        x = x.contiguous(memory_format=torch.channels_last)
        wk = weight.contiguous(memory_format=torch.channels_last)          # [Cout, k, k, Cin] in memory
        ctx.save_for_backward(x, weight)
        ctx.conv = (stride, pad)
        return forward_product(x, wk, stride, pad)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        stride, pad = ctx.conv
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dwt = None
        if ctx.needs_input_grad[0]:
            dx = input_gradient(dy, weight.contiguous(memory_format=torch.channels_last), x.shape, stride, pad)
        if ctx.needs_input_grad[1]:
            dwt = filter_gradient(dy, x, weight.shape[2], stride, pad)
        return dx, dwt, None, None


def conv2d(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, padding: int = 0) -> torch.Tensor:
    if eligible(x, weight, stride, padding):
        return _ConvFn.apply(x, weight, stride, padding)
    return F.conv2d(x, weight, stride=stride, padding=padding)


def conv3x3(x: torch.Tensor, weight: torch.Tensor, stride: int = 1) -> torch.Tensor:
    return conv2d(x, weight, stride, 1)


class _StemFn(torch.autograd.Function):
    """4x4 / stride 1 convolution of a 16-channel space-to-depth image [N, 16, Hb, Wb] with a [64, 16, 4, 4] filter;
    the image needs no gradient."""

    @staticmethod
    def forward(ctx, xs, w16):
        n, _, hb, wb = xs.shape
        wk = w16.contiguous(memory_format=torch.channels_last)             # [64, 4, 4, 16]: row r holds 4 x 16 values
        ctx.save_for_backward(xs)
        y = torch.empty((n, w16.shape[0], hb - 3, wb - 3), dtype=xs.dtype, device=xs.device,
                        memory_format=torch.channels_last)
        return _b.native.conv_igemm(xs, wk, y, hb - 3, wb - 3, [0, 1, 2, 3], [0, 0, 0, 0], [0, 1, 2, 3], 4, 1, 0, 1, 0, 0, True)

    @staticmethod
    def backward(ctx, dy):
        (xs,) = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        g = _b.native.conv_wgrad(dy, xs, [0, 1, 2, 3], [0, 0, 0, 0], [0, 1, 2, 3], 4, 1, True)   # [64, 4, 64]
        return None, g.view(g.shape[0], 4, 4, 16).permute(0, 3, 1, 2)


def stem_eligible(xs: torch.Tensor, w16: torch.Tensor) -> bool:
    if not (xs.is_cuda and xs.dtype == torch.bfloat16 and w16.dtype == torch.bfloat16 and xs.dim() == 4
            and xs.shape[1] == 16 and tuple(w16.shape[1:]) == (16, 4, 4) and w16.shape[0] % 64 == 0
            and xs.is_contiguous(memory_format=torch.channels_last) and not xs.requires_grad and available()):
        return False
    n, _, hb, wb = xs.shape
    if hb < 4 or wb < 4:
        return False
    C = _b.native
    return bool(C.conv_igemm_supported(n, hb - 3, wb - 3, 64, w16.shape[0], 1)
                and C.conv_wgrad_supported(n, hb - 3, wb - 3, 64, w16.shape[0], 1))


def stem_conv(xs: torch.Tensor, w16: torch.Tensor) -> torch.Tensor:
    """``F.conv2d(xs, w16)`` for the space-to-depth stem (see ``models.resnet.StemConv``)."""
    if stem_eligible(xs, w16):
        return _StemFn.apply(xs, w16)
    return F.conv2d(xs, w16)
