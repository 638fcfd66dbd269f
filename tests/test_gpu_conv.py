"""tcgen05 implicit-GEMM 3x3 convolution against an fp32 convolution of the same bf16 inputs."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _inputs(n, cin, cout, h, w):
    torch.manual_seed(n * 1000 + cin + cout + h)
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, 3, 3, device="cuda") / (3.0 * cin ** 0.5)).to(torch.bfloat16)
    return x, wt


def _close(a, ref, tol):
    err = (a.float() - ref).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, (err, bound)


@pytest.mark.parametrize("n,cin,cout,h,w", [
    (2, 64, 64, 56, 56),       # patch 56 x 2
    (3, 128, 128, 28, 28),     # patch 28 x 4
    (5, 256, 256, 14, 14),     # patch 14 x 7
    (5, 512, 512, 7, 7),       # two images per patch, odd batch: the last patch hangs over the batch
    (1, 64, 192, 9, 5),        # tiny image; Cout = 1.5 output tiles of 128
    (2, 64, 72, 30, 20),       # rows of the last patch hang over the image; Cout % 64 != 0
    (4, 128, 320, 16, 16),     # 256-wide and partial output tiles
    (8, 256, 256, 4, 4),       # whole images, eight per patch
    (8, 512, 512, 2, 2),       # 2x2 images: every tap but the centre one is mostly padding
    (3, 64, 64, 1, 1),         # a single pixel per image
])
def test_conv3x3_forward_and_input_gradient(n, cin, cout, h, w):
    from bluefog_b200 import _C
    from bluefog_b200.ops import conv
    x, wt = _inputs(n, cin, cout, h, w)
    if not conv.available():
        pytest.fail("the native module has no tcgen05 convolution on this GPU")
    assert _C.conv3x3_supported(n, h, w, cin, cout)
    y = _C.conv3x3_nhwc(x, wt.contiguous(memory_format=torch.channels_last))
    ref = F.conv2d(x.float(), wt.float(), padding=1)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    _close(y, ref, 1e-2)
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("n,cin,cout,h,w", [(2, 64, 64, 56, 56), (3, 128, 256, 14, 14), (4, 512, 512, 7, 7),
                                           (8, 512, 512, 2, 2), (8, 128, 128, 8, 8), (5, 64, 320, 16, 16)])
def test_conv3x3_autograd_matches_fp32(n, cin, cout, h, w):
    from bluefog_b200 import _C
    from bluefog_b200.ops import conv
    x, wt = _inputs(n, cin, cout, h, w)
    dy = torch.randn(n, cout, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x1, w1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True)
    assert conv.eligible(x1, w1)
    conv.conv3x3(x1, w1).backward(dy)
    x2, w2 = x.float().requires_grad_(True), wt.float().requires_grad_(True)
    F.conv2d(x2, w2, padding=1).backward(dy.float())
    _close(x1.grad, x2.grad, 1e-2)
    _close(w1.grad, w2.grad, 2e-2)
    assert _C.gemm_status() == 0


def test_conv3x3_falls_back_for_unsupported_shapes():
    from bluefog_b200.ops import conv
    x = torch.randn(2, 3, 16, 16, device="cuda").to(torch.bfloat16)
    wt = torch.randn(8, 3, 3, 3, device="cuda").to(torch.bfloat16)
    assert not conv.eligible(x, wt)
    torch.testing.assert_close(conv.conv3x3(x, wt), F.conv2d(x, wt, padding=1))
