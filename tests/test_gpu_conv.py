"""tcgen05 implicit-GEMM convolutions (forward, input gradient, split-K filter gradient; 3x3 and 1x1, stride 1 and 2,
the space-to-depth stem) against fp32 convolutions of the same bf16 inputs."""
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
    assert conv.eligible(x1, w1, 1, 1)
    conv.conv3x3(x1, w1).backward(dy)
    x2, w2 = x.float().requires_grad_(True), wt.float().requires_grad_(True)
    F.conv2d(x2, w2, padding=1).backward(dy.float())
    _close(x1.grad, x2.grad, 1e-2)
    _close(w1.grad, w2.grad, 2e-2)
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("n,cin,cout,h,w,k,stride", [
    (4, 64, 64, 56, 56, 3, 1),        # 49-way split of the pixel patches, one 64-wide tile per tap group
    (3, 128, 128, 56, 56, 3, 2),      # stride 2: strided reads forward, four parity classes backward
    (5, 256, 256, 28, 28, 3, 2),
    (6, 512, 512, 14, 14, 3, 2),      # 7x7 outputs: two images per patch, the last patch hangs over the batch
    (4, 256, 512, 56, 56, 1, 2),      # strided shortcut convolution: three of four input positions get zero gradient
    (3, 512, 1024, 28, 28, 1, 2),
    (2, 128, 192, 9, 7, 3, 2),        # odd extents: the parity classes differ in size
    (2, 64, 128, 12, 10, 3, 1),       # no patch of a multiple of 16 positions in one image row block: whole images
    (7, 192, 64, 8, 8, 3, 1),         # Cin = 1.5 tiles of 128
])
def test_conv2d_autograd_all_products_match_fp32(n, cin, cout, h, w, k, stride):
    from bluefog_b200 import _C
    from bluefog_b200.ops import conv
    torch.manual_seed(h * 100 + cin + stride)
    pad = k // 2
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, k, k, device="cuda") / (k * cin ** 0.5)).to(torch.bfloat16)
    x1, w1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True)
    assert conv.eligible(x1, w1, stride, pad), "the shape should run on the tcgen05 kernels"
    before = _C.kernel_launch_count()
    y = conv.conv2d(x1, w1, stride, pad)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert _C.kernel_launch_count() - before >= 3
    x2, w2 = x.float().requires_grad_(True), wt.float().requires_grad_(True)
    ref = F.conv2d(x2, w2, stride=stride, padding=pad)
    ref.backward(dy.float())
    _close(y, ref.detach(), 1e-2)
    _close(x1.grad, x2.grad, 1e-2)
    _close(w1.grad, w2.grad, 2e-2)
    assert w1.grad.shape == wt.shape
    assert _C.gemm_status() == 0


def test_filter_gradient_leaves_its_scratch_clean():
    """The split-K scratch is shared by all layers and cleared by the kernel itself: a second, different layer right
    after the first must not see the first one's partial sums."""
    from bluefog_b200.ops import conv
    torch.manual_seed(3)
    outs = []
    for cin, cout, hw in ((64, 64, 56), (128, 64, 28), (64, 64, 56)):
        x = torch.randn(2, cin, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        dy = torch.randn(2, cout, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        g = conv.filter_gradient(dy, x, 3, 1, 1)
        ref = torch.ops.aten.convolution_backward(dy.float(), x.float(), torch.zeros(cout, cin, 3, 3, device="cuda"), None,
                                                  (1, 1), (1, 1), (1, 1), False, (0, 0), 1, (False, True, False))[1]
        _close(g, ref, 2e-2)


@pytest.mark.parametrize("plan", ["128,1,2,1", "256,1,4,1", "64,1,8,1", "128,1,2,2", "128,1,1,4", "64,3,1,6", "64,2,4,1"])
@pytest.mark.parametrize("k", [1, 3])
def test_filter_gradient_plans_cluster_and_workspace_splits(plan, k, monkeypatch):
    """Every way the reduction over pixels can be shared out - CTAs of one cluster adding up through distributed
    shared memory (third number), clusters or single CTAs adding up in the fp32 workspace (fourth number), several
    taps per MMA (second number) - gives the same filter gradient, and leaves the workspace clean."""
    from bluefog_b200 import _C
    from bluefog_b200.ops import conv
    if k == 1 and plan.split(",")[1] != "1":
        pytest.skip("a 1x1 filter has one tap")
    torch.manual_seed(11)
    n, cin, cout, hw = 16, 256, 192, 14
    x = torch.randn(n, cin, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    dy = torch.randn(n, cout, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    ref = torch.ops.aten.convolution_backward(dy.float(), x.float(), torch.zeros(cout, cin, k, k, device="cuda"), None,
                                              (1, 1), (k // 2, k // 2), (1, 1), False, (0, 0), 1, (False, True, False))[1]
    monkeypatch.setenv("BLUEFOG_B200_WGRAD_PLAN", plan)
    for _ in range(2):                       # twice: the second call finds the workspace as the first one left it
        g = conv.filter_gradient(dy, x, k, 1, k // 2)
        torch.cuda.synchronize()
        assert _C.gemm_status() == 0
        _close(g, ref, 2e-2)


@pytest.mark.parametrize("m,n_out,k_in", [(64, 1000, 2048), (200, 64, 128), (4096, 256, 64), (50, 72, 192)])
def test_linear_weight_gradient_through_the_split_k_kernel(m, n_out, k_in):
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    torch.manual_seed(m + n_out)
    dy = torch.randn(m, n_out, device="cuda").to(torch.bfloat16)
    a = torch.randn(m, k_in, device="cuda").to(torch.bfloat16)
    before = _C.kernel_launch_count()
    g = gemm._weight_gradient(dy, a)
    assert _C.kernel_launch_count() == before + 1
    _close(g, dy.float().t() @ a.float(), 1e-2)
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("n,hw", [(3, 224), (2, 64), (1, 32)])
def test_stem_convolution_matches_the_7x7_stride_2_convolution(n, hw):
    from bluefog_b200 import _C
    from bluefog_b200.models.resnet import StemConv
    torch.manual_seed(hw)
    stem = StemConv(space_to_depth=True).cuda().to(torch.bfloat16)
    x = torch.randn(n, 3, hw, hw, device="cuda")
    before = _C.kernel_launch_count()
    y = stem.forward_from_raw(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert _C.kernel_launch_count() - before >= 3       # input transform, forward, filter gradient
    w32 = stem.weight.detach().float().requires_grad_(True)
    ref = F.conv2d(x.to(torch.bfloat16).float(), w32, stride=2, padding=3)
    ref.backward(dy.float())
    _close(y, ref.detach(), 1e-2)
    _close(stem.weight.grad, w32.grad, 2e-2)
    assert _C.gemm_status() == 0


def test_global_average_pool_matches_fp32():
    from bluefog_b200.ops.fused_pool import global_avgpool
    x = torch.randn(5, 2048, 7, 7, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x1 = x.clone().requires_grad_(True)
    y = global_avgpool(x1)
    dy = torch.randn_like(y)
    y.backward(dy)
    x2 = x.float().requires_grad_(True)
    ref = x2.mean((2, 3))
    ref.backward(dy.float())
    _close(y, ref.detach(), 1e-2)
    _close(x1.grad, x2.grad, 1e-2)


def test_conv3x3_falls_back_for_unsupported_shapes():
    from bluefog_b200.ops import conv
    x = torch.randn(2, 3, 16, 16, device="cuda").to(torch.bfloat16)
    wt = torch.randn(8, 3, 3, 3, device="cuda").to(torch.bfloat16)
    assert not conv.eligible(x, wt)
    torch.testing.assert_close(conv.conv3x3(x, wt), F.conv2d(x, wt, padding=1))
