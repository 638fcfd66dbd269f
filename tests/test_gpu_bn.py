"""Fused BatchNorm+ReLU(+residual) kernels against PyTorch in fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _case(N, C, H, W, relu, with_res, param_dtype):
    from bluefog_b200.ops.fused_bn import bn_act
    torch.manual_seed(C + H)
    dev = torch.device("cuda", 0)
    x = (torch.randn(N, C, H, W, device=dev) * 1.5 + 0.7).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn(N, C, H, W, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last) if with_res else None
    bn = torch.nn.BatchNorm2d(C).to(dev)
    with torch.no_grad():
        bn.weight.copy_(torch.rand(C, device=dev) + 0.5)
        bn.bias.copy_(torch.randn(C, device=dev) * 0.2)
    ref_bn = torch.nn.BatchNorm2d(C).to(dev)
    ref_bn.load_state_dict(bn.state_dict())
    if param_dtype == torch.bfloat16:
        bn.weight.data = bn.weight.data.to(torch.bfloat16)
        bn.bias.data = bn.bias.data.to(torch.bfloat16)
        with torch.no_grad():
            ref_bn.weight.copy_(bn.weight.float())
            ref_bn.bias.copy_(bn.bias.float())
    x1 = x.clone().requires_grad_(True)
    r1 = res.clone().requires_grad_(True) if with_res else None
    y = bn_act(x1, bn, relu=relu, residual=r1)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2 = x.float().requires_grad_(True)
    r2 = res.float().requires_grad_(True) if with_res else None
    z = ref_bn(x2)
    if with_res:
        z = z + r2
    y2 = F.relu(z) if relu else z
    y2.backward(gy.float())
    torch.cuda.synchronize()

    def close(a, b, tol, outliers=0.0):
        """max-abs check; ``outliers`` = fraction of elements allowed to miss it.  An activation
        that lands within rounding distance of zero may get a different ReLU mask in bf16 than in
        the fp32 reference, which changes its gradient by the whole upstream value."""
        err = (a.float() - b).abs()
        bound = tol * max(1.0, b.abs().max().item())
        bad = (err > bound).float().mean().item()
        assert bad <= outliers, (err.max().item(), bound, bad)

    close(y, y2, 2e-2)
    # the kernel's ReLU bits come from its own fp32 value of bf16 inputs; compare gradients where both agree
    close(x1.grad, x2.grad, 4e-2, outliers=1e-4 if relu else 0.0)
    if with_res:
        close(r1.grad, r2.grad, 2e-2, outliers=1e-4 if relu else 0.0)
    close(bn.weight.grad, ref_bn.weight.grad, 3e-2)
    close(bn.bias.grad, ref_bn.bias.grad, 3e-2)
    close(bn.running_mean, ref_bn.running_mean, 1e-2)
    close(bn.running_var, ref_bn.running_var, 1e-2)
    assert int(bn.num_batches_tracked) == 1


# sizes on both sides of the limits of the one-launch kernels: rows of x (and of dz) kept in shared memory, rows of x
# only (25.7 MB), and the two-kernel form (102.8 MB)
@pytest.mark.parametrize("N,C,H,W", [(4, 64, 56, 56), (8, 256, 14, 14), (2, 2048, 7, 7), (3, 128, 9, 5), (64, 64, 112, 112),
                                     (64, 64, 56, 56), (64, 128, 28, 28), (1, 8, 3, 3)])
@pytest.mark.parametrize("relu,with_res", [(True, False), (True, True), (False, False)])
def test_fused_bn_matches_pytorch(N, C, H, W, relu, with_res):
    _case(N, C, H, W, relu, with_res, torch.float32)


@pytest.mark.parametrize("N,C,H,W", [(64, 512, 7, 7), (64, 256, 14, 14), (64, 1024, 14, 14)])
def test_one_launch_and_two_kernel_forms_agree(N, C, H, W):
    """The same layer with a barrier word behind the sums (one cooperative launch per pass) and without (statistics
    kernel + apply kernel): same results up to the order of the fp32 sums, and the launch counts say which ran."""
    from bluefog_b200 import _C
    dev = torch.device("cuda", 0)
    torch.manual_seed(C)
    x = (torch.randn(N, C, H, W, device=dev) + 0.3).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn_like(x)
    dy = torch.randn_like(x)
    gamma, beta = torch.rand(C, device=dev) + 0.5, torch.randn(C, device=dev)
    outs = []
    for words in (_C.bn_workspace_floats(C), 2 * C + 1, 2 * C):
        before = _C.kernel_launch_count()
        y, mean, rstd, mask = _C.bn_forward(x, res, gamma, beta, None, None, 1e-5, 0.1, True, torch.zeros(words, device=dev))
        dx, dres, dgamma, dbeta = _C.bn_backward(dy, mask, x, mean, rstd, gamma, True, True, torch.zeros(words, device=dev))
        torch.cuda.synchronize()
        assert _C.kernel_launch_count() - before == (2 if words > 2 * C else 4)
        assert _C.gemm_status() == 0
        outs.append((y, mean, rstd, dx, dres, dgamma, dbeta))
    for a, b in list(zip(outs[0], outs[2])) + list(zip(outs[1], outs[2])):
        # an activation within rounding distance of zero may get a different ReLU bit from differently ordered sums
        scale = max(1.0, b.float().abs().max().item())
        bad = ((a.float() - b.float()).abs() > 2e-2 * scale).float().mean().item()
        assert bad <= 1e-5, bad


@pytest.mark.parametrize("big", [False, True])
def test_gradient_pairs_equal_autograd_addition(big):
    """Two bottlenecks in a row: the gradients of the second block's input (through its first convolution and
    through its shortcut) reach the first block's last BatchNorm as a pair; the result must be what autograd's own
    addition gives.  ``big`` takes the two-kernel form of the BatchNorm backward (51 MB activations)."""
    from bluefog_b200.models import resnet
    from bluefog_b200.ops import fused_bn
    dev = torch.device("cuda", 0)
    n, hw = (64, 56) if big else (8, 14)
    grads = []
    for pairs in (True, False):
        torch.manual_seed(3)
        blocks = torch.nn.Sequential(resnet.Bottleneck(256, 64, 1, resnet.Downsample(256, 256, 1, True), True, True),
                                     resnet.Bottleneck(256, 64, 1, None, True, True)).to(dev)
        blocks = blocks.to(memory_format=torch.channels_last).train()
        for prm in blocks.parameters():                      # bf16 parameters, fp32 running statistics
            prm.data = prm.data.to(torch.bfloat16)
        x = torch.randn(n, 256, hw, hw, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        x.requires_grad_(True)
        fused_bn.PAIR_GRADIENTS = pairs
        try:
            fused_bn.begin_step(dev)
            y = blocks(x)
            y.float().square().mean().backward()
        finally:
            fused_bn.PAIR_GRADIENTS = True
        torch.cuda.synchronize()
        assert not fused_bn._pending_pairs
        grads.append([x.grad.float()] + [p.grad.float() for p in blocks.parameters()])
    for a, b in zip(*grads):
        scale = max(b.abs().max().item(), 1e-6)
        # the pair is added in fp32, autograd's sum is rounded to bf16 first: a few ReLU bits may differ
        assert ((a - b).abs() > 3e-2 * scale).float().mean().item() <= 1e-3, (a - b).abs().max().item() / scale


def test_fused_bn_with_bf16_parameters():
    _case(8, 512, 7, 7, True, True, torch.bfloat16)


def test_eval_mode_and_unsupported_inputs_fall_back():
    from bluefog_b200.ops.fused_bn import bn_act
    bn = torch.nn.BatchNorm2d(24).cuda().eval()
    x = torch.randn(2, 24, 5, 5, device="cuda")
    assert torch.allclose(bn_act(x, bn, relu=True), F.relu(bn(x)))
    bn.train()
    x16 = torch.randn(2, 24, 5, 5, device="cuda").to(torch.bfloat16)   # NCHW, C/8 does not divide 256
    out = bn_act(x16, bn.to(torch.bfloat16), relu=False)
    assert out.shape == x16.shape


@pytest.mark.parametrize("shape", [(2, 64, 112, 112), (3, 8, 7, 9), (1, 128, 5, 5), (4, 64, 56, 57)])
def test_maxpool_matches_pytorch(shape):
    from bluefog_b200.ops.fused_pool import maxpool3x3s2
    torch.manual_seed(shape[2])
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x1 = x.clone().requires_grad_(True)
    y = maxpool3x3s2(x1)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2 = x.float().requires_grad_(True)
    y2 = F.max_pool2d(x2, 3, 2, 1)
    y2.backward(gy.float())
    torch.cuda.synchronize()
    assert y.shape == y2.shape
    assert torch.equal(y.float(), y2)
    # bf16 inputs contain ties; PyTorch also sends the gradient to the first maximum in scan order
    assert (x1.grad.float() - x2.grad).abs().max().item() <= 2e-2 * max(1.0, x2.grad.abs().max().item())
