"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, w, bias, act):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == 1:
        y = torch.relu(y)
    elif act == 2:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    return y


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 512), (256, 384, 1024), (200, 136, 72),
                                   (1, 1000, 2048), (3136, 64, 256), (4096, 4096, 1024), (777, 50264, 64),
                                   (130, 100, 64), (20000, 256, 64), (12544, 1000, 256)])
@pytest.mark.parametrize("with_bias,act", [(False, 0), (True, 1), (True, 2)])
def test_gemm_matches_fp32_reference(M, N, K, with_bias, act):
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    assert gemm.available(), "the tcgen05 GEMM must be usable on a B200 box"
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, generator=g) * 0.5).cuda().to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.5).cuda().to(torch.bfloat16)
    bias = torch.randn(N, generator=g).cuda().to(torch.bfloat16) if with_bias else None
    out = _C.gemm_bf16_nt(a, w, bias, act)
    torch.cuda.synchronize()
    assert _C.gemm_status() == 0, "a bounded wait inside the kernel expired"
    ref = _ref(a, w, bias, act)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (M, N, K, err, scale)


def test_linear_autograd_matches_torch():
    from bluefog_b200.ops import gemm
    torch.manual_seed(0)
    a = torch.randn(300, 256, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(512, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = gemm.linear(a, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    a2, w2, b2 = (t.detach().float().requires_grad_(True) for t in (a, w, b))
    y2 = torch.nn.functional.linear(a2, w2, b2)
    y2.backward(gy.float())
    for got, ref in ((y, y2), (a.grad, a2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("n,cin,cout,h,w", [(4, 64, 256, 56, 56), (3, 1024, 256, 14, 14), (2, 72, 40, 9, 7)])
def test_conv1x1_autograd_matches_fp32(n, cin, cout, h, w):
    import torch.nn.functional as F
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    torch.manual_seed(cin + cout)
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, 1, 1, device="cuda") / cin ** 0.5).to(torch.bfloat16)
    dy = torch.randn(n, cout, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x1, w1 = x.clone().requires_grad_(True), wt.clone().requires_grad_(True)
    y1 = gemm.conv1x1(x1, w1)
    assert y1.is_contiguous(memory_format=torch.channels_last)
    y1.backward(dy)
    x2, w2 = x.float().requires_grad_(True), wt.float().requires_grad_(True)
    y2 = F.conv2d(x2, w2)
    y2.backward(dy.float())

    def close(a, ref, tol):
        err = (a.float() - ref).abs().max().item()
        assert err <= tol * max(1.0, ref.abs().max().item()), err

    close(y1, y2, 1e-2)
    close(x1.grad, x2.grad, 1e-2)
    close(w1.grad, w2.grad, 2e-2)
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 128, 128), (512, 256, 256), (1000, 200, 72), (4096, 1024, 4096),
                                   (12544, 256, 1024), (300, 520, 136)])
def test_gemm_nn_reads_row_major_b_as_mn_major_operand(M, N, K):
    """a[M,K] @ b[K,N] with b in its row-major memory (the input-gradient product dY @ W)."""
    from bluefog_b200 import _C
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.5).to(torch.bfloat16)
    out = _C.gemm_bf16_nn(a, b).float()
    ref = a.float() @ b.float()
    err = (out - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()), err
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("K,M,N", [(64, 128, 64), (256, 256, 256), (1000, 200, 72), (8192, 4096, 1024), (4100, 1024, 3072)])
def test_gemm_tn_reads_both_operands_mn_major(K, M, N):
    """a[K,M]^T @ b[K,N] with both matrices in their row-major memory (the weight-gradient product dY^T X)."""
    from bluefog_b200 import _C
    torch.manual_seed(M + N + K)
    a = (torch.randn(K, M, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.5).to(torch.bfloat16)
    out = _C.gemm_bf16_tn(a, b).float()
    ref = a.float().t() @ b.float()
    err = (out - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()), err
    assert _C.gemm_status() == 0


def test_linear_backward_runs_all_three_products_on_the_kernel():
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    torch.manual_seed(3)
    a = (torch.randn(2048, 1024, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(4096, 1024, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)   # 32 x 4 output tiles
    b = torch.zeros(4096, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(2048, 4096, device="cuda").to(torch.bfloat16)
    before = _C.kernel_launch_count()
    gemm.linear(a, w, b).backward(dy)
    assert _C.kernel_launch_count() - before >= 4          # forward, input gradient, weight gradient, bias gradient
    a2, w2 = a.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    torch.nn.functional.linear(a2, w2).backward(dy.float())
    for got, ref in ((a.grad, a2.grad), (w.grad, w2.grad), (b.grad, dy.float().sum(0))):
        assert (got.float() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,K,H", [(512, 256, 1024), (8192, 1024, 4096), (300, 72, 136)])
def test_mlp_gelu_with_epilogue_fusion_matches_fp32(M, K, H):
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    import torch.nn.functional as F
    torch.manual_seed(M + K + H)
    mk = lambda *s, scale=1.0: (torch.randn(*s, device="cuda") * scale).to(torch.bfloat16).requires_grad_(True)
    a, w1, b1, w2, b2 = mk(M, K), mk(H, K, scale=K ** -0.5), mk(H, scale=0.1), mk(K, H, scale=H ** -0.5), mk(K, scale=0.1)
    dy = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    y = gemm.mlp_gelu(a, w1, b1, w2, b2)
    y.backward(dy)
    ref_in = [t.detach().float().requires_grad_(True) for t in (a, w1, b1, w2, b2)]
    yr = F.linear(F.gelu(F.linear(ref_in[0], ref_in[1], ref_in[2]), approximate="tanh"), ref_in[3], ref_in[4])
    yr.backward(dy.float())
    for name, got, ref in [("y", y, yr)] + [(n, t.grad, r.grad) for n, t, r in zip("a w1 b1 w2 b2".split(), (a, w1, b1, w2, b2), ref_in)]:
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * max(1.0, ref.abs().max().item()), (name, err, ref.abs().max().item())
    assert _C.gemm_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 136, 72), (3136, 64, 256), (130, 104, 64), (51200, 256, 64),
                                   (12544, 1024, 256), (40000, 512, 128), (33, 2048, 512)])
def test_gemm_epilogue_column_statistics_match_the_stored_output(M, N, K):
    """The sums that a following BatchNorm consumes are those of the rounded bf16 output, taken in the epilogue;
    they are added to what the buffer held before."""
    from bluefog_b200 import _C
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5 + 0.1).cuda().to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.5).cuda().to(torch.bfloat16)
    stats = torch.full((2 * N,), 3.0, device="cuda")
    out = _C.gemm_bf16_nt(a, w, None, 0, stats)
    torch.cuda.synchronize()
    assert _C.gemm_status() == 0
    plain = _C.gemm_bf16_nt(a, w, None, 0)
    assert torch.equal(out, plain)
    o = out.double()
    s1, s2 = o.sum(0), (o * o).sum(0)
    got1, got2 = stats[:N].double() - 3.0, stats[N:].double() - 3.0
    assert (got1 - s1).abs().max().item() <= 1e-4 * o.abs().sum(0).max().item() + 1e-3
    assert (got2 - s2).abs().max().item() <= 1e-4 * s2.max().item() + 1e-3


def test_batchnorm_fed_by_the_gemm_statistics_matches_its_own_pass():
    from bluefog_b200 import _C
    from bluefog_b200.models.resnet import Conv1x1, MixedBatchNorm2d
    from bluefog_b200.ops.fused_bn import bn_act
    torch.manual_seed(5)
    results = []
    # a channel-reducing convolution: the kind whose statistics the model takes in the GEMM epilogue
    x0 = (torch.randn(8, 256, 14, 14) + 0.3).cuda().to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn(8, 64, 14, 14).cuda().to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    conv = Conv1x1(256, 64, use_b200_gemm=True).cuda().to(torch.bfloat16)
    bn = MixedBatchNorm2d(64).cuda()
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.5, 0.5)
    for fused in (True, False):
        bn.running_mean.zero_()
        bn.running_var.fill_(1.0)
        x = x0.clone().requires_grad_(True)
        conv.weight.grad = bn.weight.grad = bn.bias.grad = None
        if fused:
            launches = _C.kernel_launch_count() if hasattr(_C, "kernel_launch_count") else None
            y = conv.forward_bn_act(x, bn, relu=True, residual=res)
            if launches is not None:     # GEMM + apply: no statistics kernel
                assert _C.kernel_launch_count() - launches == 2
        else:
            y = bn_act(conv(x), bn, relu=True, residual=res)
        y.float().square().sum().backward()
        results.append((y.detach().float(), x.grad.float(), conv.weight.grad.float(), bn.weight.grad.float(),
                        bn.running_mean.clone(), bn.running_var.clone()))
    for got, want in zip(*results):
        assert (got - want).norm().item() <= 2e-2 * want.norm().item() + 1e-3


def test_two_sm_mode_on_ragged_shapes_in_a_process_of_its_own():
    """BLUEFOG_B200_GEMM_PAIR=1 sends every eligible product (M, N >= 256) to the cta_group::2 mode, also shapes
    whose edges fall inside a 256 x 256 pair tile; the switch is read once per process, hence the child process."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from bluefog_b200 import _C
torch.manual_seed(5)
for M, N, K in [(304, 264, 72), (1000, 520, 200), (520, 1032, 1024)]:
    a = (torch.randn(M, K) * 0.5).cuda().to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.5).cuda().to(torch.bfloat16)
    b = (torch.randn(K, N) * 0.5).cuda().to(torch.bfloat16)
    bias = torch.randn(N).cuda().to(torch.bfloat16)
    at = (torch.randn(K, M) * 0.5).cuda().to(torch.bfloat16)
    cases = [(_C.gemm_bf16_nt(a, w, bias, 1), torch.relu(a.float() @ w.float().t() + bias.float())),
             (_C.gemm_bf16_nn(a, b), a.float() @ b.float()),
             (_C.gemm_bf16_tn(at, b), at.float().t() @ b.float())]
    torch.cuda.synchronize()
    assert _C.gemm_status() == 0
    for out, ref in cases:
        err = (out.float() - ref).abs().max().item()
        assert err <= 1e-2 * ref.abs().max().item() + 1e-2, (M, N, K, err)
print("ok")
'''
    env = dict(os.environ, BLUEFOG_B200_GEMM_PAIR="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stdout[-500:] + out.stderr[-1500:]


@pytest.mark.parametrize("M,K,N", [(512, 256, 384), (8192, 1024, 1024), (300, 72, 136)])
def test_linear_with_the_residual_added_in_the_epilogue(M, K, N):
    """out = a w^T + bias + residual from one kernel; gradients of all four inputs against fp32 autograd."""
    from bluefog_b200 import _C
    from bluefog_b200.ops import gemm
    torch.manual_seed(M + N)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(N, device="cuda").to(torch.bfloat16).requires_grad_(True)
    r = torch.randn(M, N, device="cuda").to(torch.bfloat16).requires_grad_(True)
    before = _C.kernel_launch_count()
    y = gemm.linear(a, w, b, r)
    assert _C.kernel_launch_count() == before + 1            # no separate addition
    gy = torch.randn_like(y)
    y.backward(gy)
    a2, w2, b2, r2 = (t.detach().float().requires_grad_(True) for t in (a, w, b, r))
    y2 = a2 @ w2.t() + b2 + r2
    y2.backward(gy.float())
    torch.cuda.synchronize()
    assert _C.gemm_status() == 0
    for got, ref in [(y, y2), (a.grad, a2.grad), (w.grad, w2.grad), (b.grad, b2.grad), (r.grad, r2.grad)]:
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 2e-2, err
