"""Model-level GPU tests on one device: fused optimizer vs torch.optim, CUDA-graph step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bf():
    import bluefog_b200.torch as bf
    bf.init()
    yield bf


@pytest.fixture
def exact_fp32_convolutions():
    """fp32 convolutions on TF32 tensor cores round differently from one algorithm to the next, and the
    library's choice depends on the allocator state left by earlier tests; comparisons of two fp32
    models need true fp32 arithmetic."""
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32 = old


def test_fused_sgd_single_rank_matches_torch_sgd(bf, exact_fp32_convolutions):
    from bluefog_b200.models import resnet
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    m1 = resnet.resnet18(num_classes=10).to(dev)
    m2 = resnet.resnet18(num_classes=10).to(dev)
    m2.load_state_dict(m1.state_dict())
    o1 = torch.optim.SGD(m1.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    o2 = bf.DistributedNeighborAllreduceOptimizer(
        torch.optim.SGD(m2.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4), m2)
    assert type(o2).__name__ == "SGD" and isinstance(o2, torch.optim.SGD) and hasattr(o2, "master_parameters")
    x = torch.randn(4, 3, 32, 32, device=dev)
    y = torch.randint(0, 10, (4,), device=dev)
    # Both optimizers get the SAME gradients (those of the fused model), so that the comparison is about
    # the update arithmetic and not about which convolution algorithm the library picked for which copy.
    for _ in range(3):
        o1.zero_grad()
        o2.zero_grad()
        torch.nn.functional.cross_entropy(m2(x), y).backward()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            p1.grad = p2.grad.detach().clone()
        o1.step()
        o2.step()
        torch.cuda.synchronize()
        o2.check()
        for (n1, p1), (n2, p2) in zip(m1.named_parameters(), m2.named_parameters()):
            assert torch.allclose(p1, p2, rtol=1e-5, atol=1e-6), (n1, (p1 - p2).abs().max().item())
    sd = o2.state_dict()
    assert "momentum_buffer" in sd["state"][0]


def test_bf16_compute_keeps_fp32_master_and_checkpoint_names(bf, tmp_path):
    from bluefog_b200.models import resnet
    dev = torch.device("cuda", 0)
    model = resnet.resnet18(num_classes=10).to(dev).to(memory_format=torch.channels_last)
    opt = bf.DistributedAdaptWithCombineOptimizer(torch.optim.AdamW(model.parameters(), lr=1e-3), model,
                                                  compute_dtype=torch.bfloat16)
    assert model.conv1.weight.dtype == torch.bfloat16
    x = torch.randn(8, 3, 32, 32, device=dev)
    y = torch.randint(0, 10, (8,), device=dev)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    masters = opt.master_parameters()
    assert masters["conv1.weight"].dtype == torch.float32
    path = str(tmp_path / "ck.pth.tar")
    bf.save_checkpoint(path, model, opt)
    payload = torch.load(path, weights_only=False)
    assert payload["model"]["conv1.weight"].dtype == torch.float32
    assert set(payload["model"].keys()) == set(model.state_dict().keys())
    model2 = resnet.resnet18(num_classes=10).to(dev).to(memory_format=torch.channels_last)
    opt2 = bf.DistributedAdaptWithCombineOptimizer(torch.optim.AdamW(model2.parameters(), lr=1e-3), model2,
                                                   compute_dtype=torch.bfloat16)
    bf.load_checkpoint(path, model2, opt2)
    assert torch.equal(opt2.master_parameters()["fc.weight"], masters["fc.weight"])


def test_graphed_forward_backward_matches_eager(bf, exact_fp32_convolutions):
    from bluefog_b200.models import resnet
    from bluefog_b200.utils.graphs import GraphedForwardBackward
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    models = [resnet.resnet18(num_classes=10).to(dev).to(memory_format=torch.channels_last) for _ in range(2)]
    models[1].load_state_dict(models[0].state_dict())
    opts = [bf.DistributedNeighborAllreduceOptimizer(torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9), m)
            for m in models]
    x = torch.randn(8, 3, 32, 32, device=dev)
    y = torch.randint(0, 10, (8,), device=dev)
    loss_fn = torch.nn.CrossEntropyLoss()
    for m in models:
        m.eval()      # frozen BatchNorm statistics: warm-up passes must not change the model
    graphed = GraphedForwardBackward(models[1], loss_fn, opts[1], x, y)
    for _ in range(3):
        opts[0].zero_grad()
        l0 = loss_fn(models[0](x).float(), y)
        l0.backward()
        opts[0].step()
        l1 = graphed(x, y)
        opts[1].step()
        assert abs(l0.item() - l1.item()) < 1e-3


def test_space_to_depth_stem_matches_direct_convolution_on_gpu():
    from bluefog_b200.models.resnet import StemConv
    torch.manual_seed(3)
    conv = StemConv(space_to_depth=True).cuda().to(torch.bfloat16)
    x = torch.randn(4, 3, 64, 64, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = conv(x)                                         # 4x4 convolution over 2x2 pixel blocks
    ref = torch.nn.Conv2d.forward(conv.float(), x.float())
    assert y.shape == ref.shape
    assert (y.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_bottleneck_with_tcgen05_convolutions_matches_library_path():
    """Training-mode forward/backward of one bottleneck block with its 1x1 and 3x3 convolutions on the
    tcgen05 kernels against the same weights on the library kernels."""
    from bluefog_b200.models import resnet
    from bluefog_b200.ops import conv, gemm
    if not (gemm.available() and conv.available()):
        pytest.fail("tcgen05 kernels are not available on this GPU")
    torch.manual_seed(5)
    a = resnet.Bottleneck(256, 64, use_b200_gemm=True, use_b200_conv=True).cuda()
    b = resnet.Bottleneck(256, 64).cuda()
    b.load_state_dict(a.state_dict())
    for m in (a, b):
        for p in m.parameters():                      # bf16 parameters, fp32 BatchNorm statistics
            p.data = p.data.to(torch.bfloat16)
    a, b = a.to(memory_format=torch.channels_last), b.to(memory_format=torch.channels_last)
    x = torch.randn(8, 256, 28, 28, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = a(xa), b(xb)
    dy = torch.randn_like(ya)
    ya.backward(dy)
    yb.backward(dy)

    def rel(u, v):
        return ((u.float() - v.float()).norm() / v.float().norm().clamp_min(1e-6)).item()

    assert rel(ya, yb) < 2e-2
    assert rel(xa.grad, xb.grad) < 3e-2
    for (name, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert rel(pa.grad, pb.grad) < 5e-2, name


def test_fused_sgd_keeps_channels_last_filters_and_matches_torch_sgd(bf, exact_fp32_convolutions):
    """Channels_last filters stay channels_last inside the bucket (no per-step re-layout), gradients are
    read in the same memory order, and the result equals torch.optim.SGD on the same model."""
    torch.manual_seed(11)
    dev = torch.device("cuda", 0)

    def make():
        return torch.nn.Sequential(torch.nn.Conv2d(8, 16, 3, padding=1), torch.nn.ReLU(),
                                   torch.nn.Conv2d(16, 16, 1), torch.nn.ReLU(),
                                   torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(16, 4))

    m1, m2 = make().to(dev), make().to(dev)
    m2.load_state_dict(m1.state_dict())
    m1, m2 = m1.to(memory_format=torch.channels_last), m2.to(memory_format=torch.channels_last)
    o1 = torch.optim.SGD(m1.parameters(), lr=0.1, momentum=0.9)
    o2 = bf.DistributedNeighborAllreduceOptimizer(torch.optim.SGD(m2.parameters(), lr=0.1, momentum=0.9), m2)
    w = m2[0].weight
    assert w.is_contiguous(memory_format=torch.channels_last) and not w.is_contiguous()
    x = torch.randn(4, 8, 12, 12, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 4, (4,), device=dev)
    for _ in range(3):
        o1.zero_grad()
        o2.zero_grad()
        torch.nn.functional.cross_entropy(m2(x), y).backward()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            p1.grad = p2.grad.detach().clone()            # same gradients for both optimizers
        o1.step()
        o2.step()
    torch.cuda.synchronize()
    o2.check()
    for (n1, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p1, p2, rtol=1e-5, atol=1e-6), (n1, (p1 - p2).abs().max().item())
    masters = o2.master_parameters()
    assert torch.allclose(masters["0.weight"], m1[0].weight, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype,channels_last", [(torch.float32, False), (torch.bfloat16, True), (torch.bfloat16, False)])
def test_stem_input_kernel_matches_the_python_rearrangement(dtype, channels_last):
    from bluefog_b200 import _C
    torch.manual_seed(7)
    x = torch.randn(3, 3, 20, 36, device="cuda").to(dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    out = _C.s2d_stem_input(x)
    n, c, h, w = x.shape
    hb, wb = (h + 6) // 2, (w + 6) // 2
    xp = torch.nn.functional.pad(x.to(torch.bfloat16), (3, 3, 3, 3))
    xs = xp.reshape(n, 3, hb, 2, wb, 2).permute(0, 1, 3, 5, 2, 4).reshape(n, 12, hb, wb)
    ref = torch.nn.functional.pad(xs, (0, 0, 0, 0, 0, 4))
    assert out.shape == ref.shape and out.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(out, ref)


def test_resnet_raw_stem_path_equals_generic_path():
    """Inputs without a gradient take the one-kernel stem transform; the result must equal the generic path
    (forced here by asking for an input gradient)."""
    from bluefog_b200.models import resnet
    torch.manual_seed(9)
    m = resnet.resnet18(num_classes=10).cuda()
    for p in m.parameters():
        p.data = p.data.to(torch.bfloat16)
    m = m.to(memory_format=torch.channels_last).eval()
    x = torch.randn(4, 3, 64, 64, device="cuda")
    with torch.no_grad():
        y_raw = m(x)
    y_gen = m(x.clone().requires_grad_(True))
    assert (y_raw.float() - y_gen.float()).abs().max().item() <= 2e-2 * max(1.0, y_gen.float().abs().max().item())


def test_resnet50_on_own_kernels_matches_the_library_routing():
    """One training step of the whole network (stem, strided 3x3 and 1x1 convolutions, filter gradients, pooling,
    classifier, loss) with every contraction on the tcgen05 kernels against the same weights on library kernels."""
    from bluefog_b200.models import resnet
    from bluefog_b200.ops.fused_ce import cross_entropy
    torch.manual_seed(11)
    a = resnet.resnet50(num_classes=1000, use_b200_gemm=True, use_b200_conv=True, stem_space_to_depth=True).cuda()
    b = resnet.resnet50(num_classes=1000, use_b200_gemm=False, use_b200_conv=False, stem_space_to_depth=True).cuda()
    b.load_state_dict(a.state_dict())
    for m in (a, b):
        for p in m.parameters():
            p.data = p.data.to(torch.bfloat16)
    a, b = a.to(memory_format=torch.channels_last), b.to(memory_format=torch.channels_last)
    x = torch.randn(8, 3, 96, 96, device="cuda")
    y = torch.randint(0, 1000, (8,), device="cuda")
    la = cross_entropy(a(x), y)
    lb = torch.nn.functional.cross_entropy(b(x).float(), y)
    la.backward()
    lb.backward()
    assert abs(la.item() - lb.item()) < 5e-2 * max(1.0, abs(lb.item())), (la.item(), lb.item())

    def rel(u, v):
        return ((u.float() - v.float()).norm() / v.float().norm().clamp_min(1e-6)).item()

    # At a random initialisation the gradients of the deep layers are dominated by bf16 rounding (two runs of the
    # library path with different cuDNN algorithms differ by 100 % there), so only the classifier's gradients,
    # which see the loss directly, are compared; the per-block tests above cover the convolution gradients.
    ga, gb = dict(a.named_parameters()), dict(b.named_parameters())
    assert rel(ga["fc.bias"].grad, gb["fc.bias"].grad) < 2e-2
    assert rel(ga["fc.weight"].grad, gb["fc.weight"].grad) < 0.25
    assert all(p.grad is not None and torch.isfinite(p.grad.float()).all() for p in a.parameters())


@pytest.mark.parametrize("make", [
    lambda ps: torch.optim.RMSprop(ps, lr=1e-3, alpha=0.95, weight_decay=1e-4),
    lambda ps: torch.optim.RMSprop(ps, lr=1e-3, momentum=0.9, centered=True),
    lambda ps: torch.optim.Adagrad(ps, lr=0.05, lr_decay=0.01, initial_accumulator_value=0.1, weight_decay=1e-4),
    lambda ps: torch.optim.Adadelta(ps, lr=1.0, rho=0.9, weight_decay=1e-4),
    lambda ps: torch.optim.Adam(ps, lr=1e-3, amsgrad=True),
], ids=["rmsprop", "rmsprop-centered-momentum", "adagrad", "adadelta", "adam-amsgrad"])
def test_fused_update_of_every_supported_optimizer_matches_torch(bf, make):
    """The bucket kernel's update arithmetic against torch.optim on the same gradients, four steps, and the state
    dictionary under torch's own key names."""
    torch.manual_seed(1)
    dev = torch.device("cuda", 0)
    m1 = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.Tanh(), torch.nn.Linear(64, 10)).to(dev)
    m2 = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.Tanh(), torch.nn.Linear(64, 10)).to(dev)
    m2.load_state_dict(m1.state_dict())
    o1 = make(m1.parameters())
    o2 = bf.DistributedNeighborAllreduceOptimizer(make(m2.parameters()), m2)
    assert hasattr(o2, "master_parameters"), "the bucket engine did not take this optimizer"
    x = torch.randn(16, 37, device=dev)
    y = torch.randint(0, 10, (16,), device=dev)
    for _ in range(4):
        o1.zero_grad()
        o2.zero_grad()
        torch.nn.functional.cross_entropy(m2(x), y).backward()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            p1.grad = p2.grad.detach().clone()
        o1.step()
        o2.step()
        torch.cuda.synchronize()
        o2.check()
        for p1, p2 in zip(m1.parameters(), m2.parameters()):
            assert torch.allclose(p1, p2, rtol=2e-5, atol=2e-6), (p1 - p2).abs().max().item()
    s1, s2 = o1.state_dict()["state"], o2.state_dict()["state"]
    for k in s1:
        assert set(s1[k]) == set(s2[k]), (set(s1[k]), set(s2[k]))
        for name, v in s1[k].items():
            if name != "step":
                assert torch.allclose(v, s2[k][name].to(v.dtype), rtol=1e-4, atol=1e-7), name
            else:
                assert float(v) == float(s2[k][name])
