"""Model-level GPU tests on one device: fused optimizer vs torch.optim, CUDA-graph step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bf():
    import bluefog_b200.torch as bf
    bf.init()
    yield bf


def test_fused_sgd_single_rank_matches_torch_sgd(bf):
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
    for _ in range(3):
        for m, o in ((m1, o1), (m2, o2)):
            o.zero_grad()
            torch.nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    torch.cuda.synchronize()
    o2.check()
    for (n1, p1), (n2, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p1, p2, rtol=1e-4, atol=1e-5), n1
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


def test_graphed_forward_backward_matches_eager(bf):
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
