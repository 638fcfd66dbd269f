"""LayerNorm kernels against PyTorch's fp32 layer_norm (forward, input and parameter gradients)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _case(shape, param_dtype):
    from bluefog_b200.ops.fused_ln import layer_norm, _eligible
    torch.manual_seed(shape[-1])
    C = shape[-1]
    x = (torch.randn(*shape, device="cuda") * 2 + 0.5).to(torch.bfloat16)
    w = (torch.rand(C, device="cuda") + 0.5).to(param_dtype)
    b = torch.randn(C, device="cuda").to(param_dtype)
    dy = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    x1, w1, b1 = (t.clone().requires_grad_(True) for t in (x, w, b))
    assert _eligible(x1, w1, b1)
    y1 = layer_norm(x1, w1, b1, 1e-5)
    y1.backward(dy)
    x2, w2, b2 = (t.float().clone().requires_grad_(True) for t in (x, w, b))
    y2 = F.layer_norm(x2, (C,), w2, b2, 1e-5)
    y2.backward(dy.float())

    def close(a, ref, tol):
        err = (a.float() - ref).abs().max().item()
        bound = tol * max(1.0, ref.abs().max().item())
        assert err <= bound, (err, bound)

    close(y1, y2, 1e-2)
    close(x1.grad, x2.grad, 2e-2)
    ptol = 2e-2 if param_dtype == torch.bfloat16 else 5e-3
    close(w1.grad, w2.grad, ptol)
    close(b1.grad, b2.grad, ptol)


@pytest.mark.parametrize("shape", [(4, 128, 768), (2, 1024, 1024), (3000, 1600), (7, 8), (5, 33, 2048), (1, 1280)])
def test_layer_norm_matches_pytorch(shape):
    _case(shape, torch.float32)


def test_layer_norm_with_bf16_parameters():
    _case((8, 256, 1024), torch.bfloat16)


def test_layer_norm_module_falls_back_for_fp32():
    from bluefog_b200.ops.fused_ln import LayerNorm
    ln = LayerNorm(48).cuda()
    x = torch.randn(4, 48, device="cuda")
    torch.testing.assert_close(ln(x), F.layer_norm(x, (48,), ln.weight, ln.bias, ln.eps))


@pytest.mark.parametrize("R,C", [(8192, 4096), (8192, 1024), (37, 8), (1000, 264), (3, 3072)])
def test_column_sum_matches_fp32_sum(R, C):
    from bluefog_b200 import _C
    torch.manual_seed(R + C)
    x = torch.randn(R, C, device="cuda").to(torch.bfloat16)
    out = _C.column_sum(x)
    ref = x.float().sum(0)
    assert out.dtype == torch.float32
    assert (out - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("shape", [(2, 1024, 1024), (3, 37, 768), (5, 8), (9, 2048), (130, 1280)])
def test_layer_norm_with_the_residual_gradient_joined_in_the_kernel(shape):
    """(LN(x), x): the gradient past the LayerNorm is added inside the backward kernel, which also hands the column
    sums of the total to whoever computes a bias gradient from it."""
    from bluefog_b200.ops import fused_ln
    torch.manual_seed(shape[-1] + 1)
    C = shape[-1]
    x = (torch.randn(*shape, device="cuda") * 2 + 0.5).to(torch.bfloat16)
    w = torch.rand(C, device="cuda") + 0.5
    b = torch.randn(C, device="cuda")
    dy = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    dres = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    x1, w1, b1 = (t.clone().requires_grad_(True) for t in (x, w, b))
    # the layer in front of the LayerNorm sees the gradient as its backward pass does: a hook on a non-leaf tensor
    seen = {}
    xin = x1 * 1
    xin.register_hook(lambda g: seen.update(first=fused_ln.take_column_sums(g.reshape(-1, C)),
                                            second=fused_ln.take_column_sums(g.reshape(-1, C))))
    y1, r1 = fused_ln.layer_norm_residual(xin, w1, b1, 1e-5)
    assert r1.shape == x1.shape
    torch.autograd.backward([y1, r1], [dy, dres])
    x2, w2, b2 = (t.float().clone().requires_grad_(True) for t in (x, w, b))
    y2 = F.layer_norm(x2, (C,), w2, b2, 1e-5)
    torch.autograd.backward([y2, x2 * 1.0], [dy.float(), dres.float()])

    def close(a, ref, tol):
        err = (a.float() - ref).abs().max().item()
        bound = tol * max(1.0, ref.abs().max().item())
        assert err <= bound, (err, bound)

    close(y1, y2, 1e-2)
    close(x1.grad, x2.grad, 2e-2)
    close(w1.grad, w2.grad, 5e-3)
    close(b1.grad, b2.grad, 5e-3)
    # the column sums travel with the gradient tensor (and with views of it), once
    assert seen["first"] is not None and seen["second"] is None
    close(seen["first"], x2.grad.reshape(-1, C).sum(0), 1e-2)


def test_only_one_of_the_two_results_used():
    from bluefog_b200.ops import fused_ln
    x = torch.randn(16, 256, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w, b = torch.ones(256, device="cuda", requires_grad=True), torch.zeros(256, device="cuda", requires_grad=True)
    y, r = fused_ln.layer_norm_residual(x, w, b)
    r.float().sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    x.grad = None
    y, r = fused_ln.layer_norm_residual(x, w, b)
    y.float().sum().backward()
    ref = x.detach().clone().requires_grad_(True)
    fused_ln.layer_norm(ref, w.detach().requires_grad_(True), b.detach().requires_grad_(True)).float().sum().backward()
    assert torch.allclose(x.grad.float(), ref.grad.float(), atol=1e-2)


def test_transformer_block_takes_bias_gradients_from_the_layer_norm_kernel():
    """One GPT-2 block with and without the joined gradients: same parameter gradients, and the bias gradients of the
    two projections that feed the residual stream come from the LayerNorm kernel's column sums."""
    from bluefog_b200.models.gpt2 import Block
    from bluefog_b200.ops import fused_ln, gemm
    if not gemm.available():
        pytest.skip("tcgen05 GEMM not available")
    torch.manual_seed(3)
    blocks = torch.nn.Sequential(Block(256, 4, True), Block(256, 4, True)).cuda().to(torch.bfloat16)
    x = torch.randn(4, 128, 256, device="cuda").to(torch.bfloat16)
    dy = torch.randn_like(x)
    grads = {}
    for fuse in (True, False):
        fused_ln.FUSE_RESIDUAL_GRADIENT = fuse
        try:
            hits = fused_ln.column_sum_hits
            xin = x.clone().requires_grad_(True)
            blocks.zero_grad(set_to_none=True)
            blocks(xin).backward(dy)
            grads[fuse] = [p.grad.float().clone() for p in blocks.parameters()] + [xin.grad.float().clone()]
            # ln_2 of both blocks serves the attention projection; ln_1 of the second block serves the first block's MLP
            assert fused_ln.column_sum_hits - hits == (3 if fuse else 0)
        finally:
            fused_ln.FUSE_RESIDUAL_GRADIENT = True
    for a, b_ in zip(grads[True], grads[False]):
        scale = max(1.0, b_.abs().max().item())
        assert (a - b_).abs().max().item() <= 3e-2 * scale
