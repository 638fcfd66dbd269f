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
