"""GPT-2 on the GPU: bf16 model with the tcgen05 GEMM, LayerNorm kernels and the padded classifier
against the same weights evaluated in fp32 with PyTorch's own ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_gpt2_bf16_kernels_match_fp32_reference():
    from bluefog_b200.models import gpt2
    torch.manual_seed(0)
    ref = gpt2.GPT2(vocab_size=1001, n_positions=64, d_model=128, n_layer=2, n_head=4, use_b200_gemm=False).cuda()
    fast = gpt2.GPT2(vocab_size=1001, n_positions=64, d_model=128, n_layer=2, n_head=4, use_b200_gemm=True).cuda()
    fast.load_state_dict(ref.state_dict())
    fast = fast.to(torch.bfloat16)
    x = torch.randint(0, 1001, (4, 64), device="cuda")
    y = torch.randint(0, 1001, (4, 64), device="cuda")
    logits_ref = ref(x)
    logits = fast(x)
    assert logits.shape == (4, 64, 1001)                        # the padding columns never leave the model
    assert (logits.float() - logits_ref).abs().max().item() < 0.08
    loss_ref = ref(x, y)
    loss = fast(x, y)
    assert abs(loss.item() - loss_ref.item()) < 0.05
    loss.backward()
    loss_ref.backward()
    g, g_ref = fast.wte.weight.grad.float(), ref.wte.weight.grad
    assert g.shape == g_ref.shape and torch.isfinite(g).all()
    rel = ((g - g_ref).norm() / g_ref.norm()).item()
    assert rel < 0.08, rel
    g2, g2_ref = fast.h[0].mlp.c_fc.weight.grad.float(), ref.h[0].mlp.c_fc.weight.grad
    assert ((g2 - g2_ref).norm() / g2_ref.norm()).item() < 0.08


@pytest.mark.parametrize("R,C,pad", [(64, 1008, 7), (1000, 50304, 47), (3, 8, 0), (257, 4096, 0)])
def test_fused_cross_entropy_matches_fp32(R, C, pad):
    from bluefog_b200.ops.fused_ce import cross_entropy
    torch.manual_seed(R + C)
    logits = (torch.randn(R, C, device="cuda") * 3).to(torch.bfloat16)
    if pad:
        logits[:, C - pad:] = float("-inf")
    targets = torch.randint(0, C - pad, (R,), device="cuda")
    a = logits.clone().requires_grad_(True)
    loss = cross_entropy(a, targets)
    (loss * 2.5).backward()                      # a non-trivial upstream gradient
    b = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(b, targets)
    (ref * 2.5).backward()
    assert loss.dtype == torch.float32 and abs(loss.item() - ref.item()) < 1e-3 * max(1.0, abs(ref.item()))
    assert a.grad.dtype == torch.bfloat16
    err = (a.grad.float() - b.grad).abs().max().item()
    assert err <= 1e-2 * max(b.grad.abs().max().item(), 1e-6), err
    if pad:
        assert a.grad[:, C - pad:].abs().max().item() == 0.0


@pytest.mark.parametrize("B,T,V,C,P", [(8, 128, 1000, 256, 128), (3, 17, 50, 64, 40), (4, 64, 20, 1024, 64), (1, 1, 5, 8, 1)])
def test_token_position_embedding_matches_pytorch(B, T, V, C, P):
    """wte[idx] + wpe[:T] and both table gradients (repeated tokens summed in fp32) against fp32 PyTorch; twice, so that
    the scratch buffers are seen to come back clean."""
    from bluefog_b200.ops import fused_embedding
    torch.manual_seed(B * T + V)
    idx = torch.randint(0, V, (B, T), device="cuda")
    wte = torch.randn(V, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
    wpe = torch.randn(P, C, device="cuda").to(torch.bfloat16).requires_grad_(True)
    assert fused_embedding._eligible(idx, wte, wpe)
    for _ in range(2):
        wte.grad = wpe.grad = None
        out = fused_embedding.token_position_embedding(idx, wte, wpe)
        ref = wte.detach().float()[idx] + wpe.detach().float()[:T]
        assert out.shape == (B, T, C) and torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
        dy = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
        out.backward(dy)
        fused_embedding.check_indices()
        ref_wte = torch.zeros(V, C, device="cuda").index_add_(0, idx.reshape(-1), dy.float().reshape(-1, C))
        ref_wpe = torch.zeros(P, C, device="cuda")
        ref_wpe[:T] = dy.float().sum(0)
        for got, want in ((wte.grad, ref_wte), (wpe.grad, ref_wpe)):
            assert got.shape == want.shape
            err = (got.float() - want).abs().max().item()
            assert err <= 1e-2 * max(1.0, want.abs().max().item()), err


def test_token_outside_the_table_is_skipped_and_reported():
    from bluefog_b200.ops import fused_embedding
    wte = torch.randn(10, 16, device="cuda").to(torch.bfloat16)
    wpe = torch.randn(4, 16, device="cuda").to(torch.bfloat16)
    idx = torch.tensor([[1, 2, 12, 3]], device="cuda")
    out = fused_embedding.token_position_embedding(idx, wte, wpe)
    assert torch.equal(out[0, 2], wpe[2])                  # the position term alone
    with pytest.raises(IndexError):
        fused_embedding.check_indices()
