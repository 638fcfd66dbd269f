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
