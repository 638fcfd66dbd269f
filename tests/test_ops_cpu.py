"""CPU behaviour of the model-side ops (their kernels need a GPU; the fallbacks do not)."""

def test_layer_norm_cpu_fallback_matches_torch():
    import torch
    import torch.nn.functional as F
    from bluefog_b200.ops.fused_ln import LayerNorm, layer_norm
    ln = LayerNorm(24)
    x = torch.randn(3, 5, 24)
    torch.testing.assert_close(ln(x), F.layer_norm(x, (24,), ln.weight, ln.bias, ln.eps))
    torch.testing.assert_close(layer_norm(x, None, None), F.layer_norm(x, (24,)))
