"""CPU behaviour of the model-side ops (their kernels need a GPU; the fallbacks do not)."""

def test_layer_norm_cpu_fallback_matches_torch():
    import torch
    import torch.nn.functional as F
    from bluefog_b200.ops.fused_ln import LayerNorm, layer_norm
    ln = LayerNorm(24)
    x = torch.randn(3, 5, 24)
    torch.testing.assert_close(ln(x), F.layer_norm(x, (24,), ln.weight, ln.bias, ln.eps))
    torch.testing.assert_close(layer_norm(x, None, None), F.layer_norm(x, (24,)))


def test_space_to_depth_stem_equals_the_7x7_convolution():
    import torch
    from bluefog_b200.models.resnet import StemConv
    torch.manual_seed(0)
    conv = StemConv(space_to_depth=True).double()
    x = torch.randn(2, 3, 32, 48, dtype=torch.float64)
    torch.testing.assert_close(conv.forward_space_to_depth(x), torch.nn.Conv2d.forward(conv, x), rtol=1e-10, atol=1e-10)


def test_conv_ops_fall_back_on_cpu():
    import torch
    import torch.nn.functional as F
    from bluefog_b200.ops import conv, gemm
    x = torch.randn(2, 16, 6, 6)
    w3 = torch.randn(8, 16, 3, 3)
    w1 = torch.randn(8, 16, 1, 1)
    torch.testing.assert_close(conv.conv3x3(x, w3), F.conv2d(x, w3, padding=1))
    torch.testing.assert_close(gemm.conv1x1(x, w1), F.conv2d(x, w1))


def test_gpt2_small_config_runs_on_cpu_and_uses_hf_names():
    import torch
    from bluefog_b200.models import gpt2
    torch.manual_seed(0)
    m = gpt2.GPT2(vocab_size=101, n_positions=16, d_model=32, n_layer=2, n_head=2)
    names = set(m.state_dict().keys())
    assert {"wte.weight", "wpe.weight", "h.0.ln_1.weight", "h.0.attn.c_attn.weight", "h.0.attn.c_proj.bias",
            "h.1.mlp.c_fc.weight", "h.1.mlp.c_proj.weight", "ln_f.bias"} <= names
    x = torch.randint(0, 101, (2, 16))
    y = torch.randint(0, 101, (2, 16))
    assert m(x).shape == (2, 16, 101)
    loss = m(x, y)
    loss.backward()
    assert torch.isfinite(loss) and m.wte.weight.grad.shape == (101, 32)


def test_mlp_gelu_falls_back_to_the_plain_ops_on_cpu():
    import torch
    import torch.nn.functional as F
    from bluefog_b200.ops import gemm
    torch.manual_seed(0)
    a, w1, b1 = torch.randn(6, 16), torch.randn(32, 16), torch.randn(32)
    w2, b2 = torch.randn(16, 32), torch.randn(16)
    want = F.linear(F.gelu(F.linear(a, w1, b1), approximate="tanh"), w2, b2)
    assert torch.allclose(gemm.mlp_gelu(a, w1, b1, w2, b2), want)


def test_conv1x1_with_batchnorm_statistics_needs_the_kernel_path():
    import pytest
    import torch
    from bluefog_b200.models.resnet import Conv1x1, MixedBatchNorm2d, bn_act
    from bluefog_b200.ops import gemm
    x = torch.randn(2, 16, 4, 4)
    conv, bn = Conv1x1(16, 8, use_b200_gemm=True), MixedBatchNorm2d(8)
    assert not gemm.conv1x1_supported(x, conv.weight)
    with pytest.raises(ValueError):
        gemm.conv1x1(x, conv.weight, col_stats=torch.zeros(16))
    # the model-level entry point silently takes the library convolution and the BatchNorm's own statistics
    torch.manual_seed(1)
    got = conv.forward_bn_act(x, bn, relu=True)
    bn2 = MixedBatchNorm2d(8)
    want = bn_act(conv(x), bn2, relu=True)
    assert torch.allclose(got, want)
    assert torch.allclose(bn.running_mean, bn2.running_mean)


def test_split_for_two_uses_leaves_other_tensors_alone():
    """Gradient pairs are only formed for outputs of the fused BatchNorm kernels; any other tensor comes back twice
    unchanged and autograd adds its gradients as usual."""
    import torch
    from bluefog_b200.ops import fused_bn
    x = torch.randn(2, 8, 4, 4, requires_grad=True)
    a, b = fused_bn.split_for_two_uses(x)
    assert a is x and b is x
    (a * 2 + b * 3).sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x, 5.0))
    bn = torch.nn.BatchNorm2d(8)
    y = fused_bn.bn_act(x, bn, relu=True)            # CPU: PyTorch fallback, no pairs
    assert not getattr(y, "_bfb_takes_pairs", False)
    fused_bn.begin_step(x.device)                    # nothing pending, nothing raised


def test_layer_norm_residual_falls_back_on_cpu():
    """Off the kernels, ``layer_norm_residual`` is ``(F.layer_norm(x), x)`` and autograd adds the two gradients."""
    import torch
    import torch.nn.functional as F
    from bluefog_b200.ops import fused_ln
    x = torch.randn(3, 5, 16, requires_grad=True)
    w, b = torch.rand(16) + 0.5, torch.randn(16)
    y, r = fused_ln.layer_norm_residual(x, w, b)
    assert r is x and torch.allclose(y, F.layer_norm(x, (16,), w, b))
    (y.sum() + 2 * r.sum()).backward()
    ref = x.detach().clone().requires_grad_(True)
    (F.layer_norm(ref, (16,), w, b).sum() + 2 * ref.sum()).backward()
    assert torch.allclose(x.grad, ref.grad)
    assert fused_ln.take_column_sums(x.grad.reshape(-1, 16)) is None


def test_symmetric_empty_without_a_gpu_world_is_an_ordinary_tensor():
    import torch
    import bluefog_b200.torch as bf
    x = bf.symmetric_empty(3, 5, dtype=torch.bfloat16)
    assert x.shape == (3, 5) and x.dtype == torch.bfloat16
    assert bf.symmetric_empty((4,)).shape == (4,)
    assert not bf.is_symmetric(x)


def test_column_sums_offered_with_a_gradient_are_taken_once_and_only_for_that_tensor():
    """The hand-over of bias-gradient sums between two backward passes: keyed by the gradient's address, honoured only
    while the tensor it was made for is alive and has the same extent, and only once."""
    import gc
    import torch
    from bluefog_b200.ops import fused_ln
    g = torch.randn(6, 8)
    sums = g.sum(0)
    fused_ln._offer_column_sums(g, sums)
    assert fused_ln.take_column_sums(torch.randn(6, 8)) is None          # another tensor
    view = g.reshape(2, 3, 8).reshape(-1, 8)                              # same memory, seen through views
    assert fused_ln.take_column_sums(view) is sums
    assert fused_ln.take_column_sums(view) is None                        # taken
    # an entry whose tensor has died is not honoured, even if the address comes back
    h = torch.randn(6, 8)
    fused_ln._offer_column_sums(h, h.sum(0))
    addr = h.data_ptr()
    del h
    gc.collect()
    again = torch.randn(6, 8)
    if again.data_ptr() == addr:                                          # the allocator usually hands the block back
        assert fused_ln.take_column_sums(again) is None
    # a different extent at the same address does not match either
    k = torch.randn(6, 8)
    fused_ln._offer_column_sums(k, k.sum(0))
    assert fused_ln.take_column_sums(k[:3]) is None
