"""Fused bucket kernel (combine + optimizer update + casts) against torch.optim in fp32.

Ranks are emulated in one process: ``Bucket.create_local`` maps all ranks' published copies
on one GPU and the per-rank kernels run one after the other.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

MODE_AWC, MODE_ADAPT_PUBLISH, MODE_COMBINE_ONLY, MODE_GRAD_REDUCE, MODE_PUBLISH_ONLY = 0, 1, 2, 3, 4


def _C():
    from bluefog_b200 import _C
    return _C


def _ring_weights(W):
    """Row r: (self_w, {src: w}) for a directed ring r-1 -> r with lazy weights."""
    return [(0.6, {(r - 1) % W: 0.4}) for r in range(W)]


def _make(C, W, n, pub):
    buckets = C.Bucket.create_local(W, n, pub, 0)
    g = torch.Generator().manual_seed(7)
    master = [torch.randn(n, generator=g).cuda() for _ in range(W)]
    for r in range(W):
        a = C.BucketStepArgs()
        a.mode = MODE_PUBLISH_ONLY
        a.master = master[r]
        buckets[r].step(a)
    return buckets, master


@pytest.mark.parametrize("opt_name", ["sgd", "sgd_nesterov_wd", "adam", "adamw_amsgrad"])
@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_awc_matches_torch_optim(opt_name, grad_dtype):
    C = _C()
    W, n, steps = 3, 10007, 4
    buckets, master = _make(C, W, n, "float32")
    ref_p = [m.clone().double().requires_grad_(False) for m in master]
    params = [torch.nn.Parameter(p.clone()) for p in ref_p]
    if opt_name == "sgd":
        kw = dict(lr=0.1, momentum=0.9)
        opts = [torch.optim.SGD([p], **kw) for p in params]
    elif opt_name == "sgd_nesterov_wd":
        kw = dict(lr=0.05, momentum=0.8, nesterov=True, weight_decay=0.01)
        opts = [torch.optim.SGD([p], **kw) for p in params]
    elif opt_name == "adam":
        kw = dict(lr=0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.02)
        opts = [torch.optim.Adam([p], **kw) for p in params]
    else:
        kw = dict(lr=0.01, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.02, amsgrad=True)
        opts = [torch.optim.AdamW([p], **kw) for p in params]
    is_sgd = opt_name.startswith("sgd")
    s1 = [torch.zeros(n, device="cuda") for _ in range(W)]
    s2 = [torch.zeros(n, device="cuda") for _ in range(W)]
    s3 = [torch.zeros(n, device="cuda") for _ in range(W)]
    shadow = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    weights = _ring_weights(W)
    g = torch.Generator().manual_seed(3)
    for t in range(steps):
        grads = [torch.randn(n, generator=g).cuda().to(grad_dtype) for _ in range(W)]
        # reference: combine with the *previous* iterates of all ranks, then the local update
        old = [p.detach().clone() for p in params]
        for r in range(W):
            sw, src = weights[r]
            comb = sw * old[r]
            for s, w in src.items():
                comb = comb + w * old[s]
            with torch.no_grad():
                params[r].copy_(comb)
            params[r].grad = grads[r].double()
            opts[r].step()
        for r in range(W):
            sw, src = weights[r]
            a = C.BucketStepArgs()
            a.mode = MODE_AWC
            a.opt = 1 if is_sgd else 2
            a.master, a.grad, a.shadow = master[r], grads[r], shadow[r]
            a.state1, a.state2, a.state3 = s1[r], s2[r], s3[r]
            a.lr = kw["lr"]
            a.weight_decay = kw.get("weight_decay", 0.0)
            if is_sgd:
                a.momentum, a.nesterov, a.first_step = kw["momentum"], kw.get("nesterov", False), t == 0
            else:
                a.beta1, a.beta2 = kw["betas"]
                a.eps = kw["eps"]
                a.bias1, a.bias2 = 1 - kw["betas"][0] ** (t + 1), 1 - kw["betas"][1] ** (t + 1)
                a.adamw = opt_name.startswith("adamw")
                a.amsgrad = kw.get("amsgrad", False)
            a.self_weight = sw
            a.src_ranks = list(src.keys())
            a.src_weights = list(src.values())
            a.n_readers = 1
            buckets[r].step(a)
    torch.cuda.synchronize()
    for r in range(W):
        assert buckets[r].status()[0] == 0
        err = (master[r].double() - params[r].detach()).abs().max().item()
        assert err < 2e-4, (opt_name, r, err)
        assert (shadow[r].float() - master[r]).abs().max().item() <= 0.01 * master[r].abs().max().item() + 1e-3


@pytest.mark.parametrize("pub", ["float32", "bfloat16"])
def test_atc_two_phase(pub):
    C = _C()
    W, n = 4, 4099
    buckets, master = _make(C, W, n, pub)
    ref = [m.clone() for m in master]
    g = torch.Generator().manual_seed(11)
    lr = 0.1
    for t in range(3):
        grads = [torch.randn(n, generator=g).cuda() for _ in range(W)]
        adapted = [ref[r] - lr * grads[r] for r in range(W)]
        # neighbors are seen in the exchange format; the own term stays in fp32
        seen = [a.to(torch.bfloat16).float() for a in adapted] if pub == "bfloat16" else adapted
        ref = [0.5 * adapted[r] + 0.25 * seen[(r - 1) % W] + 0.25 * seen[(r + 1) % W] for r in range(W)]
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.opt, a.master, a.grad, a.lr = MODE_ADAPT_PUBLISH, 1, master[r], grads[r], lr
            buckets[r].step(a)
        for r in range(W):
            c = C.BucketStepArgs()
            c.mode, c.master = MODE_COMBINE_ONLY, master[r]
            c.self_weight, c.src_ranks, c.src_weights, c.n_readers = 0.5, [(r - 1) % W, (r + 1) % W], [0.25, 0.25], 2
            buckets[r].step(c)
    torch.cuda.synchronize()
    tol = 1e-5          # also with the 16-bit exchange: the reference rounds exactly what the kernel rounds
    for r in range(W):
        assert buckets[r].status()[0] == 0
        assert (master[r] - ref[r]).abs().max().item() < tol


def test_grad_reduce_equals_mean_gradient_sgd():
    C = _C()
    W, n = 4, 2050
    buckets, master = _make(C, W, n, "float32")
    # drop the initial publication of the masters: gradient allreduce publishes gradients
    ref = [m.clone() for m in master]
    g = torch.Generator().manual_seed(5)
    lr = 0.05
    for t in range(3):
        grads = [torch.randn(n, generator=g).cuda() for _ in range(W)]
        mean = sum(grads) / W
        ref = [p - lr * mean for p in ref]
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.grad = MODE_PUBLISH_ONLY, grads[r]
            buckets[r].step(a)
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.opt, a.master, a.grad, a.lr = MODE_GRAD_REDUCE, 1, master[r], grads[r], lr
            a.src_ranks = [s for s in range(W) if s != r]
            a.src_weights = [1.0] * (W - 1)
            a.n_readers = W - 1
            a.post_scale = 1.0 / W
            buckets[r].step(a)
    torch.cuda.synchronize()
    for r in range(W):
        assert buckets[r].status()[0] == 0
        assert (master[r] - ref[r]).abs().max().item() < 1e-5
