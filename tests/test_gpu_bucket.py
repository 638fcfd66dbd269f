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


MODE_ANNOUNCE = 5


def test_awc_with_destination_weights_announced_per_step():
    """Adapt-with-combine where every sender scales what each destination pulls: the weights of a step are
    announced for the version published one step earlier.  (Ranks share one GPU here and run one after the other,
    so the announcement is a launch of its own; on real ranks the step kernel makes it when it starts.)"""
    C = _C()
    W, n, lr = 4, 3001, 0.1
    buckets, master = _make(C, W, n, "float32")
    ref = [m.clone() for m in master]
    g = torch.Generator().manual_seed(21)
    for t in range(4):
        grads = [torch.randn(n, generator=g).cuda() for _ in range(W)]
        # rank s sends to s+1 with weight 0.5 + 0.1*s + 0.05*t, and to s+2 with weight 2
        dstw = [[1.0] * W for _ in range(W)]
        for s in range(W):
            dstw[s][(s + 1) % W] = 0.5 + 0.1 * s + 0.05 * t
            dstw[s][(s + 2) % W] = 2.0
        old = [p.clone() for p in ref]
        for r in range(W):
            comb = 0.4 * old[r] + 0.3 * dstw[(r - 1) % W][r] * old[(r - 1) % W] + 0.3 * dstw[(r - 2) % W][r] * old[(r - 2) % W]
            ref[r] = comb - lr * grads[r]
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.dst_weights = MODE_ANNOUNCE, dstw[r]
            buckets[r].step(a)
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.opt, a.master, a.grad, a.lr = MODE_AWC, 1, master[r], grads[r], lr
            a.self_weight, a.src_ranks, a.src_weights, a.n_readers = 0.4, [(r - 1) % W, (r - 2) % W], [0.3, 0.3], 2
            a.dst_weights, a.read_dst_weights = dstw[r], True
            buckets[r].step(a)
    torch.cuda.synchronize()
    for r in range(W):
        assert buckets[r].status()[0] == 0, buckets[r].status()
        assert (master[r] - ref[r]).abs().max().item() < 1e-4


def test_atc_with_destination_weights_stored_beside_the_version():
    C = _C()
    W, n, lr = 3, 2500, 0.05
    buckets, master = _make(C, W, n, "float32")
    ref = [m.clone() for m in master]
    g = torch.Generator().manual_seed(22)
    for t in range(3):
        grads = [torch.randn(n, generator=g).cuda() for _ in range(W)]
        dstw = [[1.0] * W for _ in range(W)]
        for s in range(W):
            dstw[s][(s + 1) % W] = 0.25 * (s + 1) + t
        adapted = [ref[r] - lr * grads[r] for r in range(W)]
        ref = [0.5 * adapted[r] + 0.5 * dstw[(r - 1) % W][r] * adapted[(r - 1) % W] for r in range(W)]
        for r in range(W):
            a = C.BucketStepArgs()
            a.mode, a.opt, a.master, a.grad, a.lr = MODE_ADAPT_PUBLISH, 1, master[r], grads[r], lr
            a.dst_weights = dstw[r]
            buckets[r].step(a)
        for r in range(W):
            c = C.BucketStepArgs()
            c.mode, c.master = MODE_COMBINE_ONLY, master[r]
            c.self_weight, c.src_ranks, c.src_weights, c.n_readers = 0.5, [(r - 1) % W], [0.5], 1
            c.read_dst_weights = True
            buckets[r].step(c)
    torch.cuda.synchronize()
    for r in range(W):
        assert buckets[r].status()[0] == 0
        assert (master[r] - ref[r]).abs().max().item() < 1e-4


def test_hierarchical_average_as_one_weighted_pull():
    """Four ranks on two machines of two: mean inside each machine, then the machines average each other."""
    C = _C()
    W, n = 4, 1030
    buckets, master = _make(C, W, n, "float32")
    start = [m.clone() for m in master]
    machine_mean = [(start[0] + start[1]) / 2, (start[2] + start[3]) / 2]
    expect = [0.5 * machine_mean[r // 2] + 0.5 * machine_mean[1 - r // 2] for r in range(W)]
    for r in range(W):
        a = C.BucketStepArgs()
        a.mode, a.master = MODE_AWC, master[r]
        mine, other = r // 2, 1 - r // 2
        a.self_weight = 0.5 / 2
        a.src_ranks = [s for s in range(2 * mine, 2 * mine + 2) if s != r] + list(range(2 * other, 2 * other + 2))
        a.src_weights = [0.25] * 3
        a.n_readers = 3
        buckets[r].step(a)
    torch.cuda.synchronize()
    for r in range(W):
        assert buckets[r].status()[0] == 0
        assert (master[r] - expect[r]).abs().max().item() < 1e-5


def test_parameters_without_a_gradient_are_left_alone():
    """Per-parameter gradient table with a missing entry: that parameter gets the combined value and no optimizer
    update (no weight decay, no momentum decay), like torch.optim, which skips parameters whose grad is None."""
    C = _C()
    n_a, n_b = 1024, 2048
    n = n_a + n_b
    buckets, master = _make(C, 1, n, "float32")
    before = master[0].clone()
    mom = torch.full((n,), 0.5, device="cuda")
    ga = torch.randn(n_a, device="cuda")
    table = torch.tensor([ga.data_ptr(), 0], dtype=torch.int64, device="cuda")
    a = C.BucketStepArgs()
    a.mode, a.opt, a.master, a.state1 = MODE_AWC, 1, master[0], mom
    a.lr, a.momentum, a.weight_decay, a.first_step = 0.1, 0.9, 0.1, False
    a.grad_ptrs = table
    a.seg_start = torch.tensor([0, n_a], dtype=torch.int64, device="cuda")
    a.seg_numel = torch.tensor([n_a, n_b], dtype=torch.int64, device="cuda")
    a.self_weight = 1.0
    buckets[0].step(a)
    torch.cuda.synchronize()
    d = ga + 0.1 * before[:n_a]
    buf = 0.9 * 0.5 + d
    assert torch.allclose(master[0][:n_a], before[:n_a] - 0.1 * buf, atol=1e-5)
    assert torch.equal(master[0][n_a:], before[n_a:])
    assert torch.equal(mom[n_a:], torch.full((n_b,), 0.5, device="cuda"))


def test_a_version_whose_owner_gave_up_is_marked_and_not_combined():
    """The owner's wait for its readers runs out (50 ms limit, nobody reads): it announces the version anyway so
    that nobody hangs, marked as failed; a reader of that version reports the failure and leaves its output alone."""
    C = _C()
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(2, 1 << 16, 0)
    world.set_timeout_ms(50.0)
    x = torch.ones(256, device=dev)
    for _ in range(2):
        world.publish(0, [x], None, 1)           # versions 0 and 1: one reader each, who never comes
        world.publish(1, [x], None, 0)
    r0 = world.publish(0, [x * 3], None, 1)      # version 2 must wait for the reader of version 0: times out
    r1 = world.publish(1, [x], None, 0)
    torch.cuda.synchronize()
    assert world.status(0)[0] == 2               # kCommTimeoutDone on the owner
    out = torch.full((256,), -7.0, device=dev)
    world.combine(1, r1, [out], 0.5, [0], [0.5], False, 1.0)
    torch.cuda.synchronize()
    err, peer, _, _ = world.status(1)
    assert err == 4 and peer == 0                # kCommPeerFailed
    assert torch.equal(out, torch.full((256,), -7.0, device=dev))
    assert torch.ones(4, device=dev).sum().item() == 4.0
