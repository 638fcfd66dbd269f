"""Numerics of the peer-memory kernels against plain fp32 PyTorch, on one GPU.

All "ranks" are buffers of this process (LocalWorld / Bucket.create_local) and the kernels of
the ranks are launched one after the other, so no kernel ever waits for another one.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from bluefog_b200 import _C
    return _C


DTYPES = [torch.float32, torch.float64, torch.bfloat16, torch.float16]
TOL = {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 2e-2, torch.float16: 2e-3}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("numel", [1, 7, 1000, 65537, 1 << 20])
def test_combine_matches_reference(dtype, numel):
    C = _C()
    W = 4
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(W, 8 << 20, 0)
    g = torch.Generator(device="cpu").manual_seed(numel)
    xs = [torch.randn(numel, generator=g).to(dev).to(dtype) for _ in range(W)]
    rounds = [world.publish(r, [xs[r]], None, W - 1) for r in range(W)]
    for r in range(W):
        src = [s for s in range(W) if s != r]
        w = [0.1 * (s + 1) for s in src]
        out = torch.empty(numel, dtype=dtype, device=dev)
        world.combine(r, rounds[r], [out], 0.3, src, w, False, 1.0)
        ref = 0.3 * xs[r].double()
        for s, ws in zip(src, w):
            ref = ref + ws * xs[s].double()
        torch.cuda.synchronize()
        assert world.status(r)[0] == 0
        err = (out.double() - ref).abs().max().item()
        assert err <= TOL[dtype] * max(1.0, ref.abs().max().item()), (dtype, numel, err)


def test_combine_fused_segments_and_dst_weights():
    C = _C()
    W = 3
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(W, 4 << 20, 0)
    sizes = [5, 1024, 333, 70000]
    xs = [[torch.full((n,), float(r + 1) + 0.01 * i, device=dev) for i, n in enumerate(sizes)] for r in range(W)]
    dstw = [[1.0, 2.0, 3.0], [4.0, 1.0, 5.0], [6.0, 7.0, 1.0]]  # dstw[sender][receiver]
    rounds = [world.publish(r, xs[r], dstw[r], W - 1) for r in range(W)]
    for r in range(W):
        src = [s for s in range(W) if s != r]
        outs = [torch.empty(n, device=dev) for n in sizes]
        world.combine(r, rounds[r], outs, 0.5, src, [0.25, 0.125], True, 2.0)
        torch.cuda.synchronize()
        for i, n in enumerate(sizes):
            ref = 0.5 * xs[r][i]
            for s, ws in zip(src, [0.25, 0.125]):
                ref = ref + ws * dstw[s][r] * xs[s][i]
            assert torch.allclose(outs[i], 2.0 * ref, rtol=1e-5, atol=1e-5)


def test_integer_sum_is_exact():
    C = _C()
    W = 4
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(W, 1 << 20, 0)
    for dtype in (torch.int32, torch.int64):
        xs = [torch.arange(1001, device=dev, dtype=dtype) * (r + 1) for r in range(W)]
        rounds = [world.publish(r, [xs[r]], None, W - 1) for r in range(W)]
        out = torch.empty(1001, dtype=dtype, device=dev)
        world.combine(0, rounds[0], [out], 1.0, [1, 2, 3], [1.0, 1.0, 1.0], False, 1.0)
        for r in range(1, W):   # keep the reader accounting balanced
            world.combine(r, rounds[r], [torch.empty_like(out)], 1.0, [s for s in range(W) if s != r], [1.0] * 3, False, 1.0)
        torch.cuda.synchronize()
        assert torch.equal(out, sum(xs))


def test_gather_variable_sizes():
    C = _C()
    W = 3
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(W, 1 << 20, 0)
    xs = [torch.arange(10 * (r + 1) + 3, device=dev, dtype=torch.float32) + 100 * r for r in range(W)]
    rounds = [world.publish(r, [xs[r]], None, W - 1) for r in range(W)]
    for r in range(W):
        outs = [torch.empty_like(xs[s]) for s in range(W)]
        world.gather(r, rounds[r], [s for s in range(W) if s != r], list(range(W)), [0] * W, outs)
        torch.cuda.synchronize()
        for s in range(W):
            assert torch.equal(outs[s], xs[s])


def test_many_rounds_reuse_both_arena_halves():
    C = _C()
    W = 2
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(W, 1 << 16, 0)
    x = [torch.ones(4096, device=dev) * (r + 1) for r in range(W)]
    for it in range(7):
        rounds = [world.publish(r, [x[r]], None, 1) for r in range(W)]
        new = []
        for r in range(W):
            out = torch.empty(4096, device=dev)
            world.combine(r, rounds[r], [out], 0.5, [1 - r], [0.5], False, 1.0)
            new.append(out)
        x = new
    torch.cuda.synchronize()
    assert all(world.status(r)[0] == 0 for r in range(W))
    assert torch.allclose(x[0], torch.full_like(x[0], 1.5)) and torch.allclose(x[1], x[0])


def test_wait_times_out_with_error_status_instead_of_hanging():
    """A reader whose source never publishes gives up after the limit and reports it."""
    C = _C()
    dev = torch.device("cuda", 0)
    world = C.LocalWorld(2, 1 << 16, 0)
    world.set_timeout_ms(50.0)
    x = torch.ones(128, device=dev)
    r0 = world.publish(0, [x], None, 1)      # rank 1 never publishes
    out = torch.zeros(128, device=dev)
    world.combine(0, r0, [out], 0.5, [1], [0.5], False, 1.0)
    torch.cuda.synchronize()
    err, peer, want, seen = world.status(0)
    assert err == 1 and peer == 1 and want == 1 and seen == 0
    # the context is still usable
    assert torch.ones(4, device=dev).sum().item() == 4.0


def test_scale_kernel():
    C = _C()
    for dtype in (torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int32, torch.int64):
        x = (torch.arange(1003, device="cuda") % 17).to(dtype)
        ref = (x.double() * 3.0).to(dtype)
        C.scale_(x, 3.0)
        torch.cuda.synchronize()
        assert torch.equal(x, ref)
