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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_registered_tensors_are_published_in_place(dtype):
    """Tensors in registered symmetric memory: the publish is a header and a flag, the pull reads the neighbors'
    tensors where they are, and a closing wait returns once every reader is done.  Ring of three ranks, several
    versions (both arena halves), a tensor that starts inside its buffer."""
    from bluefog_b200 import _C
    W, n = 3, 100003
    es = torch.empty((), dtype=dtype).element_size()
    world = _C.LocalWorld(W, 4096, 0)                     # an arena far too small for the tensors: they never go there
    bufs = world.alloc_symmetric(n * es + 64)
    xs = [bufs[r][32:32 + n * es].view(dtype) for r in range(W)]
    outs = [torch.empty(n, device="cuda", dtype=dtype) for _ in range(W)]
    for it in range(4):
        for r in range(W):
            xs[r].copy_(torch.randn(n, device="cuda").to(dtype))
        rounds = [world.publish_in_place(r, xs[r], None, 1) for r in range(W)]
        for r in range(W):
            world.combine_in_place(r, rounds[r], xs[r], outs[r], 0.25, [(r - 1) % W], [0.75], False, 1.0)
        for r in range(W):
            world.wait_readers(r, rounds[r])
        torch.cuda.synchronize()
        for r in range(W):
            assert world.status(r)[0] == 0, world.status(r)
            ref = 0.25 * xs[r].float() + 0.75 * xs[(r - 1) % W].float()
            assert torch.allclose(outs[r].float(), ref, atol=2e-2 if dtype == torch.bfloat16 else 1e-6)


def test_registered_and_copied_payloads_mix_and_mismatches_are_reported():
    """A reader follows what each source announces: a source that copied into its arena is read there even by a rank
    that published in place; a source that published in place towards a rank without the matching registered tensor
    makes that rank report a layout mismatch (and nobody waits for ever)."""
    from bluefog_b200 import _C
    W, n = 2, 4096
    world = _C.LocalWorld(W, n * 4 + 4096, 0)
    bufs = world.alloc_symmetric(n * 4)
    x0 = torch.randn(n, device="cuda")                   # rank 0: an ordinary tensor -> arena
    x1 = bufs[1].view(torch.float32)                     # rank 1: registered -> in place
    x1.copy_(torch.randn(n, device="cuda"))
    outs = [torch.zeros(n, device="cuda") for _ in range(W)]
    r0 = world.publish_in_place(0, x0, None, 1)
    r1 = world.publish_in_place(1, x1, None, 1)
    world.combine_in_place(0, r0, x0, outs[0], 0.5, [1], [0.5], False, 1.0)
    world.combine_in_place(1, r1, x1, outs[1], 0.5, [0], [0.5], False, 1.0)
    world.wait_readers(1, r1)
    torch.cuda.synchronize()
    assert world.status(1)[0] == 0, world.status(1)
    assert torch.allclose(outs[1], 0.5 * x1 + 0.5 * x0, atol=1e-6)
    err, peer, _, _ = world.status(0)
    assert err == 6 and peer == 1, world.status(0)       # kCommLayoutMismatch, reported about rank 1
    assert torch.count_nonzero(outs[0]) == 0             # nothing was combined


def test_reader_reports_a_source_whose_payload_is_shorter_than_what_it_reads():
    """Ranks that disagree about a tensor's size (possible when negotiation is skipped): the rank that expects more
    than its source published reports a layout mismatch and combines nothing; the other direction is unaffected."""
    from bluefog_b200 import _C
    world = _C.LocalWorld(2, 1 << 20, 0)
    small, large = torch.randn(1000, device="cuda"), torch.randn(5000, device="cuda")
    out0, out1 = torch.zeros(1000, device="cuda"), torch.zeros(5000, device="cuda")
    r0 = world.publish(0, [small], None, 1)
    r1 = world.publish(1, [large], None, 1)
    world.combine(0, r0, [out0], 0.5, [1], [0.5], False, 1.0)
    world.combine(1, r1, [out1], 0.5, [0], [0.5], False, 1.0)
    torch.cuda.synchronize()
    assert world.status(0)[0] == 0
    assert torch.allclose(out0, 0.5 * small + 0.5 * large[:1000], atol=1e-6)
    err, peer, want, seen = world.status(1)
    assert err == 6 and peer == 0 and want == 20000 and seen < want, world.status(1)
    assert torch.count_nonzero(out1) == 0
