"""Window kernels (win_put / win_accumulate / win_get / win_update, versions, associated p, the device-side mutex)
on one GPU: ``LocalWindows`` lays out every rank's window block on the same device and the per-rank kernels run one
after the other, so no kernel ever waits for another launch.  Expected values are closed forms of the rank ids, as
in the reference's test/torch_win_ops_test.py, re-derived for these semantics."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int32, torch.int64]
TOL = {torch.float32: 1e-6, torch.float64: 1e-12, torch.bfloat16: 2e-2, torch.float16: 2e-3, torch.int32: 0, torch.int64: 0}


def _C():
    from bluefog_b200 import _C
    return _C


def _fill(world, W, dtype, n):
    xs = []
    for r in range(W):
        x = (torch.arange(n, device="cuda") % 7 + r + 1).to(dtype)
        world.self_tensor(r).copy_(x)
        xs.append(x.clone())
    return xs


def _close(a, ref, dtype):
    err = (a.double() - ref.double()).abs().max().item()
    assert err <= TOL[dtype] * max(1.0, ref.double().abs().max().item()), (dtype, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [4096, 1003])          # a multiple of every vector width, and a ragged length
def test_put_then_update_averages_the_ring(dtype, n):
    C = _C()
    W = 4
    world = C.LocalWindows(W, n, dtype, 0)
    xs = _fill(world, W, dtype, n)
    before = C.kernel_launch_count()
    for r in range(W):                                # everybody puts to the right neighbor
        world.put(r, world.self_tensor(r), [(r + 1) % W], [1.0])
    torch.cuda.synchronize()
    for r in range(W):
        v = world.versions(r)
        assert v[(r - 1) % W] == 1 and sum(v) == 1
        _close(world.slot_tensor(r, (r - 1) % W), xs[(r - 1) % W], dtype)
    weight = 0.5 if dtype.is_floating_point else 1.0
    for r in range(W):
        world.update(r, [(r - 1) % W], [weight], weight)
    torch.cuda.synchronize()
    assert C.kernel_launch_count() - before == 2 * W
    for r in range(W):
        ref = weight * xs[r].double() + weight * xs[(r - 1) % W].double()
        _close(world.self_tensor(r), ref.to(dtype), dtype)
        assert sum(world.versions(r)) == 0            # an update clears the versions


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32])
def test_accumulate_adds_from_several_sources_and_reset_clears(dtype):
    C = _C()
    W, n = 4, 2051
    world = C.LocalWindows(W, n, dtype, 0)
    xs = _fill(world, W, dtype, n)
    for r in range(1, W):                             # ranks 1..3 accumulate twice into rank 0
        for _ in range(2):
            world.put(r, world.self_tensor(r), [0], [1.0], 1.0, True)
    torch.cuda.synchronize()
    assert world.versions(0)[1:] == [2, 2, 2]
    for r in range(1, W):
        _close(world.slot_tensor(0, r), (2 * xs[r].double()).to(dtype), dtype)
    world.update(0, [1, 2, 3], [1.0, 1.0, 1.0], 1.0, True)
    torch.cuda.synchronize()
    ref = xs[0].double() + 2 * sum(x.double() for x in xs[1:])
    _close(world.self_tensor(0), ref.to(dtype), dtype)
    for r in range(1, W):
        assert world.slot_tensor(0, r).double().abs().max().item() == 0.0


def test_put_weights_scale_the_sent_copy_and_then_the_local_tensor():
    C = _C()
    W, n = 3, 515
    world = C.LocalWindows(W, n, torch.float32, 0)
    xs = _fill(world, W, torch.float32, n)
    world.put(0, world.self_tensor(0), [1, 2], [0.25, 2.0], 0.5)
    torch.cuda.synchronize()
    assert torch.allclose(world.slot_tensor(1, 0), 0.25 * xs[0])
    assert torch.allclose(world.slot_tensor(2, 0), 2.0 * xs[0])
    assert torch.allclose(world.self_tensor(0), 0.5 * xs[0])      # self_weight applies after sending


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_get_pulls_the_neighbors_window_tensors(dtype):
    C = _C()
    W, n = 3, 1500
    world = C.LocalWindows(W, n, dtype, 0)
    xs = _fill(world, W, dtype, n)
    w = 0.5 if dtype.is_floating_point else 1.0
    world.get(0, [1, 2], [w, 1.0])
    torch.cuda.synchronize()
    _close(world.slot_tensor(0, 1), (w * xs[1].double()).to(dtype), dtype)
    _close(world.slot_tensor(0, 2), xs[2], dtype)
    assert world.versions(0) == [0, 1, 1]


def test_push_sum_weights_follow_the_data():
    """Associated p: every rank keeps half and accumulates a quarter to each ring neighbor; collecting restores
    mass 1 per rank on average and p mirrors exactly what happened to the data."""
    C = _C()
    W, n = 4, 640
    world = C.LocalWindows(W, n, torch.float64, 0)
    for r in range(W):
        world.self_tensor(r).fill_(float(r + 1))
    for r in range(W):
        world.put(r, world.self_tensor(r), [(r + 1) % W, (r - 1) % W], [0.25, 0.25], 0.5, True, True)
    for r in range(W):
        world.update(r, [(r + 1) % W, (r - 1) % W], [1.0, 1.0], 1.0, True, True)
    torch.cuda.synchronize()
    total_p, total_x = 0.0, 0.0
    for r in range(W):
        p = world.p_values(r)
        x = world.self_tensor(r)[0].item()
        expect = 0.5 * (r + 1) + 0.25 * ((r + 1) % W + 1) + 0.25 * ((r - 1) % W + 1)
        assert abs(x - expect) < 1e-12
        assert abs(p[r] - 1.0) < 1e-12 and all(abs(p[s]) < 1e-15 for s in range(W) if s != r)
        total_p += p[r]
        total_x += x
    assert abs(total_p - W) < 1e-12 and abs(total_x - sum(range(1, W + 1))) < 1e-12


def test_device_mutex_is_taken_freed_and_times_out_without_hanging():
    C = _C()
    W, n = 2, 256
    world = C.LocalWindows(W, n, torch.float32, 0)
    xs = _fill(world, W, torch.float32, n)
    # rank 0 takes the word that guards its slot on rank 1, puts under it, frees it
    world.lock(0, [1], [0], True, 50.0)
    world.put(0, world.self_tensor(0), [1], [1.0], 1.0, False, False, True)
    world.lock(0, [1], [0], False, 50.0)
    torch.cuda.synchronize()
    assert world.lock_state(0) == [0, 0, 0]
    assert torch.equal(world.slot_tensor(1, 0), xs[0])
    # rank 1 takes the same word and keeps it; rank 0's next attempt gives up after 50 ms, reports it, and the put
    # that was to run under the mutex does nothing
    world.lock(1, [1], [0], True, 50.0)
    world.slot_tensor(1, 0).zero_()
    world.lock(0, [1], [0], True, 50.0)
    world.put(0, world.self_tensor(0), [1], [1.0], 1.0, False, False, True)
    torch.cuda.synchronize()
    assert world.lock_state(0)[:2] == [1, 1]
    assert world.slot_tensor(1, 0).abs().max().item() == 0.0
    world.lock(0, [1], [0], False, 50.0)              # frees nothing (it holds nothing) and clears the failure
    world.lock(1, [1], [0], False, 50.0)
    world.lock(0, [1], [0], True, 50.0)               # now it succeeds
    world.put(0, world.self_tensor(0), [1], [1.0], 1.0, False, False, True)
    world.lock(0, [1], [0], False, 50.0)
    torch.cuda.synchronize()
    assert world.lock_state(0) == [0, 1, 0] or world.lock_state(0)[0] == 0
    assert torch.equal(world.slot_tensor(1, 0), xs[0])
    assert torch.ones(4, device="cuda").sum().item() == 4.0
