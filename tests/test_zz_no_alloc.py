"""The allocation-free combine entry point, called through its exported C symbol.

Some users of this library must not allocate device memory when they combine buffers: their
process gave all GPU memory to a pool at start-up, or they sit in a loop where the
device-wide synchronisation of cudaMalloc would stall other streams.  For them
``bfb200_combine_noalloc`` keeps its control words in a static device array.  This test
checks it against the regular entry point (publish into a channel arena + pull-combine) on
the same data, twice in a row because the static array keeps the previous call's contents.
The file name sorts last so that a run that stops at the first failure has already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ELEM = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3}
TOL = {torch.float32: 1e-6, torch.float64: 1e-13, torch.float16: 2e-3, torch.bfloat16: 2e-2}


def _lib():
    from bluefog_b200 import _C
    lib = ctypes.CDLL(_C.__file__)
    fn = lib.bfb200_combine_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_double), ctypes.c_int,
                   ctypes.c_double, ctypes.c_double, ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return _C, fn


def _call(fn, xs, weights, self_w, post, out, stream=None):
    n_src = len(xs) - 1
    ptrs = (ctypes.c_void_p * max(n_src, 1))(*[x.data_ptr() for x in xs[1:]])
    ws = (ctypes.c_double * max(n_src, 1))(*weights)
    err = ctypes.create_string_buffer(256)
    rc = fn(xs[0].data_ptr(), ptrs, ws, n_src, self_w, post, out.data_ptr(), out.numel(), ELEM[out.dtype],
            stream, err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64, torch.float16])
def test_matches_regular_entry_point_twice_in_a_row(dtype):
    C, fn = _lib()
    dev = torch.device("cuda", 0)
    W, numel = 4, 262144 + 64
    world = C.LocalWorld(W, 4 << 20, 0)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        g = torch.Generator().manual_seed(100 + call)
        xs = [torch.randn(numel, generator=g).to(dev).to(dtype) for _ in range(W)]
        weights = [0.2, 0.3, 0.15]
        # regular path: every rank publishes into its arena, rank 0 pulls and combines
        rounds = [world.publish(r, [xs[r]], None, 1 if r else 0) for r in range(W)]
        ref = torch.empty(numel, dtype=dtype, device=dev)
        world.combine(0, rounds[0], [ref], 0.35, [1, 2, 3], weights, False, 2.0)
        out = torch.full((numel,), float("nan"), dtype=dtype, device=dev)
        rc, msg = _call(fn, xs, weights, 0.35, 2.0, out, stream)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert world.status(0)[0] == 0
        # the static scratch after a finished call: arrival counter re-armed, one call counted (the array is
        # cleared at the start of every call), every source marked consumed exactly once
        block_counter, calls_done, done = C.noalloc_scratch_words(W - 1)
        assert block_counter == 0 and calls_done == 1 and list(done) == [1] * (W - 1), (block_counter, calls_done, done)
        scale = max(1.0, ref.double().abs().max().item())
        assert (out.double() - ref.double()).abs().max().item() <= TOL[dtype] * scale, (dtype, call)


def test_rejects_what_does_not_fit():
    C, fn = _lib()
    dev = torch.device("cuda", 0)
    x = torch.ones(64, device=dev)
    out = torch.empty(64, device=dev)
    rc, msg = _call(fn, [x] * 66, [1.0] * 65, 1.0, 1.0, out)
    assert rc != 0 and "64 sources" in msg
    odd = torch.ones(63, device=dev)
    rc, msg = _call(fn, [odd, odd], [1.0], 1.0, 1.0, torch.empty(63, device=dev))
    assert rc != 0 and "multiple of 16" in msg
    host = torch.ones(64)
    rc, msg = _call(fn, [host, x], [1.0], 1.0, 1.0, out)
    assert rc != 0 and "device-accessible" in msg
    # and a valid call still works afterwards
    rc, msg = _call(fn, [x, x], [2.0], 1.0, 1.0, out)
    torch.cuda.synchronize()
    assert rc == 0 and torch.allclose(out, torch.full_like(out, 3.0))
    assert C.noalloc_scratch_words(1) == (0, 1, [1])


def test_stream_of_another_device_is_rejected():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    C, fn = _lib()
    x = torch.ones(64, device="cuda:0")
    out = torch.empty(64, device="cuda:0")
    other = torch.cuda.Stream(device=1)
    torch.cuda.set_device(0)
    rc, msg = _call(fn, [x, x], [1.0], 1.0, 1.0, out, other.cuda_stream)
    assert rc != 0 and "current device" in msg
