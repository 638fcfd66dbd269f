"""One rank of a multi-process test case: ``python tests/_worker.py <case>`` with the
torchrun-style environment set by tests/conftest.py::run_ranks.  Expected values are closed
forms of the rank ids and the known topology, as in the reference's test strategy
(test/torch_ops_test.py), re-derived here."""
import itertools
import json
import os
import sys
import time

import numpy as np
import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util as tu

CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


def dev():
    return torch.device("cuda", torch.cuda.current_device()) if bf._b.device() >= 0 else torch.device("cpu")


def close(a, b, tol=1e-5):
    assert torch.allclose(a.double().cpu(), torch.as_tensor(b, dtype=torch.float64).expand_as(a).cpu(),
                          atol=tol, rtol=tol), (a.flatten()[:4], b)


FLOATS = [torch.float32, torch.float64, torch.float16, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.float64: 1e-9, torch.float16: 1e-2, torch.bfloat16: 5e-2}


@case
def basics():
    r, n = bf.rank(), bf.size()
    assert r == int(os.environ["RANK"]) and n == int(os.environ["WORLD_SIZE"])
    assert bf.local_size() == n and bf.local_rank() == r
    assert tu.IsTopologyEquivalent(bf.load_topology(), tu.ExponentialGraph(n))
    assert bf.set_topology(tu.RingGraph(n))
    assert sorted(bf.in_neighbor_ranks()) == sorted({(r - 1) % n, (r + 1) % n} - {r})
    assert bf.set_topology(tu.ExponentialTwoGraph(n))
    expect = sorted({(r - 2 ** k) % n for k in range(int(np.log2(n - 1)) + 1)} - {r}) if n > 1 else []
    assert bf.in_neighbor_ranks() == expect
    x = torch.zeros(3, device=dev())
    assert bf.win_create(x, "basics.win")
    if n > 2:   # (for n <= 2 the ring equals the current topology, which is a no-op True)
        assert bf.set_topology(tu.RingGraph(n)) is False      # refused while a window exists
    assert bf.win_free("basics.win")
    assert bf.set_topology(tu.RingGraph(n)) is True
    for graph in (tu.ExponentialGraph(n), tu.RingGraph(n), tu.StarGraph(n), tu.MeshGrid2DGraph(n), tu.FullyConnectedGraph(n)):
        bf.set_topology(graph)
        assert bf.InferSourceFromDestinationRanks(bf.out_neighbor_ranks()) == bf.in_neighbor_ranks()
        assert bf.InferDestinationFromSourceRanks(bf.in_neighbor_ranks()) == bf.out_neighbor_ranks()
    src, W = bf.InferSourceFromDestinationRanks(bf.out_neighbor_ranks(), construct_adjacency_matrix=True)
    assert np.allclose(W.sum(axis=1), 1.0)


@case
def collectives():
    r, n, d = bf.rank(), bf.size(), dev()
    for dtype, dims in itertools.product(FLOATS, [1, 2, 3]):
        x = torch.full([3] * dims, float(r), dtype=dtype, device=d)
        close(bf.allreduce(x), (n - 1) / 2, TOL[dtype])
        close(bf.allreduce(x, average=False), n * (n - 1) / 2, TOL[dtype] * n)
        y = x.clone()
        bf.allreduce_(y)
        close(y, (n - 1) / 2, TOL[dtype])
        close(bf.broadcast(x, n - 1), n - 1, 0)
        close(x, r, 0)
        z = x.clone()
        bf.broadcast_(z, 0)
        close(z, 0, 0)
    xi = torch.full((5,), r, dtype=torch.int64, device=d)
    assert bf.allreduce(xi, average=False).tolist() == [n * (n - 1) // 2] * 5
    # allgather with a different first dimension on every rank
    g = bf.allgather(torch.full((r + 1, 2), float(r), device=d))
    assert g.shape[0] == n * (n + 1) // 2
    pos = 0
    for s in range(n):
        close(g[pos:pos + s + 1], s, 0)
        pos += s + 1
    # many small named tensors at once exercise the fusion planner
    hs = [bf.allreduce_nonblocking(torch.full((17,), float(r + i), device=d), name=f"fuse.{i}") for i in range(40)]
    for i, h in enumerate(hs):
        close(bf.synchronize(h), (n - 1) / 2 + i, 1e-5)
    # duplicate name in flight is rejected: rank 0 submits late, so the first request of the
    # other ranks is certainly still pending when their second one arrives
    if r == 0:
        time.sleep(0.5)
        close(bf.allreduce(torch.ones(8, device=d), name="dup"), 1.0, 1e-6)
    else:
        h1 = bf.allreduce_nonblocking(torch.ones(8, device=d), name="dup")
        h2 = bf.allreduce_nonblocking(torch.ones(8, device=d), name="dup")
        try:
            bf.synchronize(h2)
            raise AssertionError("duplicate name must be rejected")
        except ValueError as exc:
            assert "same name" in str(exc)
        close(bf.synchronize(h1), 1.0, 1e-6)
    bf.barrier()


@case
def neighbor_ops():
    r, n, d = bf.rank(), bf.size(), dev()
    # symmetric_empty is collective and usable everywhere: registered GPU memory on GPU ranks, an ordinary tensor on
    # CPU ranks; the operation gives the same values either way
    bf.set_topology(tu.RingGraph(n))
    sym = bf.symmetric_empty(7, 5)
    sym.fill_(float(r))
    assert sym.shape == (7, 5) and sym.device.type == d.type and bf.is_symmetric(sym) == (d.type == "cuda" and n > 1)
    ring_nb = bf.in_neighbor_ranks()
    close(bf.neighbor_allreduce(sym, name="sym.ring"), (r + sum(ring_nb)) / (len(ring_nb) + 1), 1e-6)
    for graph_fn in (tu.ExponentialTwoGraph, tu.RingGraph, tu.StarGraph, tu.MeshGrid2DGraph):
        graph = graph_fn(n)
        bf.set_topology(graph)
        nb = bf.in_neighbor_ranks()
        for dtype in FLOATS:
            x = torch.full((23, 3), float(r), dtype=dtype, device=d)
            close(bf.neighbor_allreduce(x), (r + sum(nb)) / (len(nb) + 1), TOL[dtype])
        # weighted by the topology
        bf.set_topology(graph, is_weighted=True)
        sw, nw = tu.GetRecvWeights(graph, r)
        x = torch.full((9,), float(r), dtype=torch.float64, device=d)
        close(bf.neighbor_allreduce(x), sw * r + sum(w * s for s, w in nw.items()), 1e-9)
        bf.set_topology(graph, is_weighted=False)
        # neighbor_allgather: sorted in-neighbors, self excluded
        g = bf.neighbor_allgather(torch.full((1,), float(r), device=d))
        assert g.tolist() == [float(s) for s in nb]
    bf.set_topology(tu.ExponentialTwoGraph(n))
    # explicit weights (static): sum instead of average
    x = torch.full((4,), float(r), device=d)
    nb = bf.in_neighbor_ranks()
    close(bf.neighbor_allreduce(x, self_weight=1.0, src_weights={s: 1.0 for s in nb}), r + sum(nb), 1e-5)
    # dynamic: everybody sends to rank+1 with destination weight 2
    out = bf.neighbor_allreduce(x, self_weight=0.5, src_weights={(r - 1) % n: 0.25},
                                dst_weights={(r + 1) % n: 2.0})
    close(out, 0.5 * r + 0.25 * 2.0 * ((r - 1) % n), 1e-5)
    # dynamic pattern that does not match raises on every rank instead of hanging
    try:
        bf.neighbor_allreduce(x, self_weight=0.5, src_weights={(r - 1) % n: 0.5}, dst_weights=[(r + 2) % n]
                              if n > 2 else [], name="mismatch")
        matched = (n <= 2)
    except ValueError:
        matched = True
    assert matched or n == 3
    # argument rules
    for bad in (dict(self_weight=0.5), dict(src_weights={0: 1.0}), dict(dst_weights=[(r + 1) % n])):
        try:
            bf.neighbor_allreduce(x, **bad)
            raise AssertionError("expected ValueError")
        except ValueError:
            pass
    # one-peer dynamic schedule over exp2: after log2(n) rounds everybody holds the exact mean
    if n & (n - 1) == 0 and n > 1:
        gen = tu.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), r)
        v = torch.full((3,), float(r), dtype=torch.float64, device=d)
        for _ in range(int(np.log2(n))):
            send, recv = next(gen)
            w = 1.0 / (len(recv) + 1)
            v = bf.neighbor_allreduce(v, self_weight=w, src_weights={s: w for s in recv}, dst_weights=send)
        close(v, (n - 1) / 2, 1e-9)
    # pair gossip
    partner = r ^ 1
    if partner < n:
        close(bf.pair_gossip(x, partner), (r + partner) / 2, 1e-6)
        close(bf.pair_gossip(x, partner, self_weight=0.25, pair_weight=0.75), 0.25 * r + 0.75 * partner, 1e-6)
    bf.barrier()


@case
def hierarchical():
    r, n, d = bf.rank(), bf.size(), dev()
    L = bf.local_size()
    assert L == 2 and bf.machine_size() == n // 2 and bf.machine_rank() == r // 2
    x = torch.full((6,), float(r), device=d)
    base = (r // L) * L
    close(bf.allreduce(x, is_hierarchical_local=True), sum(range(base, base + L)) / L, 1e-6)
    M = bf.machine_size()
    bf.set_machine_topology(tu.RingGraph(M))
    mean = lambda m: sum(range(m * L, m * L + L)) / L
    nbm = bf.in_neighbor_machine_ranks()
    expect = (mean(r // L) + sum(mean(m) for m in nbm)) / (len(nbm) + 1)
    close(bf.hierarchical_neighbor_allreduce(x), expect, 1e-6)
    m = r // L
    out = bf.hierarchical_neighbor_allreduce(x, self_weight=0.5, src_machine_weights={(m - 1) % M: 0.5},
                                             dst_machine_weights={(m + 1) % M: 3.0})
    close(out, 0.5 * mean(m) + 0.5 * 3.0 * mean((m - 1) % M), 1e-5)
    bf.barrier()


@case
def windows():
    r, n, d = bf.rank(), bf.size(), dev()
    bf.set_topology(tu.ExponentialTwoGraph(n))
    nb_in, nb_out = bf.in_neighbor_ranks(), bf.out_neighbor_ranks()
    for dtype in (torch.float32, torch.float64):
        x = torch.full((11, 2), float(r), dtype=dtype, device=d)
        assert bf.win_create(x, "w")
        assert bf.get_current_created_window_names() == ["w"]
        # slots start as copies of the local tensor
        close(bf.win_update("w", clone=True), r, 1e-6)
        bf.barrier()
        assert bf.win_put(x, "w")
        bf.barrier()
        assert bf.get_win_version("w") == {s: 1 for s in nb_in}
        out = bf.win_update("w")
        assert out.data_ptr() == x.data_ptr()
        close(x, (r + sum(nb_in)) / (len(nb_in) + 1), 1e-6)
        assert bf.get_win_version("w") == {s: 0 for s in nb_in}
        bf.barrier()
        # accumulate twice with weights, then collect
        x.fill_(float(r))
        bf.win_update("w", self_weight=1.0, neighbor_weights={s: 0.0 for s in nb_in}, reset=True)
        bf.barrier()
        for _ in range(2):
            bf.win_accumulate(x, "w", dst_weights={s: 0.5 for s in nb_out})
        bf.barrier()
        close(bf.win_update_then_collect("w"), r + sum(nb_in), 1e-5)
        bf.barrier()
        # get pulls the neighbors' registered tensors
        x.fill_(float(r))
        bf.barrier()
        bf.win_get("w")
        bf.barrier()
        close(bf.win_update("w", self_weight=0.0, neighbor_weights={s: 1.0 for s in nb_in}), sum(nb_in), 1e-5)
        bf.barrier()
        assert bf.win_free("w")
    # push-sum weights: p tracks a ones tensor through put/update rounds
    bf.turn_on_win_ops_with_associated_p()
    x = torch.ones(5, device=d)
    bf.win_create(x, "p", zero_init=True)
    outdeg = len(nb_out)
    for _ in range(5):
        bf.barrier()
        bf.win_accumulate(x, "p", self_weight=1.0 / (outdeg + 1), dst_weights={s: 1.0 / (outdeg + 1) for s in nb_out},
                          require_mutex=True)
        bf.barrier()
        bf.win_update_then_collect("p")
        close(x, bf.win_associated_p("p"), 1e-6)
    total = bf.allreduce(torch.tensor([bf.win_associated_p("p")], dtype=torch.float64), average=True)
    close(total, 1.0, 1e-9)
    bf.turn_off_win_ops_with_associated_p()
    bf.win_free()
    # mutex: rank 0 holds its own slots for a second, writers must wait
    x = torch.zeros(3, device=d)
    bf.win_create(x, "m")
    bf.barrier()
    if r == 0:
        with bf.win_mutex("m", for_self=True, ranks=nb_in):
            bf.barrier()
            time.sleep(1.0)
    else:
        bf.barrier()
        t0 = time.time()
        if 0 in nb_out:
            bf.win_put(x, "m", dst_weights={0: 1.0}, require_mutex=True)
            assert time.time() - t0 > 0.7
    bf.barrier()
    bf.win_free("m")


@case
def errors():
    r, n = bf.rank(), bf.size()
    for kind in ("shape", "dtype", "root"):
        try:
            if kind == "shape":
                bf.allreduce(torch.zeros(3 + (r == 0)), name="e.shape")
            elif kind == "dtype":
                bf.allreduce(torch.zeros(3, dtype=torch.float32 if r else torch.float64), name="e.dtype")
            else:
                bf.broadcast(torch.zeros(3), 0 if r else 1, name="e.root")
            raise AssertionError("expected an error for " + kind)
        except ValueError as exc:
            assert "Mismatched" in str(exc)
    try:
        bf.allreduce(torch.zeros(4, dtype=torch.uint8))
        raise AssertionError("uint8 allreduce must be rejected")
    except ValueError:
        pass
    try:
        bf.allreduce(torch.zeros(4, 4).t())
        raise AssertionError("non-contiguous must be rejected")
    except ValueError:
        pass
    # the runtime is still healthy
    assert bf.allreduce(torch.ones(2)).tolist() == [1.0, 1.0]


@case
def neighbor_sweeps():
    """dtype x dimension sweeps of the neighbor operations and the exactness case with 2**-256 doubles
    (the matrix of the reference's test/torch_ops_test.py:366-428, 834-871, re-derived from the topology)."""
    r, n, d = bf.rank(), bf.size(), dev()
    bf.set_topology(tu.ExponentialTwoGraph(n))
    nb, out_nb = bf.in_neighbor_ranks(), bf.out_neighbor_ranks()
    for dtype, dim in itertools.product(FLOATS, (1, 2, 3)):
        shape = (23,) * dim
        x = torch.full(shape, float(r), dtype=dtype, device=d)
        tag = "%s.%d" % (str(dtype).split(".")[-1], dim)
        y = bf.neighbor_allreduce(x, name="sweep.avg." + tag)
        assert tuple(y.shape) == shape and y.dtype == dtype
        close(y, (r + sum(nb)) / (len(nb) + 1), TOL[dtype])
        y = bf.neighbor_allreduce(x, self_weight=1.0, src_weights={s: 1.0 for s in nb}, name="sweep.sum." + tag)
        close(y, r + sum(nb), TOL[dtype] * max(1, n))
        # destination weights as a dictionary: every sender scales what it sends by 0.5
        y = bf.neighbor_allreduce(x, self_weight=0.5, src_weights={s: 1.0 for s in nb},
                                  dst_weights={t: 0.5 for t in out_nb}, name="sweep.dst." + tag)
        close(y, 0.5 * (r + sum(nb)), TOL[dtype] * max(1, n))
        g = bf.neighbor_allgather(x, name="sweep.gather." + tag)
        assert tuple(g.shape) == (23 * len(nb),) + shape[1:]
        for k, s in enumerate(nb):
            close(g[23 * k:23 * (k + 1)], float(s), TOL[dtype])
    # variable first dimension in neighbor_allgather
    g = bf.neighbor_allgather(torch.full((r + 1, 2), float(r), device=d), name="sweep.ragged")
    assert g.shape[0] == sum(s + 1 for s in nb)
    # sums and averages of 2**-256 are exact in double precision: no detour through a narrower type
    tiny = 2.0 ** -256
    for dim in (1, 2, 3):
        x = torch.full((23,) * dim, tiny, dtype=torch.float64, device=d)
        y = bf.neighbor_allreduce(x, self_weight=1.0, src_weights={s: 1.0 for s in nb}, name="tiny.sum.%d" % dim)
        assert (y.cpu() - (len(nb) + 1) * tiny).abs().max().item() == 0.0
        if (len(nb) + 1) & len(nb) == 0:       # 1/(deg+1) is a power of two: the average is exact as well
            y = bf.neighbor_allreduce(x, name="tiny.avg.%d" % dim)
            assert (y.cpu() - tiny).abs().max().item() == 0.0
        y = bf.allreduce(x, average=False, name="tiny.allreduce.%d" % dim)
        assert (y.cpu() - n * tiny).abs().max().item() == 0.0
    bf.barrier()


@case
def win_random_p():
    """Ten rounds of puts, updates and accumulates with random weights: the associated p must follow the window
    value exactly, whatever the weights were (reference test/torch_win_ops_test.py:822-857)."""
    r, n, d = bf.rank(), bf.size(), dev()
    bf.set_topology(tu.ExponentialTwoGraph(n))
    bf.turn_on_win_ops_with_associated_p()
    rng = np.random.RandomState(1000 + r)
    for dtype in (torch.float32, torch.float64):
        x = torch.ones(23, dtype=dtype, device=d)
        name = "win.random.p.%s" % str(dtype).split(".")[-1]
        assert bf.win_create(x, name, zero_init=True)
        outs = bf.out_neighbor_ranks()
        for _ in range(10):
            w = rng.rand(len(outs) + 1)
            w /= w.sum()
            dst = {t: float(w[i]) for i, t in enumerate(outs)}
            bf.win_put(x, name=name, self_weight=float(w[-1]), dst_weights=dst, require_mutex=True)
            bf.win_update(name=name, require_mutex=True)
            bf.win_accumulate(x, name=name, self_weight=float(w[-1]), dst_weights=dst, require_mutex=True)
            bf.win_update_then_collect(name=name)
        bf.barrier()
        y = bf.win_update_then_collect(name=name)
        p = bf.win_associated_p(name=name)
        tol = 1e-4 if dtype == torch.float32 else 1e-9
        assert abs(p - float(y[0])) < tol * max(1.0, abs(p)), (p, float(y[0]))
        assert (y - y[0]).abs().max().item() < tol * max(1.0, abs(p))
        bf.barrier()
        bf.win_free(name)
    bf.turn_off_win_ops_with_associated_p()
    # the sum of p over all ranks is the number of ranks: mass is only moved
    bf.barrier()


@case
def optimizer_warnings():
    """A layer that runs twice per forward pass must not trip the local-step check; a forward pass too many
    without step() must (reference test/torch_optimizer_test.py:601-717)."""
    import warnings
    r, n = bf.rank(), bf.size()

    class Duplicated(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = torch.nn.Linear(6, 4)
            self.fc2 = torch.nn.Linear(4, 4)

        def forward(self, x):
            return self.fc2(self.fc2(self.fc1(x)))

    factories = [
        lambda o, m, j: bf.DistributedAdaptWithCombineOptimizer(o, m, num_steps_per_communication=j),
        lambda o, m, j: bf.DistributedAdaptThenCombineOptimizer(o, m, num_steps_per_communication=j),
        lambda o, m, j: bf.DistributedGradientAllreduceOptimizer(o, m, num_steps_per_communication=j),
        lambda o, m, j: bf.DistributedWinPutOptimizer(o, m, num_steps_per_communication=j),
    ]
    x = torch.randn(8, 6, generator=torch.Generator().manual_seed(r))
    for k, make in enumerate(factories):
        for j in (1, 2):
            torch.manual_seed(7)
            model = Duplicated()
            opt = make(torch.optim.SGD(model.parameters(), lr=0.05), model, j)
            with warnings.catch_warnings():
                warnings.filterwarnings("error", message="Unexpected behavior")
                for it in range(2 * j):
                    if it % j == 0:
                        opt.zero_grad()
                    model(x).pow(2).mean().backward()
                    opt.step()
            if hasattr(opt, "unregister_window"):
                opt.unregister_window()
            bf.barrier()
    # one forward/backward too many between two steps
    torch.manual_seed(7)
    model = Duplicated()
    opt = bf.DistributedAdaptWithCombineOptimizer(torch.optim.SGD(model.parameters(), lr=0.05), model)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        opt.zero_grad()
        model(x).pow(2).mean().backward()
        model(x).pow(2).mean().backward()
        opt.step()
    assert any("Unexpected behavior" in str(w.message) for w in caught), [str(w.message)[:40] for w in caught]
    bf.barrier()


@case
def checkpoint_root_only():
    """Only the root finds the file: parameters, optimizer state, BatchNorm buffers and the extra entry must reach
    every rank."""
    r, n = bf.rank(), bf.size()
    path = os.environ["BFB_CKPT"]

    def make():
        torch.manual_seed(100 + r)
        m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.BatchNorm1d(3))
        o = bf.DistributedAdaptWithCombineOptimizer(torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9), m)
        return m, o

    model, opt = make()
    for _ in range(2):
        opt.zero_grad()
        model(torch.randn(5, 4)).sum().backward()
        opt.step()
    bf.save_checkpoint(path, model, opt, extra={"iteration": 11, "schedule": [1, 2]})
    bf.barrier()
    saved = torch.load(path, weights_only=False)
    model2, opt2 = make()
    extra = bf.load_checkpoint(path if r == 0 else path + ".not.here", model2, opt2)
    assert extra == {"iteration": 11, "schedule": [1, 2]}, extra
    for k, v in model2.state_dict().items():
        assert torch.allclose(v.double(), saved["model"][k].double()), k
    mom = [opt2.state[p]["momentum_buffer"] for p in model2.parameters()]
    ref = [saved["optimizer"]["state"][i]["momentum_buffer"] for i in range(len(mom))]
    for a, b in zip(mom, ref):
        assert torch.allclose(a, b)
    bf.barrier()


@case
def consensus():
    """Average-consensus workload: 100 000 fp32 values N(0,1) from seed=rank, static exp2, 200 rounds."""
    r, n = bf.rank(), bf.size()
    bf.set_topology(tu.ExponentialTwoGraph(n))
    x = torch.randn(100000, generator=torch.Generator().manual_seed(r))
    mean = bf.allreduce(x)
    devs, early = [], []
    for it in range(200):
        x = bf.neighbor_allreduce(x, name="consensus")
        if it < 10:
            early.append(bf.allreduce((x - mean).abs().max().reshape(1), average=False).item())
        if it % 10 == 9:
            devs.append(bf.allreduce((x - mean).abs().max().reshape(1), average=False).item())
    assert devs[-1] < 1e-5, devs
    # geometric decay: the fitted rate of the first rounds (before fp32 rounding takes over) is the second largest
    # eigenvalue modulus of the uniform-weight combination matrix of the topology
    W = np.zeros((n, n))
    topo = bf.load_topology()
    for i in range(n):
        srcs = [s for s in topo.predecessors(i) if s != i]
        for s in srcs + [i]:
            W[i, s] = 1.0 / (len(srcs) + 1)
    rho = sorted(np.abs(np.linalg.eigvals(W)))[-2] if n > 1 else 0.0
    usable = [v for v in early if v > 1e-5]
    if len(usable) >= 4 and rho > 0:
        rate = float(np.exp(np.polyfit(np.arange(len(usable)), np.log(usable), 1)[0]))
        assert rate < rho * 1.25 + 0.02, (rate, rho, early)
        if r == 0:
            print("consensus fitted rate %.4f, second eigenvalue modulus %.4f" % (rate, rho))
    if r == 0:
        print("consensus deviations", devs[:6])


@case
def timeline():
    r = bf.rank()
    x = torch.ones(10)
    for i in range(3):
        bf.neighbor_allreduce(x, name="tl.tensor")
        bf.allreduce(x, name="tl.ar")
    with bf.timeline_context("user.tensor", "USER_ACTIVITY"):
        time.sleep(0.01)
    bf.barrier()
    bf.shutdown()
    path = os.environ["BLUEFOG_TIMELINE"] + str(r) + ".json"
    text = open(path).read()
    for token in ("ENQUEUE_NEIGHBOR_ALLREDUCE", "PROC_NEIGHBOR_ALLREDUCE", "COMMUNICATE", "COMPUTE_AVERAGE",
                  "USER_ACTIVITY", "tl.tensor", "process_name"):
        assert token in text, token
    events = json.loads(text.rstrip().rstrip(",") + "]")
    assert sum(e["ph"] == "B" for e in events) == sum(e["ph"] == "E" for e in events)


@case
def skip_negotiate():
    r, n = bf.rank(), bf.size()
    bf.set_skip_negotiate_stage(True)
    assert bf.get_skip_negotiate_stage()
    x = torch.full((4,), float(r))
    close(bf.allreduce(x), (n - 1) / 2, 1e-6)
    bf.barrier()
    bf.set_skip_negotiate_stage(False)
    close(bf.allreduce(x), (n - 1) / 2, 1e-6)


@case
def rank_exits_early():
    """A rank that leaves makes the others' next collective fail instead of hang."""
    r = bf.rank()
    bf.allreduce(torch.ones(1))
    if r == 1:
        bf.shutdown()
        return
    time.sleep(0.5)
    try:
        bf.allreduce(torch.ones(1), name="after")
        raise AssertionError("expected failure after a rank left")
    except RuntimeError as exc:
        assert "shut down" in str(exc)


@case
def stall_warning():
    r = bf.rank()
    bf._b.native.set_stall_warning_seconds(1.0)
    if r == 1:
        time.sleep(7.0)
    bf.allreduce(torch.ones(1), name="late.tensor")


@case
def optimizers():
    r, n, d = bf.rank(), bf.size(), dev()
    torch.manual_seed(0)
    w_true = torch.randn(16, 3)
    g = torch.Generator().manual_seed(100 + r)
    x = torch.randn(256, 16, generator=g)
    y = x @ w_true + 0.1 * torch.randn(256, 3, generator=g)
    x, y = x.to(d), y.to(d)
    styles = [("awc", bf.DistributedAdaptWithCombineOptimizer, {}),
              ("atc", bf.DistributedAdaptThenCombineOptimizer, {}),
              ("grad", bf.DistributedGradientAllreduceOptimizer, {}),
              ("awc_allreduce", bf.DistributedAllreduceOptimizer, {}),
              ("awc_j2", bf.DistributedAdaptWithCombineOptimizer, {"num_steps_per_communication": 2}),
              ("win_put", bf.DistributedWinPutOptimizer, {}),
              ("pull_get", bf.DistributedPullGetOptimizer, {}),
              ("push_sum", bf.DistributedPushSumOptimizer, {}),
              # one window per parameter, the layout of the reference
              ("win_put", bf.DistributedWinPutOptimizer, {"bucket_bytes": 0}),
              ("push_sum", bf.DistributedPushSumOptimizer, {"bucket_bytes": 0})]
    for name, factory, kw in styles:
        torch.manual_seed(1)
        model = torch.nn.Linear(16, 3).to(d)
        bf.broadcast_parameters(model.state_dict(), 0)
        opt = factory(torch.optim.Adam(model.parameters(), lr=0.05), model, **kw)
        if name in ("win_put", "pull_get"):
            opt.force_barrier = True
        assert isinstance(opt, torch.optim.Adam)
        J = kw.get("num_steps_per_communication", 1)
        for ep in range(60):
            opt.zero_grad()
            for _ in range(J if name != "awc_j2" else 1):
                loss = torch.nn.functional.mse_loss(model(x), y)
                loss.backward()
            opt.step()
        assert loss.item() < 0.08, (name, loss.item())
        if name in ("win_put", "pull_get", "push_sum"):
            windows = bf.get_current_created_window_names()
            # bias and weight share one bucket window by default; per-parameter mode keeps one window each
            assert len(windows) == (2 if kw.get("bucket_bytes") == 0 else 1), windows
        sd = opt.state_dict()
        assert set(sd.keys()) == {"state", "param_groups"}
        bf.win_free()
        bf.barrier()
    # dynamic one-peer weights set between steps
    model = torch.nn.Linear(16, 3).to(d)
    opt = bf.DistributedNeighborAllreduceOptimizer(torch.optim.SGD(model.parameters(), lr=0.2), model)
    gen = tu.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), r)
    for ep in range(80):
        send, recv = next(gen)
        opt.dst_weights = send
        opt.src_weights = {s: 1.0 / (len(recv) + 1) for s in recv}
        opt.self_weight = 1.0 / (len(recv) + 1)
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
    assert loss.item() < 0.5
    bf.barrier()


@case
def checkpoint():
    r, n = bf.rank(), bf.size()
    path = os.environ["BFB_CKPT"]
    torch.manual_seed(r)
    model = torch.nn.Linear(4, 2)
    opt = bf.DistributedAdaptWithCombineOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9), model)
    opt.zero_grad()
    model(torch.ones(1, 4)).sum().backward()
    opt.step()
    bf.save_checkpoint(path, model, opt, extra={"iteration": 7})
    bf.barrier()
    payload = torch.load(path, weights_only=False)
    assert set(payload.keys()) == {"model", "optimizer", "extra"}
    assert set(payload["model"].keys()) == {"weight", "bias"}
    model2 = torch.nn.Linear(4, 2)
    opt2 = bf.DistributedAdaptWithCombineOptimizer(torch.optim.SGD(model2.parameters(), lr=0.1, momentum=0.9), model2)
    extra = bf.load_checkpoint(path, model2, opt2)
    assert extra == {"iteration": 7}
    w0 = bf.broadcast(model2.weight.data, 0)
    assert torch.equal(w0, model2.weight.data) and torch.equal(model2.weight.data, payload["model"]["weight"])
    bf.barrier()


@case
def gpu_fused_wrap_then_broadcast():
    """The order of the reference's examples: every rank starts from its own random model, wraps the optimizer,
    THEN broadcasts parameters and optimizer state.  The first combine must see the broadcast values on every
    neighbor (fp32 compute: the master is written in place; bf16 compute: the shadow is), and after one step with
    zero gradients every rank must still hold exactly the root's model."""
    r, n, d = bf.rank(), bf.size(), dev()
    assert d.type == "cuda"
    bf.set_topology(tu.RingGraph(n))
    for compute in (torch.float32, torch.bfloat16):
        for factory in (bf.DistributedAdaptWithCombineOptimizer, bf.DistributedAdaptThenCombineOptimizer):
            torch.manual_seed(1000 + r)                      # a different model on every rank
            model = torch.nn.Sequential(torch.nn.Linear(32, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4)).to(d)
            opt = factory(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9), model, compute_dtype=compute)
            assert hasattr(opt, "master_parameters")
            bf.broadcast_parameters(model.state_dict(), root_rank=0)
            bf.broadcast_optimizer_state(opt, root_rank=0)
            root = torch.cat([v.float().reshape(-1) for v in model.state_dict().values()]).clone()
            root0 = bf.broadcast(root, 0)
            assert torch.equal(root, root0), "the broadcast itself did not reach this rank"
            opt.zero_grad()
            (model(torch.zeros(2, 32, device=d, dtype=compute)).sum() * 0.0).backward()     # zero gradients
            opt.step()
            torch.cuda.synchronize()
            opt.check()
            now = torch.cat([v.float().reshape(-1) for v in model.state_dict().values()])
            tol = 0.0 if compute == torch.float32 else 1e-2
            assert (now - root0).abs().max().item() <= tol + 1e-6, (compute, factory.__name__, (now - root0).abs().max().item())
            masters = torch.cat([v.reshape(-1) for v in opt.master_parameters().values()])
            assert (masters - root0).abs().max().item() <= tol + 1e-6
            bf.barrier()


@case
def gpu_fused_dst_weights_and_hierarchical():
    """Fused engine against the per-parameter path (fused=False) with destination weights that change every step,
    and with hierarchical averaging over two machines."""
    r, n, d = bf.rank(), bf.size(), dev()
    assert d.type == "cuda"
    bf.set_topology(tu.RingGraph(n))

    def run(fused, comm, steps=4):
        torch.manual_seed(5)
        model = torch.nn.Linear(24, 6).to(d)
        with torch.no_grad():
            for p in model.parameters():
                p.add_(0.1 * r)
        factory = bf.DistributedAdaptWithCombineOptimizer if comm[0] == "awc" else bf.DistributedAdaptThenCombineOptimizer
        ctype = bf.CommunicationType.hierarchical_neighbor_allreduce if comm[1] == "hier" else bf.CommunicationType.neighbor_allreduce
        opt = factory(torch.optim.SGD(model.parameters(), lr=0.05), model, communication_type=ctype, fused=fused)
        x = torch.randn(16, 24, generator=torch.Generator().manual_seed(r)).to(d)
        for t in range(steps):
            if comm[1] == "dst":
                opt.self_weight = 0.5
                opt.src_weights = {(r - 1) % n: 0.5}
                opt.dst_weights = {(r + 1) % n: 0.5 + 0.25 * ((r + t) % 3)}
            opt.zero_grad()
            model(x).pow(2).mean().backward()
            opt.step()
        torch.cuda.synchronize()
        return torch.cat([p.detach().reshape(-1) for p in model.parameters()]).clone()

    kinds = [("awc", "dst"), ("atc", "dst")] if n > 1 else []
    if bf.local_size() > 1 and bf.machine_size() > 1:
        bf.set_machine_topology(tu.RingGraph(bf.machine_size()))
        kinds += [("awc", "hier"), ("atc", "hier")]
    for comm in kinds:
        a, b = run(True, comm), run(False, comm)
        assert (a - b).abs().max().item() < 1e-4, (comm, (a - b).abs().max().item())
        bf.barrier()


@case
def gpu_fused_optimizers():
    """Fused bucket engine on real GPUs: consensus of the parameters and convergence."""
    r, n, d = bf.rank(), bf.size(), dev()
    assert d.type == "cuda"
    torch.manual_seed(0)
    w_true = torch.randn(64, 8)
    g = torch.Generator().manual_seed(100 + r)
    x = torch.randn(512, 64, generator=g)
    y = (x @ w_true + 0.1 * torch.randn(512, 8, generator=g)).to(d)
    x = x.to(d)
    for style, factory in (("awc", bf.DistributedAdaptWithCombineOptimizer),
                           ("atc", bf.DistributedAdaptThenCombineOptimizer),
                           ("grad", bf.DistributedGradientAllreduceOptimizer)):
        for compute in (torch.float32, torch.bfloat16):
            torch.manual_seed(1)
            model = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8)).to(d)
            bf.broadcast_parameters(model.state_dict(), 0)
            opt = factory(torch.optim.Adam(model.parameters(), lr=0.01), model, compute_dtype=compute)
            assert hasattr(opt, "master_parameters"), "the fused engine must be used on GPUs"
            gen = tu.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), r)
            first = None
            for it in range(150):
                if style != "grad" and n > 1:
                    send, recv = next(gen)
                    opt.dst_weights, opt.self_weight = send, 1.0 / (len(recv) + 1)
                    opt.src_weights = {s: 1.0 / (len(recv) + 1) for s in recv}
                opt.zero_grad()
                loss = torch.nn.functional.mse_loss(model(x.to(compute)).float(), y)
                loss.backward()
                opt.step()
                first = first if first is not None else loss.item()
            torch.cuda.synchronize()
            opt.check()
            assert loss.item() < 0.25 * first, (style, compute, first, loss.item())
            flat = torch.cat([v.reshape(-1) for v in opt.master_parameters().values()])
            spread = bf.allreduce((flat - bf.allreduce(flat)).abs().max().reshape(1), average=False).item()
            assert spread < (1e-5 if style == "grad" else 0.2), (style, compute, spread)
            bf.barrier()


@case
def runtime_stats():
    """Counters of the runtime: per-type operation counts, payload bytes, failures, and the Prometheus view of them."""
    r, n = bf.rank(), bf.size()
    d = dev()
    bf.set_topology(bf.RingGraph(n))
    before = bf.runtime_stats()
    x = torch.full((1000,), float(r), device=d)
    for k in range(5):
        bf.neighbor_allreduce(x, name=f"stats.na.{k}")
    bf.allreduce(x, name="stats.ar")
    hs = [bf.neighbor_allreduce_nonblocking(torch.full((10,), 1.0, device=d), name=f"stats.small.{k}") for k in range(6)]
    for h in hs:
        bf.synchronize(h)
    after = bf.runtime_stats()

    def delta(key):
        return after.get(key, 0) - before.get(key, 0)

    assert delta("enqueued.NEIGHBOR_ALLREDUCE") == 11 and delta("enqueued.ALLREDUCE") == 1, after
    assert delta("input_bytes") == 6 * 4000 + 6 * 40
    assert delta("operations_failed") == 0
    if d.type == "cpu":
        assert delta("responses_executed") >= 1 and delta("issued_on_calling_thread") == 0
    # a failing operation is counted
    try:
        bf.neighbor_allreduce(x, self_weight=0.5, name="stats.bad")           # src_weights missing
    except ValueError:
        pass
    from bluefog_b200.utils import metrics
    snap = metrics.snapshot()
    assert snap["rank"] == r and snap["size"] == n and snap["enqueued.NEIGHBOR_ALLREDUCE"] >= 11
    try:
        import prometheus_client
    except ImportError:
        prometheus_client = None
    if prometheus_client is not None:
        reg = prometheus_client.CollectorRegistry()
        reg.register(metrics._Collector())
        text = prometheus_client.generate_latest(reg).decode()
        assert f'bluefog_b200_operations_enqueued_total{{rank="{r}",type="neighbor_allreduce"}}' in text, text[:600]
        assert "bluefog_b200_input_bytes_total" in text
    bf.barrier()


@case
def win_guard():
    """Guard words behind every region of a window: untouched by put / accumulate / get / update of ragged sizes, and
    a byte written past the end of the tensor is reported when the window is freed."""
    import ctypes
    r, n = bf.rank(), bf.size()
    d = dev()
    bf.set_topology(bf.RingGraph(n))
    for numel in (1, 100, 64, 4099):
        x = torch.full((numel,), float(r), device=d)
        assert bf.win_create(x, f"guard.{numel}", zero_init=True)
        bf.win_put(x, f"guard.{numel}")
        bf.win_accumulate(x, f"guard.{numel}")
        bf.barrier()
        bf.win_update(f"guard.{numel}")
        bf.win_get(f"guard.{numel}")
        bf.barrier()
        assert bf.win_free(f"guard.{numel}"), "guard words damaged by regular operations"
    if d.type == "cpu":
        # 100 floats = 400 bytes in a region of 512: the guard is its last 16 bytes
        y = torch.zeros(100)
        assert bf.win_create(y, "guard.hit")
        bf.barrier()
        if r == 0:
            ctypes.memset(y.data_ptr() + 500, 0x11, 1)
        ok = bf.win_free("guard.hit")
        assert ok == (r != 0), (r, ok)
    bf.barrier()


@case
def gpu_registered_tensors():
    """neighbor_allreduce of tensors in symmetric memory (published in place), with and without negotiation, static
    and per-call weights, a slice of a registered tensor, and the same values as the copying path."""
    r, n = bf.rank(), bf.size()
    d = dev()
    bf.set_topology(bf.RingGraph(n))
    nb = bf.in_neighbor_ranks()
    w = 1.0 / (len(nb) + 1)
    numel = 3 * 1024 * 1024 + 77
    x = bf.symmetric_empty(numel, dtype=torch.float32)
    assert bf.is_symmetric(x) and x.is_cuda and x.shape == (numel,)
    assert not bf.is_symmetric(torch.empty(16, device=d))
    base = torch.arange(numel, device=d, dtype=torch.float32) % 11.0
    for skip in (False, True):
        bf.set_skip_negotiate_stage(skip)
        for it in range(3):
            x.copy_(base + r + it)
            out = bf.neighbor_allreduce(x, name=f"reg.{int(skip)}.{it}")
            ref = w * ((base + r + it) + sum(base + q + it for q in nb))
            assert torch.allclose(out, ref, atol=1e-5), (out[:4], ref[:4])
            # the tensor is the caller's again when the call returns: overwrite it right away
            x.zero_()
        bf.barrier()
    bf.set_skip_negotiate_stage(False)
    # a 16-byte aligned slice, bf16, explicit weights; the copying path on an ordinary tensor gives the same values
    xb = bf.symmetric_empty(2, 70000, dtype=torch.bfloat16)
    xb.copy_(((torch.arange(140000, device=d) % 13).float() + r).view(2, 70000))
    part = xb[1, 8:60008]
    assert bf.is_symmetric(part)
    sw = {q: 0.5 / len(nb) for q in nb}
    got = bf.neighbor_allreduce(part, self_weight=0.5, src_weights=sw, name="reg.slice")
    want = bf.neighbor_allreduce(part.clone(), self_weight=0.5, src_weights=sw, name="reg.slice.copy")
    assert torch.equal(got, want)
    # nonblocking series on registered tensors
    ys = [bf.symmetric_empty(5000 + k) for k in range(4)]
    for k, y in enumerate(ys):
        y.fill_(float(r + k))
    hs = [bf.neighbor_allreduce_nonblocking(y, name=f"reg.series.{k}") for k, y in enumerate(ys)]
    for k, h in enumerate(hs):
        close(bf.synchronize(h), w * ((r + k) + sum(q + k for q in nb)), 1e-5)
    bf.barrier()


@case
def gpu_fast_path():
    """Negotiation-free GPU collectives issued on the calling thread: blocking, nonblocking series, mixed
    with queued operations, and large tensors right before small ones."""
    r, n = bf.rank(), bf.size()
    d = dev()
    bf.set_topology(bf.RingGraph(n))
    bf.set_skip_negotiate_stage(True)
    nb = bf.in_neighbor_ranks()
    w = 1.0 / (len(nb) + 1)
    expect = w * (r + sum(nb))
    # a series of nonblocking operations on the fast path, waited for at the end
    xs = [torch.full((1000 + k,), float(r + k), device=d) for k in range(6)]
    hs = [bf.neighbor_allreduce_nonblocking(x, name=f"series.{k}") for k, x in enumerate(xs)]
    for k, h in enumerate(hs):
        close(bf.synchronize(h), w * ((r + k) + sum(q + k for q in nb)), 1e-5)
    # poll completes a fast-path handle as well
    h = bf.allreduce_nonblocking(torch.full((64,), float(r), device=d), name="polled")
    while not bf.poll(h):
        pass
    close(bf.synchronize(h), (n - 1) / 2, 1e-6)
    # a duplicate name in flight is refused
    big = torch.full((1 << 22,), 1.0, device=d)
    h1 = bf.neighbor_allreduce_nonblocking(big, name="dup")
    try:
        bf.synchronize(bf.neighbor_allreduce_nonblocking(big, name="dup"))
        raised = False
    except ValueError:
        raised = True
    bf.synchronize(h1)
    assert raised, "a second operation with a name that is still in flight must be refused"
    bf.barrier()
    # CPU operations take the queue; GPU operations issued after them keep their place behind them
    c = bf.allreduce_nonblocking(torch.full((8,), float(r)), name="cpu.first")
    g = bf.allreduce_nonblocking(torch.full((8,), float(r), device=d), name="gpu.second")
    close(bf.synchronize(g), (n - 1) / 2, 1e-6)
    close(bf.synchronize(c), (n - 1) / 2, 1e-6)
    # 40 MiB + a ragged tail, fp32 and bf16, static and with explicit weights
    numel = 10 * 1024 * 1024 + 12345
    base = torch.arange(numel, device=d, dtype=torch.float32) % 7.0
    x = base + r
    out = bf.neighbor_allreduce(x, name="large.f32")
    ref = w * (x + sum(base + q for q in nb))
    assert torch.allclose(out, ref, atol=1e-5), (out[:4], ref[:4])
    assert torch.allclose(out[-5:], ref[-5:], atol=1e-5)
    xb = (base + r).to(torch.bfloat16).repeat(2)
    outb = bf.neighbor_allreduce(xb, self_weight=0.5, src_weights={q: 0.5 / len(nb) for q in nb}, name="large.bf16")
    refb = 0.5 * xb.float() + sum((0.5 / len(nb)) * (base + q).to(torch.bfloat16).repeat(2).float() for q in nb)
    assert torch.allclose(outb.float(), refb, atol=0.1), (outb[:4], refb[:4])
    # and a small operation right behind the large one
    close(bf.neighbor_allreduce(torch.full((16,), float(r), device=d), name="after"), expect, 1e-5)
    bf.barrier()
    bf.set_skip_negotiate_stage(False)
    # with negotiation the same large tensor goes through the queued path
    out2 = bf.neighbor_allreduce(x, name="large.negotiated")
    assert torch.allclose(out2, ref, atol=1e-5)


@case
def gpu_pair_gossip():
    """pair_gossip of CUDA tensors over the two-rank peer-memory channels: concurrent disjoint pairs,
    changing partners, weights, a tensor that makes the pair arena grow, 16-bit payloads."""
    r, n = bf.rank(), bf.size()
    d = dev()
    bf.set_skip_negotiate_stage(True)
    for bit in (1, 2):
        partner = r ^ bit
        if partner >= n:
            continue
        x = torch.full((1000,), float(r), device=d)
        close(bf.pair_gossip(x, partner), (r + partner) / 2, 1e-6)
        close(bf.pair_gossip(x, partner, self_weight=0.25, pair_weight=0.75), 0.25 * r + 0.75 * partner, 1e-6)
        hs = [bf.pair_gossip_nonblocking(torch.full((64 + k,), float(r + k), device=d), partner, name=f"pg.{bit}.{k}")
              for k in range(4)]
        for k, h in enumerate(hs):
            close(bf.synchronize(h), (r + partner) / 2 + k, 1e-6)
        big = torch.full((20 * 1024 * 1024 + 3,), float(r), device=d, dtype=torch.bfloat16)   # grows the pair arena
        out = bf.pair_gossip(big, partner)
        close(out[:8], (r + partner) / 2, 1e-2)
        close(out[-8:], (r + partner) / 2, 1e-2)
        close(bf.pair_gossip(torch.full((7,), float(r), device=d, dtype=torch.float64), partner), (r + partner) / 2, 1e-12)
    bf.barrier()
    # a collective of all ranks right after the gossips uses the common channel, whose versions did not move
    bf.set_skip_negotiate_stage(False)
    close(bf.allreduce(torch.full((16,), float(r), device=d)), (n - 1) / 2, 1e-6)


@case
def gpu_timeline():
    """With the timeline on, GPU collectives of both issue paths leave a DEVICE span next to the host activities."""
    r = bf.rank()
    d = dev()
    x = torch.ones(1 << 16, device=d)
    for i in range(3):
        bf.neighbor_allreduce(x, name="tl.gpu")          # negotiated: background thread + finalizer
    bf.set_skip_negotiate_stage(True)
    for i in range(3):
        bf.neighbor_allreduce(x, name="tl.gpu.fast")     # issued on this thread
    bf.barrier()
    bf.set_skip_negotiate_stage(False)
    bf.shutdown()
    text = open(os.environ["BLUEFOG_TIMELINE"] + str(r) + ".json").read()
    for token in ("ENQUEUE_NEIGHBOR_ALLREDUCE", "COMMUNICATE", "DEVICE", "tl.gpu", "tl.gpu.fast"):
        assert token in text, token
    events = json.loads(text.rstrip().rstrip(",") + "]")
    assert sum(e["ph"] == "B" for e in events) == sum(e["ph"] == "E" for e in events)
    pids = {e["pid"] for e in events if e.get("name") == "DEVICE"}
    assert len(pids) >= 2, "both tensors must carry device spans"


@case
def gpu_wait_timeout():
    """Rank 1 never issues the operation rank 0 is waiting for: rank 0's kernel gives up after
    the wait limit (set to 300 ms by the test) and the operation raises; nothing hangs."""
    r, n, d = bf.rank(), bf.size(), dev()
    x = torch.ones(1024, device=d)
    bf.neighbor_allreduce(x)          # creates the channel while everything still matches
    bf.barrier()
    bf.set_skip_negotiate_stage(True)
    if r == 0:
        try:
            bf.neighbor_allreduce(x, self_weight=0.5, src_weights={1: 0.5}, dst_weights=[1], enable_topo_check=False)
            raise AssertionError("expected the device wait to time out")
        except RuntimeError as exc:
            assert "timed out" in str(exc), str(exc)
    else:
        time.sleep(2.0)
    assert torch.ones(4, device=d).sum().item() == 4.0     # the CUDA context is still usable
    bf.barrier()


def main():
    name = sys.argv[1]
    if name not in ("timeline",):
        pass
    bf.init()
    CASES[name]()
    if bf._b.is_initialized():
        bf.barrier() if name not in ("rank_exits_early",) else None
        bf.shutdown()


if __name__ == "__main__":
    main()
