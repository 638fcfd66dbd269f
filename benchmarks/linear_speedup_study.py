"""How close to linear speed-up does a decentralized first-order method get?  Gradient tracking on a
regularised logistic regression, every rank holding its own synthetic shard, timed in three modes whose
difference separates compute from communication (the study of scripts/pytorch_opt_linear_speedup_test.py in
the reference):

  normal                   two neighbor_allreduce calls per iteration overlapped with the local gradient
  compute-only             the same arithmetic with no communication at all (the per-rank compute ceiling)
  sleep-and-communicate    the two neighbor_allreduce calls around a fixed sleep instead of the gradient

  bfrun -np 4 python benchmarks/linear_speedup_study.py --mode normal --no-cuda
  bfrun -np 4 python benchmarks/linear_speedup_study.py --mode normal --profile      # cProfile of rank 0

Rank 0 prints one JSON line: samples/s per rank (mean and 95 % interval over the timed rounds) and the
job total.  Run it at 1, 2, 4, ... ranks and divide.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import cProfile
import io
import json
import pstats
import time

import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util

MODES = ("normal", "compute-only", "sleep-and-communicate")


def make_topology(name, size):
    if name == "expo2":
        return topology_util.ExponentialTwoGraph(size)
    if name == "ring":
        return topology_util.RingGraph(size, connect_style=0)
    if name == "mesh":
        return topology_util.MeshGrid2DGraph(size)
    if name == "star":
        return topology_util.StarGraph(size)
    raise ValueError("--topology must be one of expo2, ring, mesh, star")


class GradientTracking:
    """w <- A w - lr q;  q <- A q + grad(w_new) - grad(w_old), A = the topology's averaging matrix."""

    def __init__(self, features, labels, rho, lr, by_hand):
        self.X, self.y, self.rho, self.lr, self.by_hand = features, labels, rho, lr, by_hand
        self.w = torch.zeros(features.shape[1], 1, dtype=features.dtype, device=features.device)
        self.prev_grad = self.gradient(self.w)
        self.q = self.prev_grad.clone()

    def gradient(self, w):
        if self.by_hand:
            margin = torch.exp(-self.y * (self.X @ w))
            return self.rho * w - ((margin / (1 + margin)) * self.y * self.X).mean(0).reshape(-1, 1)
        v = w.clone().requires_grad_(True)
        loss = torch.log1p(torch.exp(-self.y * (self.X @ v))).mean() + 0.5 * self.rho * (v * v).sum()
        return torch.autograd.grad(loss, v)[0]

    def step(self, mode, sleep_seconds):
        if mode == "normal":
            hw = bf.neighbor_allreduce_nonblocking(self.w, name="tracking.w")
            self.w = bf.synchronize(hw) - self.lr * self.q
            hq = bf.neighbor_allreduce_nonblocking(self.q, name="tracking.q")
            grad = self.gradient(self.w)                       # overlaps the exchange of q
            self.q = bf.synchronize(hq) + grad - self.prev_grad
            self.prev_grad = grad
        elif mode == "compute-only":
            self.w = self.w - self.lr * self.q
            grad = self.gradient(self.w)
            self.q = self.q + grad - self.prev_grad
            self.prev_grad = grad
        else:
            hw = bf.neighbor_allreduce_nonblocking(self.w, name="tracking.w")
            hq = bf.neighbor_allreduce_nonblocking(self.q, name="tracking.q")
            self.w = bf.synchronize(hw)
            time.sleep(sleep_seconds)
            self.q = bf.synchronize(hq)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", default="normal", choices=MODES)
    ap.add_argument("--topology", default="expo2")
    ap.add_argument("--samples", type=int, default=2000, help="rows of every rank's shard")
    ap.add_argument("--dim", type=int, default=500)
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--sleep-seconds", type=float, default=0.1)
    ap.add_argument("--warmup-steps", type=int, default=10)
    ap.add_argument("--steps-per-round", type=int, default=10)
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--autograd", action="store_true", help="gradient by autograd instead of the closed form")
    ap.add_argument("--no-cuda", action="store_true")
    ap.add_argument("--profile", action="store_true", help="cProfile the timed rounds on rank 0 and print the top 25")
    args = ap.parse_args()

    bf.init()
    rank, size = bf.rank(), bf.size()
    cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if size > 1:
        bf.set_topology(make_topology(args.topology, size))

    g = torch.Generator().manual_seed(123417 * (rank + 1))
    X = torch.randn(args.samples, args.dim, generator=g, dtype=torch.float64)
    w_true = torch.randn(args.dim, 1, generator=g, dtype=torch.float64)
    y = (torch.rand(args.samples, 1, generator=g, dtype=torch.float64) < torch.sigmoid(-(X @ w_true))).double() * 2 - 1
    solver = GradientTracking(X.to(dev), y.to(dev), rho=1e-2, lr=args.lr, by_hand=not args.autograd)

    def run(steps):
        t0 = time.perf_counter()
        for _ in range(steps):
            solver.step(args.mode, args.sleep_seconds)
        if cuda:
            torch.cuda.synchronize()
        return time.perf_counter() - t0

    run(args.warmup_steps)
    profiler = cProfile.Profile() if args.profile and rank == 0 else None
    if profiler is not None:
        profiler.enable()
    rates = torch.tensor([args.samples * args.steps_per_round / run(args.steps_per_round) for _ in range(args.rounds)],
                         dtype=torch.float64)
    if profiler is not None:
        profiler.disable()
    total = bf.allreduce(rates.clone(), average=False, name="rates") if size > 1 else rates

    def mean_ci(t):
        return round(t.mean().item(), 1), round(1.96 * t.std(unbiased=False).item(), 1)

    if rank == 0:
        per_rank, job = mean_ci(rates), mean_ci(total)
        print(json.dumps({"metric": "gradient tracking, logistic regression: samples/s", "mode": args.mode,
                          "n_ranks": size, "device": dev.type, "topology": args.topology,
                          "shard": [args.samples, args.dim], "per_rank": per_rank[0], "per_rank_ci95": per_rank[1],
                          "job_total": job[0], "job_total_ci95": job[1],
                          "grad_norm": round(solver.prev_grad.norm().item(), 6)}), flush=True)
        if profiler is not None:
            out = io.StringIO()
            pstats.Stats(profiler, stream=out).sort_stats("cumulative").print_stats(25)
            print(out.getvalue())
    bf.barrier()
    bf.shutdown()


if __name__ == "__main__":
    main()
