"""Optimal exchange (resource allocation) over a network:  min sum_i f_i(x_i)  s.t.  sum_i x_i = 0,
with f_i(x) = 1/2 |A_i x - b_i|^2 held by rank i only.

The reference teaches this problem in a notebook (examples/resource_allocation.ipynb); here it is a script:

  bfrun -np 8 python examples/resource_allocation.py --no-cuda [--plot exchange.png]

1. A reference solution x* comes from consensus ADMM, whose only communication is a global average
   (``bf.allreduce``); its KKT residuals  |A_i^T(A_i x_i - b_i) + y|  and  |mean_i x_i|  are printed.
2. The dual problem  min_y sum_i F_i(y),  F_i(y) = f_i^*(-y),  is a consensus problem with the local gradient
   grad F_i(y) = -(A_i^T A_i)^{-1} (A_i^T b_i - y) = -x_i(y).  Three decentralized methods solve it with
   ``bf.neighbor_allreduce`` only, and each reports  sqrt(mean_i |x_i - x_i*|^2 / |x_i*|^2):
     EXTRA            explicit halved weights  (W + I)/2  passed as self_weight / src_weights
     exact diffusion  the same matrix installed as a weighted topology (``set_topology(..., is_weighted=True)``)
     gradient tracking  the plain exponential-2 topology and its default uniform weights
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse

import networkx as nx
import numpy as np
import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util


class LocalCost:
    """f_i(x) = 1/2 |A x - b|^2 of this rank, with the pieces every method needs."""

    def __init__(self, rows, dim, seed, device):
        g = torch.Generator().manual_seed(seed)
        self.A = torch.rand(rows, dim, generator=g, dtype=torch.float64).to(device)
        self.b = torch.rand(rows, 1, generator=g, dtype=torch.float64).to(device)
        self.gram = self.A.t() @ self.A
        self.gram_inv = torch.linalg.inv(self.gram)
        self.Atb = self.A.t() @ self.b
        self.dim = dim

    def primal_from_dual(self, y):
        """argmin_x f_i(x) + y^T x."""
        return self.gram_inv @ (self.Atb - y)

    def dual_gradient(self, y):
        return -self.primal_from_dual(y)

    def stationarity(self, x, y):
        return torch.linalg.norm(self.gram @ x - self.Atb + y).item()


def consensus_admm(cost, rho, iterations):
    d, dev = cost.dim, cost.A.device
    x = torch.zeros(d, 1, dtype=torch.float64, device=dev)
    x_bar, u = x.clone(), x.clone()
    solve = torch.linalg.inv(rho * torch.eye(d, dtype=torch.float64, device=dev) + cost.gram)
    for _ in range(iterations):
        x = solve @ (cost.Atb + rho * (x - x_bar - u))
        x_bar = bf.allreduce(x, average=True, name="admm.xbar")
        u = u + x_bar
    return x, x_bar, rho * u


def relative_error(x, x_star):
    mine = (torch.linalg.norm(x - x_star) / torch.linalg.norm(x_star)) ** 2
    return bf.allreduce(mine.reshape(1), average=True, name="err").sqrt().item()


def extra(cost, x_star, lr, iterations, self_weight, src_weights):
    """y+ = Wbar (2 y - y-) - lr (g - g-)."""
    y = torch.zeros_like(x_star)
    y_prev, g_prev, errors = y.clone(), y.clone(), []
    for _ in range(iterations):
        x = cost.primal_from_dual(y)
        g = -x
        mixed = bf.neighbor_allreduce(2 * y - y_prev, self_weight=self_weight, src_weights=src_weights, name="extra.y")
        y_prev, y, g_prev = y, mixed - lr * (g - g_prev), g
        errors.append(relative_error(x, x_star))
    return errors


def exact_diffusion(cost, x_star, lr, iterations):
    """y+ = Wbar (2 y - y- - lr (g - g-)); Wbar is the installed weighted topology."""
    y = torch.zeros_like(x_star)
    y_prev, g_prev, errors = y.clone(), y.clone(), []
    for _ in range(iterations):
        x = cost.primal_from_dual(y)
        g = -x
        mixed = bf.neighbor_allreduce(2 * y - y_prev - lr * (g - g_prev), name="ed.y")
        y_prev, y, g_prev = y, mixed, g
        errors.append(relative_error(x, x_star))
    return errors


def gradient_tracking(cost, x_star, lr, iterations):
    """y+ = W (y - lr z);  z+ = W (z + g(y+) - g(y)),  z0 = g(y0)."""
    y = torch.zeros_like(x_star)
    g_prev = cost.dual_gradient(y)
    z, errors = g_prev.clone(), []
    for _ in range(iterations):
        y = bf.neighbor_allreduce(y - lr * z, name="gt.y")
        x = cost.primal_from_dual(y)
        g = -x
        z = bf.neighbor_allreduce(z + g - g_prev, name="gt.z")
        g_prev = g
        errors.append(relative_error(x, x_star))
    return errors


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=10)
    ap.add_argument("--dim", type=int, default=5)
    ap.add_argument("--seed", type=int, default=2021)
    ap.add_argument("--admm-iterations", type=int, default=500)
    ap.add_argument("--iterations", type=int, default=2000)
    ap.add_argument("--no-cuda", action="store_true")
    ap.add_argument("--plot", default="", help="write the three error curves to this PNG (a .csv without matplotlib)")
    args = ap.parse_args()

    bf.init()
    rank, size = bf.rank(), bf.size()
    cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    cost = LocalCost(args.rows, args.dim, args.seed * (rank + 1), dev)

    def say(msg):
        if rank == 0:
            print(msg, flush=True)

    x_star, x_bar, y_star = consensus_admm(cost, rho=1.0, iterations=args.admm_iterations)
    say("ADMM: stationarity %.2e, |mean x| %.2e" % (cost.stationarity(x_star, y_star), torch.linalg.norm(x_bar).item()))

    curves = {}
    # EXTRA on the exponential-2 graph with explicitly halved weights
    graph = topology_util.ExponentialTwoGraph(size)
    bf.set_topology(graph)
    self_w, src_w = topology_util.GetRecvWeights(bf.load_topology(), rank)
    curves["EXTRA"] = extra(cost, x_star, 0.06, args.iterations, (1 + self_w) / 2, {r: w / 2 for r, w in src_w.items()})

    # exact diffusion with (W + I)/2 installed as the topology's own weights
    w_bar = (nx.to_numpy_array(topology_util.ExponentialGraph(size)) + np.eye(size)) / 2
    bf.set_topology(nx.from_numpy_array(w_bar, create_using=nx.DiGraph), is_weighted=True)
    curves["exact diffusion"] = exact_diffusion(cost, x_star, 0.08, args.iterations)

    # gradient tracking with the default uniform weights of the exponential-2 graph
    bf.set_topology(graph)
    curves["gradient tracking"] = gradient_tracking(cost, x_star, 0.1, args.iterations)

    for name, err in curves.items():
        say("%-18s relative error %.2e after %d iterations (%.2e after 100)" % (name, err[-1], len(err), err[min(99, len(err) - 1)]))
    if args.plot and rank == 0:
        try:
            import matplotlib
            matplotlib.use("agg")
            import matplotlib.pyplot as plt
        except ImportError:                      # no matplotlib: keep the numbers
            path = os.path.splitext(args.plot)[0] + ".csv"
            np.savetxt(path, np.array(list(curves.values())).T, delimiter=",", header=",".join(curves), comments="")
            say("matplotlib is not installed; wrote the curves to " + path)
        else:
            for name, err in curves.items():
                plt.semilogy(err, label=name)
            plt.xlabel("iteration")
            plt.ylabel("relative error")
            plt.legend()
            plt.savefig(args.plot)
    bf.barrier()
    bf.shutdown()


if __name__ == "__main__":
    main()
