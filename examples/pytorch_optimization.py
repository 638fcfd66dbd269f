"""Decentralized optimization algorithms on a distributed least-squares / logistic problem
(role of the reference's examples/pytorch_optimization.py): diffusion, exact diffusion,
gradient tracking and push-DIGing, all written with the communication primitives only.

  bfrun -np 4 python examples/pytorch_optimization.py --method exact_diffusion
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse

import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util

parser = argparse.ArgumentParser()
parser.add_argument("--method", default="exact_diffusion",
                    choices=["diffusion", "exact_diffusion", "gradient_tracking", "push_diging"])
parser.add_argument("--task", default="linear_regression", choices=["linear_regression", "logistic_regression"])
parser.add_argument("--max-iters", "--max-iter", dest="max_iters", type=int, default=500)
parser.add_argument("--save-plot-file", default="", help="write the curve of rank 0's local gradient norm to this image file")
parser.add_argument("--plot-interactive", action="store_true", help="show the curve with plt.show()")
parser.add_argument("--lr", type=float, default=0.05)
parser.add_argument("--topology", default="mesh", choices=["mesh", "expo2", "ring", "star"])
args = parser.parse_args()


def save_curve(values, path, interactive, ylabel):
    """Semilog plot of ``values`` on rank 0 (the numbers as a .csv when matplotlib is not installed)."""
    if bf.rank() != 0 or not (path or interactive):
        return
    try:
        import matplotlib
        if not interactive:
            matplotlib.use("agg")
        import matplotlib.pyplot as plt
    except ImportError:
        if path:
            csv = os.path.splitext(path)[0] + ".csv"
            with open(csv, "w") as f:
                f.write("iteration,%s\n" % ylabel + "".join("%d,%.6e\n" % (i, v) for i, v in enumerate(values)))
            print("matplotlib is not installed; wrote " + csv)
        return
    plt.semilogy(values)
    plt.xlabel("iteration")
    plt.ylabel(ylabel)
    if path:
        plt.savefig(path)
    if interactive:
        plt.show()

bf.init()
graph = {"mesh": topology_util.MeshGrid2DGraph, "expo2": topology_util.ExponentialTwoGraph,
         "ring": topology_util.RingGraph, "star": topology_util.StarGraph}[args.topology](bf.size())
bf.set_topology(graph, is_weighted=True)

torch.manual_seed(123417 * bf.rank())
m, n = 40, 10
X = torch.randn(m, n, dtype=torch.double)
if args.task == "linear_regression":
    x_o = torch.randn(n, 1, dtype=torch.double)
    y = X @ x_o + 0.1 * torch.randn(m, 1, dtype=torch.double)

    def grad(w):
        return X.t() @ (X @ w - y) / m
else:
    x_o = torch.randn(n, 1, dtype=torch.double)
    y = torch.where(torch.rand(m, 1, dtype=torch.double) < torch.sigmoid(X @ x_o), 1.0, -1.0)
    rho = 1e-2

    def grad(w):
        return -(X * (y * torch.sigmoid(-y * (X @ w)))).mean(0, keepdim=True).t() + rho * w


def global_grad_norm(w):
    return torch.norm(bf.allreduce(grad(w), name="global.grad")).item()


w = torch.zeros(n, 1, dtype=torch.double)
lr = args.lr
curve = []          # |gradient of this rank's own loss| at its iterate, one value per iteration
if args.method == "diffusion":
    for _ in range(args.max_iters):
        w = bf.neighbor_allreduce(w - lr * grad(w), name="w")
        curve.append(torch.norm(grad(w)).item())
elif args.method == "exact_diffusion":
    # psi_k = w_k - lr*g(w_k);  phi_k = psi_k + w_k - psi_{k-1};  w_{k+1} = Abar * phi_k, Abar = (I + W)/2
    sw, nw = topology_util.GetRecvWeights(graph, bf.rank())
    sw, nw = (sw + 1) / 2, {r: v / 2 for r, v in nw.items()}
    psi_prev = w.clone()
    for _ in range(args.max_iters):
        psi = w - lr * grad(w)
        phi = psi + w - psi_prev
        w = bf.neighbor_allreduce(phi, self_weight=sw, src_weights=nw, name="w")
        psi_prev = psi
        curve.append(torch.norm(grad(w)).item())
elif args.method == "gradient_tracking":
    g_prev = grad(w)
    q = g_prev.clone()
    for _ in range(args.max_iters):
        h_w = bf.neighbor_allreduce_nonblocking(w - lr * q, name="w")
        h_q = bf.neighbor_allreduce_nonblocking(q, name="q")
        w = bf.synchronize(h_w)
        g = grad(w)
        q = bf.synchronize(h_q) + g - g_prev
        g_prev = g
        curve.append(torch.norm(g).item())
else:  # push-DIGing over one-sided accumulate: column-stochastic weights, ratio correction
    outdeg = len(bf.out_neighbor_ranks())
    a = 1.0 / (outdeg + 1)
    ext = torch.cat([w, grad(w), torch.ones(1, 1, dtype=torch.double)], 0)   # [u; y; v]
    bf.win_create(ext, name="ext", zero_init=True)
    g_prev = grad(w)
    for _ in range(args.max_iters):
        bf.barrier()
        u, yv = ext[:n], ext[n:2 * n]
        ext[:n] = u - lr * yv
        bf.win_accumulate(ext, name="ext", self_weight=a, dst_weights={r: a for r in bf.out_neighbor_ranks()},
                          require_mutex=True)
        bf.barrier()
        bf.win_update_then_collect(name="ext")
        w = ext[:n] / ext[-1]
        g = grad(w)
        ext[n:2 * n] += g - g_prev
        g_prev = g
        curve.append(torch.norm(g).item())
    bf.barrier()
    bf.win_free("ext")

gn = global_grad_norm(w)
spread = torch.norm(w - bf.allreduce(w, name="w.mean")).item()
print(f"[rank {bf.rank()}] {args.method}: |global gradient| = {gn:.3e}, distance to the mean iterate = {spread:.3e}")
save_curve(curve, args.save_plot_file, args.plot_interactive, "local gradient norm")
bf.barrier()
