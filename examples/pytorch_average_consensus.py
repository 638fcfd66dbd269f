"""Average consensus: every rank starts from its own random vector and repeatedly averages
with its neighbors until all ranks hold the global mean (role of the reference's
examples/pytorch_average_consensus.py).

  bfrun -np 4 python examples/pytorch_average_consensus.py
  bfrun -np 4 python examples/pytorch_average_consensus.py --enable-dynamic-topology
  bfrun -np 4 python examples/pytorch_average_consensus.py --asynchronous-mode
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse

import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util

parser = argparse.ArgumentParser(description="Average consensus example")
parser.add_argument("--data-size", type=int, default=100000)
parser.add_argument("--max-iters", type=int, default=200)
parser.add_argument("--virtual-topology", default="expo2", help="expo2, ring, mesh, star")
parser.add_argument("--asynchronous-mode", action="store_true", help="push-sum over one-sided windows")
parser.add_argument("--enable-dynamic-topology", action="store_true")
parser.add_argument("--no-cuda", action="store_true")
parser.add_argument("--seed", type=int, default=2020)
parser.add_argument("--save-plot-file", default="", help="write the error curve of rank 0 to this image file")
parser.add_argument("--plot-interactive", action="store_true", help="show the curve with plt.show()")
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
cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
graphs = {"expo2": topology_util.ExponentialTwoGraph, "ring": topology_util.RingGraph,
          "mesh": topology_util.MeshGrid2DGraph, "star": topology_util.StarGraph}
bf.set_topology(graphs[args.virtual_topology](bf.size()))

torch.manual_seed(args.seed * bf.rank())
x = torch.randn(args.data_size, dtype=torch.double, device=device)
x_bar = bf.allreduce(x, average=True)
mse = []

if not args.asynchronous_mode:
    gen = topology_util.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), bf.rank()) \
        if args.enable_dynamic_topology else None
    for it in range(args.max_iters):
        if gen is not None:
            send, recv = next(gen)
            w = 1.0 / (len(recv) + 1)
            x = bf.neighbor_allreduce(x, name="x", self_weight=w, src_weights={r: w for r in recv},
                                      dst_weights=send, enable_topo_check=False)
        else:
            x = bf.neighbor_allreduce(x, name="x")
        mse.append(torch.norm(x - x_bar, p=2).item() / torch.norm(x_bar, p=2).item())
else:
    # push-sum: the vector carries a scalar weight; sums are preserved, the ratio converges
    outdeg = len(bf.out_neighbor_ranks())
    ext = torch.cat([x, torch.ones(1, dtype=x.dtype, device=device)])
    bf.turn_on_win_ops_with_associated_p()
    bf.win_create(ext, name="x_ext", zero_init=True)
    for it in range(args.max_iters):
        bf.win_accumulate(ext, name="x_ext", self_weight=1.0 / (outdeg + 1),
                          dst_weights={r: 1.0 / (outdeg + 1) for r in bf.out_neighbor_ranks()},
                          require_mutex=True)
        bf.win_update_then_collect(name="x_ext")
        x = ext[:-1] / ext[-1]
        mse.append(torch.norm(x - x_bar, p=2).item() / torch.norm(x_bar, p=2).item())
    bf.barrier()
    bf.win_update_then_collect(name="x_ext")
    x = ext[:-1] / ext[-1]
    p_mean = bf.allreduce(torch.tensor([bf.win_associated_p("x_ext")], dtype=torch.double)).item()
    if bf.rank() == 0:
        print(f"mean of the push-sum weights over ranks (should be 1): {p_mean:.6f}")
    bf.win_free("x_ext")

err = torch.norm(x - x_bar, p=2).item() / torch.norm(x_bar, p=2).item()
print(f"[rank {bf.rank()}] relative error after {args.max_iters} iterations: {err:.3e}")
if bf.rank() == 0:
    print("relative MSE every 20 iterations:", ["%.2e" % m for m in mse[::20]])
save_curve(mse, args.save_plot_file, args.plot_interactive, "relative error")
bf.barrier()
