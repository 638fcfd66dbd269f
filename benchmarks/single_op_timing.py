"""Time of one communication operation on CPU or GPU ranks (the measurement of scripts/single_ops_test.py in the
reference: a fixed vector, the same operation repeated, wall time per call).

  bfrun -np 4 python benchmarks/single_op_timing.py --no-cuda                      # 100 000 floats, neighbor_allreduce
  bfrun -np 8 python benchmarks/single_op_timing.py --op win_put --numel 1048576

Each round issues ``--ops-per-round`` operations (blocking, or all nonblocking and then waited for with
``--nonblocking``) and is timed with the host clock after a device synchronisation; rank 0 prints one JSON line
with the microseconds per operation (mean and 95 % interval over the rounds, max over ranks) and the payload
rate it corresponds to.  The device-timed sweep over sizes is benchmarks/neighbor_allreduce_bandwidth.py.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import json
import time

import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util

TOPOLOGIES = {
    "expo2": topology_util.ExponentialTwoGraph,
    "expo4": lambda n: topology_util.ExponentialGraph(n, base=4),
    "ring": lambda n: topology_util.RingGraph(n, connect_style=0),
    "mesh": topology_util.MeshGrid2DGraph,
    "star": topology_util.StarGraph,
    "full": topology_util.FullyConnectedGraph,
}
OPS = ("neighbor_allreduce", "allreduce", "broadcast", "neighbor_allgather", "win_put", "win_accumulate")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="neighbor_allreduce", choices=OPS)
    ap.add_argument("--numel", type=int, default=100000)
    ap.add_argument("--dtype", default="float32", choices=["float32", "float64", "bfloat16", "float16"])
    ap.add_argument("--virtual-topology", default="expo2", choices=sorted(TOPOLOGIES))
    ap.add_argument("--ops-per-round", type=int, default=10)
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--warmup-rounds", type=int, default=3)
    ap.add_argument("--nonblocking", action="store_true")
    ap.add_argument("--skip-negotiate", action="store_true", help="the steady-state issue path (no cross-rank argument check)")
    ap.add_argument("--no-cuda", action="store_true")
    args = ap.parse_args()

    bf.init()
    rank, size = bf.rank(), bf.size()
    cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if size > 1:
        bf.set_topology(TOPOLOGIES[args.virtual_topology](size))
    if args.skip_negotiate:
        bf.set_skip_negotiate_stage(True)
    x = torch.randn(args.numel, generator=torch.Generator().manual_seed(rank)).to(dev).to(getattr(torch, args.dtype))
    window = args.op.startswith("win_")
    if window:
        bf.win_create(x.clone(), "timing.win", zero_init=True)

    def issue(k):
        name = "%s.%d" % (args.op, k)
        if args.op == "neighbor_allreduce":
            return bf.neighbor_allreduce_nonblocking(x, name=name)
        if args.op == "allreduce":
            return bf.allreduce_nonblocking(x, name=name)
        if args.op == "broadcast":
            return bf.broadcast_nonblocking(x, root_rank=0, name=name)
        if args.op == "neighbor_allgather":
            return bf.neighbor_allgather_nonblocking(x, name=name)
        if args.op == "win_put":
            return bf.win_put_nonblocking(x, "timing.win")
        return bf.win_accumulate_nonblocking(x, "timing.win")

    def finish(handle):
        return bf.win_wait(handle) if window else bf.synchronize(handle)

    def one_round():
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        if args.nonblocking:
            for h in [issue(k) for k in range(args.ops_per_round)]:
                finish(h)
        else:
            for k in range(args.ops_per_round):
                finish(issue(k))
        if cuda:
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) / args.ops_per_round * 1e6

    for _ in range(args.warmup_rounds):
        one_round()
    bf.barrier()
    mine = torch.tensor([one_round() for _ in range(args.rounds)], dtype=torch.float64)
    worst = bf.allgather(mine.reshape(1, -1), name="timing.rounds").max(0).values if size > 1 else mine
    if rank == 0:
        us = worst.mean().item()
        nbytes = x.numel() * x.element_size()
        print(json.dumps({"op": args.op, "n_ranks": size, "device": dev.type, "topology": args.virtual_topology,
                          "dtype": args.dtype, "bytes": nbytes, "nonblocking": args.nonblocking,
                          "skip_negotiate": args.skip_negotiate, "us_per_op": round(us, 1),
                          "us_per_op_ci95": round(1.96 * worst.std(unbiased=False).item(), 1),
                          "payload_gbs": round(nbytes / us / 1e3, 3)}), flush=True)
    if window:
        bf.win_free("timing.win")
    bf.barrier()
    bf.shutdown()


if __name__ == "__main__":
    main()
