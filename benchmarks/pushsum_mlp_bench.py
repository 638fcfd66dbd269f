"""Asynchronous one-sided training: MLP regression with DistributedWinPutOptimizer.

Config: 4 layers of 4096 hidden units, ReLU; batch 256 per GPU with x ~ N(0,1) of dim 4096 and
y = x . w* + 0.01 noise (w* ~ N(0, 1/dim) from seed 0); static ExponentialTwoGraph; win_put + win_update with
associated push-sum weights switched on; ranks run deliberately skewed numbers of steps per
second (rank r sleeps r/(size-1) of a step time) to exercise the one-sided path, since no
rank ever waits for another one.

  bfrun -np 8 python benchmarks/pushsum_mlp_bench.py --seconds 10
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import json
import time

import torch

import bluefog_b200.torch as bf
from bluefog_b200.models.mlp import MLP


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=10.0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--bucket-bytes", type=int, default=None,
                    help="parameters per window; 0 = one window per parameter (the reference's layout), default 64 MiB")
    args = ap.parse_args()
    bf.init()
    rank, size = bf.rank(), bf.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    bf.set_topology(bf.ExponentialTwoGraph(size))
    bf.turn_on_win_ops_with_associated_p()
    # w* ~ N(0, 1/dim): targets of unit variance keep plain SGD stable in bf16
    w_star = (torch.randn(args.dim, 1, generator=torch.Generator().manual_seed(0)) / args.dim ** 0.5).to(dev)
    torch.manual_seed(1)
    model = MLP(args.dim, args.dim, 1, 4, use_b200_gemm=True).to(dev).to(torch.bfloat16)
    bf.broadcast_parameters(model.state_dict(), root_rank=0)
    opt = bf.DistributedWinPutOptimizer(torch.optim.SGD(model.parameters(), lr=1e-3), model,
                                        bucket_bytes=args.bucket_bytes)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    skew = rank / max(size - 1, 1)          # 0 .. 1 extra step time: 1x .. 2x step duration
    steps, t_step = 0, 0.0
    bf.barrier()
    t_start = time.time()
    while time.time() - t_start < args.seconds:
        t0 = time.time()
        x = torch.randn(args.batch, args.dim, device=dev, generator=g)
        y = x @ w_star + 0.01 * torch.randn(args.batch, 1, device=dev, generator=g)
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x.to(torch.bfloat16)).float(), y)
        loss.backward()
        opt.step()
        torch.cuda.synchronize()
        t_step = time.time() - t0
        time.sleep(skew * t_step)
        steps += 1
    elapsed = time.time() - t_start
    bf.barrier()
    # ranks ran different numbers of operations, so unnamed ops would carry different handle numbers
    counts = bf.allgather(torch.tensor([float(steps)], dtype=torch.float64), name="pushsum.counts").tolist()
    losses = bf.allgather(torch.tensor([loss.item()], dtype=torch.float64), name="pushsum.losses").tolist()
    if rank == 0:
        print(json.dumps({"metric": "push-sum MLP steps/s (sum over ranks)", "value": round(sum(counts) / elapsed, 2),
                          "unit": "steps/s", "n_gpus": size, "steps_per_rank": counts, "final_losses": losses,
                          "windows": len(bf.get_current_created_window_names()),
                          "seconds": elapsed}), flush=True)
    opt.unregister_window()
    bf.barrier()
    bf.shutdown()


if __name__ == "__main__":
    main()
