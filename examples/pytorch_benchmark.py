"""Synthetic training throughput (role of the reference's examples/pytorch_benchmark.py):
10 warm-up batches, then num-iters x num-batches-per-iter timed batches; img/s is reported as
mean +- 1.96 sigma per rank and summed over ranks.

  bfrun -np 8 python examples/pytorch_benchmark.py --model resnet50 --batch-size 64
  bfrun -np 4 python examples/pytorch_benchmark.py --model lenet --dist-optimizer win_put --no-cuda
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import timeit

import numpy as np
import torch
import torch.nn.functional as F

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util
from bluefog_b200.models import lenet, resnet

parser = argparse.ArgumentParser(description="Synthetic benchmark")
parser.add_argument("--model", default="resnet50")
parser.add_argument("--batch-size", type=int, default=64)
parser.add_argument("--num-warmup-batches", type=int, default=10)
parser.add_argument("--num-batches-per-iter", type=int, default=10)
parser.add_argument("--num-iters", type=int, default=10)
parser.add_argument("--num-classes", type=int, default=1000)
parser.add_argument("--no-cuda", action="store_true")
parser.add_argument("--bf16", action="store_true", help="bf16 compute with fp32 master weights (fused path)")
parser.add_argument("--dist-optimizer", default="neighbor_allreduce",
                    help="neighbor_allreduce, allreduce, gradient_allreduce, hierarchical_neighbor_allreduce, "
                         "win_put, pull_get, push_sum, atc, empty")
parser.add_argument("--disable-dynamic-topology", action="store_true")
parser.add_argument("--atc-style", action="store_true",
                    help="adapt-then-combine instead of adapt-with-combine for the (hierarchical_)neighbor_allreduce / allreduce optimizers")
parser.add_argument("--profiler", action="store_true", help="torch.autograd.profiler around the timed iterations on rank 0")
parser.add_argument("--partition", type=int, default=None, help="accepted for compatibility with the reference's script; unused there too")
parser.add_argument("--virtual-topology", default="expo2")
args = parser.parse_args()

torch.backends.cudnn.benchmark = True      # let cuDNN time its algorithms for the fixed shapes
bf.init()
cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
if args.virtual_topology == "ring":
    bf.set_topology(topology_util.RingGraph(bf.size()))
else:
    bf.set_topology(topology_util.ExponentialTwoGraph(bf.size()))

if args.model == "lenet":
    model, shape, classes = lenet.LeNet(), (args.batch_size, 1, 28, 28), 10
else:
    model, shape, classes = getattr(resnet, args.model)(num_classes=args.num_classes), \
        (args.batch_size, 3, 224, 224), args.num_classes
model = model.to(device)
if cuda and args.model != "lenet":
    model = model.to(memory_format=torch.channels_last)
bf.broadcast_parameters(model.state_dict(), root_rank=0)
base = torch.optim.SGD(model.parameters(), lr=0.01)
kw = {"compute_dtype": torch.bfloat16} if (args.bf16 and cuda) else {}
CT = bf.CommunicationType
name = args.dist_optimizer
combine = bf.DistributedAdaptThenCombineOptimizer if args.atc_style else bf.DistributedAdaptWithCombineOptimizer
if name == "neighbor_allreduce":
    optimizer = combine(base, model, CT.neighbor_allreduce, **kw)
elif name == "allreduce":
    optimizer = combine(base, model, CT.allreduce, **kw)
elif name == "empty":
    optimizer = combine(base, model, CT.empty, **kw)
elif name == "atc":
    optimizer = bf.DistributedAdaptThenCombineOptimizer(base, model, CT.neighbor_allreduce, **kw)
elif name == "gradient_allreduce":
    optimizer = bf.DistributedGradientAllreduceOptimizer(base, model, **kw)
elif name == "hierarchical_neighbor_allreduce":
    optimizer = bf.DistributedHierarchicalNeighborAllreduceOptimizer(base, model)
    bf.set_machine_topology(topology_util.ExponentialTwoGraph(bf.machine_size()))
elif name == "win_put":
    optimizer = bf.DistributedWinPutOptimizer(base, model)
elif name == "pull_get":
    optimizer = bf.DistributedPullGetOptimizer(base, model)
elif name == "push_sum":
    optimizer = bf.DistributedPushSumOptimizer(base, model)
else:
    raise ValueError("unknown --dist-optimizer " + name)

data = torch.rand(*shape, device=device)
target = torch.randint(0, classes, (args.batch_size,), device=device)
dynamic = not args.disable_dynamic_topology and bf.size() > 1 and name in ("neighbor_allreduce", "atc", "win_put")
gen = topology_util.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), bf.rank()) if dynamic else None


def set_dynamic_weights():
    if gen is None:
        return
    send, recv = next(gen)
    if name == "win_put":
        optimizer.dst_weights = {r: 1.0 for r in send}
        return
    w = 1.0 / (len(recv) + 1)
    optimizer.dst_weights = send
    optimizer.src_weights = {r: w for r in recv}
    optimizer.self_weight = w


def benchmark_step():
    set_dynamic_weights()
    optimizer.zero_grad()
    loss = F.cross_entropy(model(data).float(), target)
    loss.backward()
    optimizer.step()
    if cuda:
        torch.cuda.synchronize()


def log(msg):
    if bf.rank() == 0:
        print(msg, flush=True)


log(f"Model: {args.model}  batch size: {args.batch_size}  ranks: {bf.size()}  optimizer: {name}")
timeit.timeit(benchmark_step, number=args.num_warmup_batches)
rates = []
profiling = args.profiler and bf.rank() == 0
with torch.autograd.profiler.profile(enabled=profiling, use_device="cuda" if cuda else None) as prof:
    for i in range(args.num_iters):
        t = timeit.timeit(benchmark_step, number=args.num_batches_per_iter)
        rates.append(args.batch_size * args.num_batches_per_iter / t)
        log(f"Iter #{i}: {rates[-1]:.1f} img/sec per rank")
if profiling:
    print(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=25), flush=True)
mean, conf = float(np.mean(rates)), float(1.96 * np.std(rates))
log(f"Img/sec per rank: {mean:.1f} +-{conf:.1f}")
total = bf.allreduce(torch.tensor([mean, conf], dtype=torch.float64), average=False)
log(f"Total img/sec on {bf.size()} rank(s): {total[0].item():.1f} +-{total[1].item():.1f}")
bf.win_free()
bf.barrier()
