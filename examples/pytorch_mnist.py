"""LeNet on MNIST-shaped data with decentralized SGD and a periodic global average every
100 batches (role of the reference's examples/pytorch_mnist.py).  Reads torchvision's MNIST
from --data-dir when it exists there; otherwise a synthetic set of the same shape is used.

  bfrun -np 4 python examples/pytorch_mnist.py --epochs 1 --no-cuda
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import os

import torch
import torch.nn.functional as F

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util
from bluefog_b200.models.lenet import LeNet

parser = argparse.ArgumentParser()
parser.add_argument("--batch-size", type=int, default=64)
parser.add_argument("--epochs", type=int, default=1)
parser.add_argument("--lr", type=float, default=0.01)
parser.add_argument("--momentum", type=float, default=0.5)
parser.add_argument("--data-dir", default="./data")
parser.add_argument("--dist-optimizer", default="neighbor_allreduce",
                    choices=["neighbor_allreduce", "allreduce", "gradient_allreduce", "win_put", "push_sum"])
parser.add_argument("--average-test-result", action="store_true")
parser.add_argument("--test-batch-size", type=int, default=1000, help="rows per forward pass of the evaluation")
parser.add_argument("--seed", type=int, default=42)
parser.add_argument("--log-interval", type=int, default=20, help="batches between two loss lines of rank 0")
parser.add_argument("--atc-style", action="store_true", help="adapt-then-combine for the (neighbor_)allreduce optimizers")
parser.add_argument("--disable-dynamic-topology", action="store_true",
                    help="static exponential-2 neighbors instead of one dynamic peer per step")
parser.add_argument("--no-cuda", action="store_true")
args = parser.parse_args()

bf.init()
cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
torch.manual_seed(args.seed)


def load_data():
    try:
        from torchvision import datasets, transforms
        if os.path.isdir(os.path.join(args.data_dir, "MNIST")):
            ds = datasets.MNIST(args.data_dir, train=True, download=False, transform=transforms.ToTensor())
            x = ds.data.float().div(255).sub(0.1307).div(0.3081).unsqueeze(1)
            return x, ds.targets
    except Exception:
        pass
    g = torch.Generator().manual_seed(7)
    y = torch.randint(0, 10, (6400,), generator=g)
    protos = torch.randn(10, 1, 28, 28, generator=g)
    return protos[y] + 0.5 * torch.randn(6400, 1, 28, 28, generator=g), y


x_all, y_all = load_data()
shard = slice(bf.rank(), None, bf.size())          # every rank trains on its own shard
x_all, y_all = x_all[shard], y_all[shard]
model = LeNet().to(device)
bf.broadcast_parameters(model.state_dict(), root_rank=0)
base = torch.optim.SGD(model.parameters(), lr=args.lr * bf.size(), momentum=args.momentum)
CT = bf.CommunicationType
combine = bf.DistributedAdaptThenCombineOptimizer if args.atc_style else bf.DistributedAdaptWithCombineOptimizer
if args.dist_optimizer == "neighbor_allreduce":
    optimizer = combine(base, model, CT.neighbor_allreduce)
elif args.dist_optimizer == "allreduce":
    optimizer = combine(base, model, CT.allreduce)
elif args.dist_optimizer == "gradient_allreduce":
    optimizer = bf.DistributedGradientAllreduceOptimizer(base, model)
elif args.dist_optimizer == "win_put":
    optimizer = bf.DistributedWinPutOptimizer(base, model)
else:
    optimizer = bf.DistributedPushSumOptimizer(base, model)

dynamic = (not args.disable_dynamic_topology and bf.size() > 1
           and args.dist_optimizer in ("neighbor_allreduce", "win_put", "push_sum"))
peers = bf.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), bf.rank()) if dynamic else None


def pick_dynamic_peer():
    """One out-neighbor per step, walking round the exponential-2 graph."""
    if peers is None:
        return
    send, recv = next(peers)
    if args.dist_optimizer == "neighbor_allreduce":
        w = 1.0 / (len(recv) + 1)
        optimizer.dst_weights, optimizer.src_weights, optimizer.self_weight = send, {r: w for r in recv}, w
    else:
        optimizer.dst_weights = {r: 1.0 for r in send}


batches = len(x_all) // args.batch_size
for epoch in range(args.epochs):
    model.train()
    perm = torch.randperm(len(x_all))
    for b in range(batches):
        idx = perm[b * args.batch_size:(b + 1) * args.batch_size]
        x, y = x_all[idx].to(device), y_all[idx].to(device)
        # every 100 batches one exact global average keeps the ranks from drifting apart
        if args.dist_optimizer == "neighbor_allreduce" and hasattr(optimizer, "communication_type"):
            optimizer.communication_type = CT.allreduce if b % 100 == 99 else CT.neighbor_allreduce
        pick_dynamic_peer()
        optimizer.zero_grad()
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        optimizer.step()
        if b % args.log_interval == 0 and bf.rank() == 0:
            print(f"epoch {epoch} batch {b}/{batches} loss {loss.item():.4f}", flush=True)
    model.eval()
    with torch.no_grad():
        n_eval, hits = min(len(x_all), 1024), 0
        for i in range(0, n_eval, args.test_batch_size):
            j = min(i + args.test_batch_size, n_eval)
            hits += (model(x_all[i:j].to(device)).argmax(1).cpu() == y_all[i:j]).sum().item()
        acc = torch.as_tensor(float(hits) / n_eval)
    acc = bf.allreduce(acc.reshape(1), name="accuracy").item() if args.average_test_result else acc.item()
    if bf.rank() == 0:
        print(f"epoch {epoch}: accuracy on the training shard {acc:.3f}")
bf.win_free()
bf.barrier()
