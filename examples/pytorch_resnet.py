"""ResNet training loop with learning-rate warm-up, periodic checkpoints and resume (role of
the reference's examples/pytorch_resnet.py).  Without a dataset directory it trains on a
synthetic ImageNet-shaped set, which is what an offline machine can do.

  bfrun -np 8 python examples/pytorch_resnet.py --model resnet50 --epochs 2 --bf16
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import math
import os

import torch
import torch.nn.functional as F

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util
from bluefog_b200.models import resnet

parser = argparse.ArgumentParser()
parser.add_argument("--model", default="resnet18")
parser.add_argument("--epochs", type=int, default=2)
parser.add_argument("--batches-per-epoch", type=int, default=20)
parser.add_argument("--batch-size", type=int, default=32)
parser.add_argument("--image-size", type=int, default=64)
parser.add_argument("--num-classes", type=int, default=100)
parser.add_argument("--base-lr", type=float, default=0.0125)
parser.add_argument("--warmup-epochs", type=float, default=1)
parser.add_argument("--momentum", type=float, default=0.9)
parser.add_argument("--wd", type=float, default=5e-5)
parser.add_argument("--dist-optimizer", default="neighbor_allreduce",
                    choices=["neighbor_allreduce", "allreduce", "gradient_allreduce", "atc", "win_put"])
parser.add_argument("--disable-dynamic-topology", action="store_true")
parser.add_argument("--checkpoint-format", default="./checkpoint-{epoch}.pth.tar")
parser.add_argument("--resume-from", default="")
parser.add_argument("--bf16", action="store_true")
parser.add_argument("--no-cuda", action="store_true")
args = parser.parse_args()

torch.backends.cudnn.benchmark = True      # let cuDNN time its algorithms for the fixed shapes
bf.init()
cuda = not args.no_cuda and torch.cuda.is_available() and bf._b.device() >= 0
device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
bf.set_topology(topology_util.ExponentialTwoGraph(bf.size()))
torch.manual_seed(42 + bf.rank())

model = getattr(resnet, args.model)(num_classes=args.num_classes).to(device)
if cuda:
    model = model.to(memory_format=torch.channels_last)
base = torch.optim.SGD(model.parameters(), lr=args.base_lr * bf.size(), momentum=args.momentum, weight_decay=args.wd)
kw = {"compute_dtype": torch.bfloat16} if (args.bf16 and cuda) else {}
CT = bf.CommunicationType
if args.dist_optimizer == "neighbor_allreduce":
    optimizer = bf.DistributedAdaptWithCombineOptimizer(base, model, CT.neighbor_allreduce, **kw)
elif args.dist_optimizer == "allreduce":
    optimizer = bf.DistributedAdaptWithCombineOptimizer(base, model, CT.allreduce, **kw)
elif args.dist_optimizer == "atc":
    optimizer = bf.DistributedAdaptThenCombineOptimizer(base, model, CT.neighbor_allreduce, **kw)
elif args.dist_optimizer == "gradient_allreduce":
    optimizer = bf.DistributedGradientAllreduceOptimizer(base, model, **kw)
else:
    optimizer = bf.DistributedWinPutOptimizer(base, model)

start_epoch = 0
if args.resume_from:
    extra = bf.load_checkpoint(args.resume_from, model, optimizer)
    start_epoch = (extra or {}).get("epoch", -1) + 1
else:
    bf.broadcast_parameters(model.state_dict(), root_rank=0)
    if hasattr(optimizer, "broadcast_from"):
        optimizer.broadcast_from(0)
    else:
        bf.broadcast_optimizer_state(optimizer, root_rank=0)

# a fixed synthetic data set per rank: class-dependent means make it learnable
g = torch.Generator().manual_seed(1000 + bf.rank())
n = args.batch_size * args.batches_per_epoch
labels = torch.randint(0, args.num_classes, (n,), generator=g)
images = torch.randn(n, 3, args.image_size, args.image_size, generator=g) + \
    (labels.float() / args.num_classes - 0.5).view(-1, 1, 1, 1) * 2.0
dynamic = not args.disable_dynamic_topology and bf.size() > 1 and args.dist_optimizer in ("neighbor_allreduce", "atc")
gen = topology_util.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), bf.rank()) if dynamic else None


def adjust_learning_rate(epoch, batch_idx):
    """Linear warm-up from base_lr to base_lr * size, then step decay at epochs 30/60/80."""
    if epoch < args.warmup_epochs:
        e = epoch + float(batch_idx + 1) / args.batches_per_epoch
        adj = 1.0 / bf.size() * (e * (bf.size() - 1) / args.warmup_epochs + 1)
    elif epoch < 30:
        adj = 1.0
    elif epoch < 60:
        adj = 1e-1
    elif epoch < 80:
        adj = 1e-2
    else:
        adj = 1e-3
    for group in optimizer.param_groups:
        group["lr"] = args.base_lr * bf.size() * adj


class Metric:
    """Running average of a scalar, averaged over ranks when read."""
    def __init__(self, name):
        self.name, self.sum, self.n = name, 0.0, 0

    def update(self, v):
        self.sum += float(v)
        self.n += 1

    @property
    def avg(self):
        return bf.allreduce(torch.tensor([self.sum / max(self.n, 1)], dtype=torch.float64), name=self.name).item()


for epoch in range(start_epoch, args.epochs):
    model.train()
    loss_m, acc_m = Metric("train_loss"), Metric("train_accuracy")
    for b in range(args.batches_per_epoch):
        adjust_learning_rate(epoch, b)
        if gen is not None:
            send, recv = next(gen)
            w = 1.0 / (len(recv) + 1)
            optimizer.dst_weights, optimizer.src_weights, optimizer.self_weight = send, {r: w for r in recv}, w
        x = images[b * args.batch_size:(b + 1) * args.batch_size].to(device)
        y = labels[b * args.batch_size:(b + 1) * args.batch_size].to(device)
        optimizer.zero_grad()
        out = model(x).float()
        loss = F.cross_entropy(out, y)
        loss.backward()
        optimizer.step()
        loss_m.update(loss.item())
        acc_m.update((out.argmax(1) == y).float().mean().item())
    la, aa = loss_m.avg, acc_m.avg
    if bf.rank() == 0:
        print(f"epoch {epoch}: loss {la:.4f} accuracy {aa:.3f} lr {optimizer.param_groups[0]['lr']:.4f}", flush=True)
    bf.save_checkpoint(args.checkpoint_format.format(epoch=epoch), model, optimizer, extra={"epoch": epoch})
bf.win_free()
bf.barrier()
