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
parser.add_argument("--atc-style", action="store_true", help="adapt-then-combine for the (neighbor_)allreduce optimizers")
parser.add_argument("--dataset", default="synthetic", choices=["synthetic", "cifar10", "imagenet"],
                    help="cifar10 / imagenet are read from --train-dir / --val-dir with torchvision (nothing is downloaded)")
parser.add_argument("--train-dir", default=os.path.expanduser("~/imagenet/train"))
parser.add_argument("--val-dir", default=os.path.expanduser("~/imagenet/validation"))
parser.add_argument("--val-batch-size", type=int, default=32)
parser.add_argument("--batches-per-allreduce", type=int, default=1,
                    help="sub-batches whose gradients are accumulated before one optimizer (and communication) step; "
                         "the learning rate is scaled by it")
parser.add_argument("--log-dir", default="", help="TensorBoard scalars of rank 0 (a metrics.jsonl there without tensorboard)")
parser.add_argument("--seed", type=int, default=42)
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
torch.manual_seed(args.seed + bf.rank())

model = getattr(resnet, args.model)(num_classes=args.num_classes).to(device)
if cuda:
    model = model.to(memory_format=torch.channels_last)
lr_scale = bf.size() * args.batches_per_allreduce
base = torch.optim.SGD(model.parameters(), lr=args.base_lr * lr_scale, momentum=args.momentum, weight_decay=args.wd)
kw = {"compute_dtype": torch.bfloat16} if (args.bf16 and cuda) else {}
CT = bf.CommunicationType
combine = bf.DistributedAdaptThenCombineOptimizer if args.atc_style else bf.DistributedAdaptWithCombineOptimizer
if args.dist_optimizer == "neighbor_allreduce":
    optimizer = combine(base, model, CT.neighbor_allreduce, **kw)
elif args.dist_optimizer == "allreduce":
    optimizer = combine(base, model, CT.allreduce, **kw)
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



def synthetic_split(count, seed):
    """Class-dependent means make the random images learnable."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, args.num_classes, (count,), generator=g)
    x = torch.randn(count, 3, args.image_size, args.image_size, generator=g) + \
        (y.float() / args.num_classes - 0.5).view(-1, 1, 1, 1) * 2.0
    return torch.utils.data.TensorDataset(x, y)


def disk_split(train):
    """CIFAR-10 or an ImageNet-style folder tree read with torchvision; every rank takes its own shard."""
    from torchvision import datasets, transforms
    if args.dataset == "cifar10":
        norm = transforms.Normalize((0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616))
        aug = [transforms.RandomCrop(32, padding=4), transforms.RandomHorizontalFlip()] if train else []
        ds = datasets.CIFAR10(args.train_dir if train else args.val_dir, train=train, download=False,
                              transform=transforms.Compose(aug + [transforms.ToTensor(), norm]))
    else:
        norm = transforms.Normalize((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
        tf = [transforms.RandomResizedCrop(224), transforms.RandomHorizontalFlip()] if train else \
            [transforms.Resize(256), transforms.CenterCrop(224)]
        ds = datasets.ImageFolder(args.train_dir if train else args.val_dir,
                                  transform=transforms.Compose(tf + [transforms.ToTensor(), norm]))
    return torch.utils.data.Subset(ds, range(bf.rank(), len(ds), bf.size()))


if args.dataset == "synthetic":
    train_set = synthetic_split(args.batch_size * args.batches_per_allreduce * args.batches_per_epoch, 1000 + bf.rank())
    val_set = synthetic_split(args.val_batch_size * 4, 5000 + bf.rank())
else:
    train_set, val_set = disk_split(True), disk_split(False)
train_loader = torch.utils.data.DataLoader(train_set, batch_size=args.batch_size * args.batches_per_allreduce,
                                           shuffle=args.dataset != "synthetic", drop_last=True)
val_loader = torch.utils.data.DataLoader(val_set, batch_size=args.val_batch_size)
steps_per_epoch = min(len(train_loader), args.batches_per_epoch) if args.dataset == "synthetic" else len(train_loader)


class ScalarLog:
    """TensorBoard on rank 0 when --log-dir is given (a JSON-lines file if tensorboard is not installed)."""
    def __init__(self, path):
        self.tb = self.fh = None
        if not path or bf.rank() != 0:
            return
        os.makedirs(path, exist_ok=True)
        try:
            from torch.utils.tensorboard import SummaryWriter
            self.tb = SummaryWriter(path)
        except ImportError:
            self.fh = open(os.path.join(path, "metrics.jsonl"), "a")

    def add(self, tag, value, step):
        if self.tb is not None:
            self.tb.add_scalar(tag, value, step)
        elif self.fh is not None:
            self.fh.write('{"tag": "%s", "value": %r, "step": %d}\n' % (tag, float(value), step))
            self.fh.flush()


scalars = ScalarLog(args.log_dir)
dynamic = not args.disable_dynamic_topology and bf.size() > 1 and args.dist_optimizer in ("neighbor_allreduce", "atc")
gen = topology_util.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), bf.rank()) if dynamic else None


def adjust_learning_rate(epoch, batch_idx):
    """Linear warm-up from base_lr to base_lr * size, then step decay at epochs 30/60/80."""
    if epoch < args.warmup_epochs:
        e = epoch + float(batch_idx + 1) / steps_per_epoch
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
        group["lr"] = args.base_lr * lr_scale * adj


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


def accuracy(out, y):
    return (out.argmax(1) == y).float().mean().item()


def validate(epoch):
    model.eval()
    loss_m, acc_m = Metric("val_loss"), Metric("val_accuracy")
    with torch.no_grad():
        for x, y in val_loader:
            x, y = x.to(device), y.to(device)
            out = model(x).float()
            loss_m.update(F.cross_entropy(out, y).item())
            acc_m.update(accuracy(out, y))
    la, aa = loss_m.avg, acc_m.avg
    scalars.add("val/loss", la, epoch)
    scalars.add("val/accuracy", aa, epoch)
    return la, aa


for epoch in range(start_epoch, args.epochs):
    model.train()
    loss_m, acc_m = Metric("train_loss"), Metric("train_accuracy")
    for b, (xb, yb) in enumerate(train_loader):
        if b >= steps_per_epoch:
            break
        adjust_learning_rate(epoch, b)
        if gen is not None:
            send, recv = next(gen)
            w = 1.0 / (len(recv) + 1)
            optimizer.dst_weights, optimizer.src_weights, optimizer.self_weight = send, {r: w for r in recv}, w
        optimizer.zero_grad()
        # gradient accumulation: the sub-batches share one optimizer step, so each contributes its share of the mean
        for x, y in zip(xb.split(args.batch_size), yb.split(args.batch_size)):
            x, y = x.to(device), y.to(device)
            out = model(x).float()
            loss = F.cross_entropy(out, y)
            (loss / args.batches_per_allreduce).backward()
            loss_m.update(loss.item())
            acc_m.update(accuracy(out, y))
        optimizer.step()
    la, aa = loss_m.avg, acc_m.avg
    vl, va = validate(epoch)
    scalars.add("train/loss", la, epoch)
    scalars.add("train/accuracy", aa, epoch)
    if bf.rank() == 0:
        print(f"epoch {epoch}: loss {la:.4f} accuracy {aa:.3f} | validation loss {vl:.4f} accuracy {va:.3f} | "
              f"lr {optimizer.param_groups[0]['lr']:.4f}", flush=True)
    bf.save_checkpoint(args.checkpoint_format.format(epoch=epoch), model, optimizer, extra={"epoch": epoch})
bf.win_free()
bf.barrier()
