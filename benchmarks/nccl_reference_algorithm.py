"""The reference's GPU algorithm, restated with PyTorch's bundled NCCL, as a comparison arm.

What the reference does per training step on its NCCL path (bluefog/common/nccl_controller.cc:
1013-1204, bluefog/torch/mpi_ops.cc:99-164, bluefog/torch/optimizers.py:297-482): parameters
are copied one by one into a fusion buffer (<= 8 MiB groups), exchanged with grouped
ncclSend/ncclRecv, copied out per tensor and per neighbor, combined with one ATen mul/add
per neighbor per tensor, and then the local optimizer applies the gradient in a separate
pass.  Compute is whatever PyTorch dispatches to (cuDNN/cuBLAS), as in the reference's
benchmark.  This is NOT the reference's code; the reference itself cannot be built offline.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import json

import torch
import torch.distributed as dist

FUSION_BYTES = 8 * 1024 * 1024


def _groups(params):
    groups, cur, cur_bytes = [], [], 0
    for p in params:
        nb = p.numel() * p.element_size()
        if cur and cur_bytes + nb > FUSION_BYTES // 2:   # self part + one recv part per in-neighbor
            groups.append(cur)
            cur, cur_bytes = [], 0
        cur.append(p)
        cur_bytes += nb
    if cur:
        groups.append(cur)
    return groups


def neighbor_average_(params, send_to, recv_from, fusion, recv_fusion):
    """One-peer neighbor averaging of ``params`` in place, the reference's way."""
    w = 1.0 / (len(recv_from) + 1)
    for group in _groups(params):
        if len(group) == 1 and group[0].numel() > fusion.numel():
            # a tensor that does not fit the fusion buffer travels on its own (the reference sends
            # such tensors unfused, straight from and into tensor memory)
            p = group[0]
            recv = [torch.empty_like(p.data) for _ in recv_from]
            ops = [dist.P2POp(dist.irecv, recv[j], r) for j, r in enumerate(recv_from)]
            ops += [dist.P2POp(dist.isend, p.data, d) for d in send_to]
            if ops:
                for req in dist.batch_isend_irecv(ops):
                    req.wait()
            p.data.mul_(w)
            for t in recv:
                p.data.add_(t, alpha=w)
            continue
        off = 0
        for p in group:                       # MemcpyInFusionBuffer: one copy per tensor
            n = p.numel()
            fusion[off:off + n].copy_(p.data.reshape(-1))
            off += n
        ops = []
        for j, r in enumerate(recv_from):
            ops.append(dist.P2POp(dist.irecv, recv_fusion[j][:off], r))
        for d in send_to:
            ops.append(dist.P2POp(dist.isend, fusion[:off], d))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        off = 0
        for p in group:                       # copy-out + combine: one mul/add per neighbor per tensor
            n = p.numel()
            p.data.mul_(w)
            for j in range(len(recv_from)):
                p.data.add_(recv_fusion[j][off:off + n].view_as(p.data), alpha=w)
            off += n


def run(args):
    import os
    from bench import ClockSampler, build_model, BASELINE_IMG_PER_SEC_PER_GPU
    from bluefog_b200.common import topology_util as tu
    rank = int(os.environ.get("RANK", "0"))
    size = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if size > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234 + rank)
    model = build_model(args.model, False).to(dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
    for m in model.modules():                 # statistics in fp32, as in mixed-precision training
        if isinstance(m, torch.nn.BatchNorm2d):
            m.running_mean.data = m.running_mean.float()
            m.running_var.data = m.running_var.float()
    master = [p.detach().clone().float() for p in model.parameters()]   # fp32 master weights
    for mp in master:
        mp.grad = torch.zeros_like(mp)
    opt = torch.optim.SGD(master, lr=0.1, momentum=0.9)
    params = list(model.parameters())
    fusion = torch.empty(FUSION_BYTES // 8, device=dev)            # self half of the 8 MiB buffer
    recv_fusion = [torch.empty(FUSION_BYTES // 8, device=dev) for _ in range(3)]
    B = args.batch
    g = torch.Generator().manual_seed(rank)
    host_x = torch.randn(B, 3, 224, 224, generator=g).pin_memory()
    host_y = torch.randint(0, 1000, (B,), generator=g).pin_memory()
    dev_x = host_x.to(dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    dev_y = host_y.to(dev)
    loss_fn = torch.nn.CrossEntropyLoss()
    gen = tu.GetDynamicOnePeerSendRecvRanks(tu.ExponentialTwoGraph(size), rank) if size > 1 else None

    def step(x, y):
        for p in params:
            p.grad = None
        loss = loss_fn(model(x).float(), y)
        loss.backward()
        if gen is not None:                   # AWC: combine the parameters, then apply the local gradient
            send, recv = next(gen)
            neighbor_average_(master, send, recv, fusion, recv_fusion)
        for mp, p in zip(master, params):
            mp.grad.copy_(p.grad)
        opt.step()
        for mp, p in zip(master, params):
            p.data.copy_(mp)
        return loss

    for _ in range(args.warmup):
        step(dev_x, dev_y)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def timed(e2e):
        if size > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            if e2e:
                last = step(host_x.to(dev, non_blocking=True), host_y.to(dev, non_blocking=True)).item()
            else:
                last = step(dev_x, dev_y)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if size > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), float(last)

    ms_dev, _ = timed(False)
    ms_e2e, loss_val = timed(True)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        value = size * B * args.steps / (ms_dev / 1e3)
        print(json.dumps({
            "metric": "ResNet-50 training throughput (img/s), neighbor_allreduce SGD, dynamic one-peer exp2",
            "impl": "nccl-reference-algorithm", "value": round(value, 2), "unit": "img/s", "n_gpus": size,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
            "vs_baseline": round(value / (BASELINE_IMG_PER_SEC_PER_GPU * size), 3),
            "config": {"model": args.model, "global_batch": B * size, "parallelism": f"dp{size}"},
            "clocks": clocks, "gpu_launches": 0,
            "e2e": {"value": round(size * B * args.steps / (ms_e2e / 1e3), 2), "unit": "img/s",
                    "h2d_bytes_per_step": int(host_x.numel() * 4 + host_y.numel() * 8), "d2h_bytes_per_step": 4},
            "final_loss": loss_val}), flush=True)
    if size > 1:
        dist.destroy_process_group()
    return 0
