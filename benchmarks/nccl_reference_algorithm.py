"""The reference's GPU algorithm at its best on this machine, restated with PyTorch's bundled NCCL, as the
comparison arm of ``bench.py`` (``--impl nccl``).

What the reference does per training step on its NCCL path (bluefog/common/nccl_controller.cc:1013-1204,
bluefog/torch/optimizers.py:354-400, 437-482): the parameter exchange of a step is *started from the forward
hooks* - fusion groups of at most 8 MiB travel with grouped ncclSend/ncclRecv on NCCL's own stream while forward
and backward run - and is *joined in step()*, where the received copies are combined with ATen mul/add and the
local optimizer then applies the gradient.  This arm keeps exactly that structure and removes everything that is
not the algorithm:

* the model, its kernels and the CUDA-graph capture of zero-grad/forward/loss/backward are the ones ``bench.py``
  uses for this library's arm (same ``build_model`` flags), so the two arms differ in the exchange and the update
  only;
* the fp32 master weights live in one flat buffer, so "copy into the fusion buffer" costs nothing and a fusion
  group is a slice; all groups of a step go out in one grouped call on a side stream that runs beside the graph;
* combine = two passes over the flat buffer (``mul_``, ``add_``); the update is ``torch.optim.SGD(fused=True)`` on
  fp32 gradient copies made by one ``_foreach_copy_``; the bf16 compute copy is refreshed by one more.

This is NOT the reference's code; the reference itself cannot be built offline.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import json

import torch
import torch.distributed as dist

FUSION_BYTES = 8 * 1024 * 1024


class _Grads:
    """What ``GraphedForwardBackward`` needs from an optimizer: ``zero_grad``."""

    def __init__(self, params):
        self.params = params

    def zero_grad(self):
        for p in self.params:
            p.grad = None


def run(args):
    from bench import (BASELINE_IMG_PER_SEC_PER_GPU, ClockSampler, build_model, make_loss, timed_end_to_end)
    from bluefog_b200.common import topology_util as tu
    from bluefog_b200.utils.graphs import GraphedForwardBackward
    rank = int(os.environ.get("RANK", "0"))
    size = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if size > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234 + rank)
    use_gemm = {"off": False, "auto": "auto", "all": True}[args.b200_gemm]
    model = build_model(args.model, use_gemm, (args.stem == "s2d"), not args.library_conv).to(dev)
    model = model.to(memory_format=torch.channels_last)
    params = [p for p in model.parameters() if p.requires_grad]
    # fp32 masters in one flat buffer (each parameter keeps its memory order), bf16 compute copies in the model
    sizes = [(p.numel() + 63) // 64 * 64 for p in params]
    flat = torch.zeros(sum(sizes), dtype=torch.float32, device=dev)
    master, off = [], 0
    for p, n in zip(params, sizes):
        m = flat.as_strided(p.shape, p.stride(), off)
        m.copy_(p.data)
        master.append(m)
        off += n
    for p in params:
        p.data = p.data.to(torch.bfloat16)
    if size > 1:
        dist.broadcast(flat, 0)
        torch._foreach_copy_([p.data for p in params], master)
    master_params = [torch.nn.Parameter(m, requires_grad=True) for m in master]
    for mp in master_params:
        mp.grad = torch.zeros_like(mp)
    opt = torch.optim.SGD(master_params, lr=0.1, momentum=0.9, fused=True)
    recv = torch.empty_like(flat) if size > 1 else None
    group_elems = FUSION_BYTES // 4
    B = args.batch
    g = torch.Generator().manual_seed(rank)
    host_x = torch.randn(B, 3, 224, 224, generator=g).pin_memory()
    host_y = torch.randint(0, 1000, (B,), generator=g).pin_memory()
    dev_x, dev_y = host_x.to(dev), host_y.to(dev)
    loss_fn = make_loss(args)
    gen = tu.GetDynamicOnePeerSendRecvRanks(tu.ExponentialTwoGraph(size), rank) if size > 1 else None
    comm_stream = torch.cuda.Stream()
    graphed = None
    if not args.no_graphs:
        graphed = GraphedForwardBackward(model, None, _Grads(params), dev_x, dev_y,
                                         forward_loss=lambda x, y: loss_fn(model(x), y))

    def start_exchange():
        """Grouped send/recv of the masters in fusion groups of 8 MiB, beside forward and backward."""
        send, recv_from = next(gen)
        comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(comm_stream):
            ops = []
            for lo in range(0, flat.numel(), group_elems):
                hi = min(flat.numel(), lo + group_elems)
                for r in recv_from:
                    ops.append(dist.P2POp(dist.irecv, recv[lo:hi], r))
                for d in send:
                    ops.append(dist.P2POp(dist.isend, flat[lo:hi], d))
            reqs = dist.batch_isend_irecv(ops) if ops else []
        return reqs, len(recv_from)

    def step(x, y):
        pending = start_exchange() if gen is not None else None
        if graphed is not None:
            loss = graphed(x, y)
        else:
            for p in params:
                p.grad = None
            loss = loss_fn(model(x), y)
            loss.backward()
        if pending is not None:
            reqs, n_recv = pending
            for req in reqs:
                req.wait()
            torch.cuda.current_stream().wait_stream(comm_stream)
            if n_recv:
                w = 1.0 / (n_recv + 1)
                flat.mul_(w).add_(recv, alpha=w)            # AWC: combine, then apply the local gradient
        torch._foreach_copy_([mp.grad for mp in master_params], [p.grad for p in params])
        opt.step()
        torch._foreach_copy_([p.data for p in params], master)
        return loss

    for _ in range(args.warmup):
        step(dev_x, dev_y)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def barrier():
        if size > 1:
            dist.barrier()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev)
        if size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(dev_x, dev_y)
    e1.record()
    torch.cuda.synchronize()
    ms_dev = max_over_ranks(e0.elapsed_time(e1))
    ms_e2e, loss_val = timed_end_to_end(step, host_x, host_y, dev_x, dev_y, args.steps, barrier)
    ms_e2e = max_over_ranks(ms_e2e)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        value = size * B * args.steps / (ms_dev / 1e3)
        print(json.dumps({
            "metric": "ResNet-50 training throughput (img/s), neighbor_allreduce SGD, dynamic one-peer exp2",
            "impl": "nccl-reference-algorithm", "value": round(value, 2), "unit": "img/s", "n_gpus": size,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
            "vs_baseline": round(value / (BASELINE_IMG_PER_SEC_PER_GPU * size), 3),
            "config": {"model": args.model, "global_batch": B * size, "parallelism": f"dp{size}",
                       "exchange": "fp32 masters, grouped NCCL send/recv in 8 MiB groups beside forward/backward",
                       "update": "mul_/add_ combine, torch.optim.SGD(fused=True), _foreach_copy_ casts",
                       "model_kernels": "as this library's arm", "cuda_graph": "forward+backward" if graphed else "none"},
            "clocks": clocks, "gpu_launches": 0,
            "e2e": {"value": round(size * B * args.steps / (ms_e2e / 1e3), 2), "unit": "img/s",
                    "h2d_bytes_per_step": int(host_x.numel() * 4 + host_y.numel() * 8), "d2h_bytes_per_step": 4},
            "final_loss": loss_val}), flush=True)
    if size > 1:
        dist.destroy_process_group()
    return 0
