"""Headline benchmark: ResNet-50 training throughput (images/s) with decentralized SGD.

Protocol of the reference's examples/pytorch_benchmark.py (synthetic 3x224x224 images,
batch 64 per GPU, SGD, neighbor averaging over the dynamic one-peer exponential-2 schedule),
timed on the device with CUDA events, max over ranks.

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

``--impl reference`` would run the unmodified reference from baseline/_ref; it cannot be
installed offline (its build needs an MPI compiler wrapper), so that arm prints an
``unavailable`` line.  ``--impl nccl`` runs the reference's *algorithm* (per-tensor copies into
a fusion buffer, grouped NCCL send/recv, torch combine, separate optimizer step) on the same
model for comparison.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

BASELINE_IMG_PER_SEC_PER_GPU = 4310.6 / 16.0  # reference docs/performance.rst:14-24 (V100)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--b200-gemm", nargs="?", const="all", default="all", choices=["off", "auto", "all"],
                    help="1x1 convolutions and the classifier on the tcgen05 GEMM / implicit-GEMM kernels: all of them "
                         "(default), 'auto' = the stride-1 ones of at most 16384 pixels, or 'off' = library kernels")
    ap.add_argument("--library-conv", action="store_true",
                    help="3x3 convolutions and the stem on the library (cuDNN) instead of the tcgen05 implicit-GEMM "
                         "kernels (forward, input gradient and filter gradient)")
    ap.add_argument("--library-loss", action="store_true", help="F.cross_entropy instead of the fused loss kernels")
    ap.add_argument("--no-graphs", action="store_true", help="drive forward/backward op by op instead of a CUDA graph")
    ap.add_argument("--stem", default="s2d", choices=["s2d", "7x7"],
                    help="evaluate the 7x7/2 stem convolution as a 4x4 convolution over 2x2 pixel blocks (s2d) or directly")
    ap.add_argument("--exchange-dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--no-cudnn-benchmark", action="store_true",
                    help="leave cuDNN on its heuristics instead of timing its algorithms per shape in the warm-up "
                         "(the reference's benchmark sets cudnn.benchmark = True, examples/pytorch_benchmark.py:76)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_model(name, use_gemm, stem_s2d=False, use_conv=False):
    from bluefog_b200.models import resnet
    return getattr(resnet, name)(use_b200_gemm=use_gemm, stem_space_to_depth=stem_s2d, use_b200_conv=use_conv)


def make_loss(args):
    """Mean cross-entropy of the bf16 logits: the fused kernels of this library, or PyTorch's on an fp32 copy."""
    if args.library_loss:
        ce = torch.nn.CrossEntropyLoss()
        return lambda logits, y: ce(logits.float(), y)
    from bluefog_b200.ops.fused_ce import cross_entropy
    return cross_entropy


def timed_end_to_end(step, host_x, host_y, like_x, like_y, steps, barrier):
    """Device time of ``steps`` steps that each take their inputs from pinned host memory (copied on a copy stream,
    one step ahead, into one of two device buffers) and deliver their loss to the host (read one step later, so that
    launching step i+1 does not wait for step i to drain).  Returns (milliseconds, last loss)."""
    copy_stream = torch.cuda.Stream()
    bufs = [(torch.empty_like(like_x), torch.empty_like(like_y)) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def prefetch(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[b])      # step i-2 has finished reading this buffer
            bufs[b][0].copy_(host_x, non_blocking=True)
            bufs[b][1].copy_(host_y, non_blocking=True)
            ready[b].record(copy_stream)

    loss_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event() for _ in range(2)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    e0.record()
    prefetch(0)
    loss_val = float("nan")
    for i in range(steps):
        if i + 1 < steps:
            prefetch(i + 1)
        b = i % 2
        torch.cuda.current_stream().wait_event(ready[b])
        loss_t = step(bufs[b][0], bufs[b][1])
        consumed[b].record(torch.cuda.current_stream())
        loss_host[b].copy_(loss_t.detach().float(), non_blocking=True)
        loss_ready[b].record(torch.cuda.current_stream())
        if i > 0:
            loss_ready[1 - b].synchronize()
            loss_val = float(loss_host[1 - b])
    loss_ready[(steps - 1) % 2].synchronize()
    loss_val = float(loss_host[(steps - 1) % 2])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), loss_val


def one_peer_schedule(bf, size, rank):
    if size == 1:
        while True:
            yield [], []
    gen = bf.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), rank)
    while True:
        yield next(gen)


def run_ours(args):
    import bluefog_b200.torch as bf
    bf.init()
    rank, size = bf.rank(), bf.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    bf.set_topology(bf.ExponentialTwoGraph(size))
    torch.manual_seed(1234 + rank)
    use_gemm = {"off": False, "auto": "auto", "all": True}[args.b200_gemm]
    model = build_model(args.model, use_gemm, (args.stem == "s2d"), not args.library_conv).to(dev).to(memory_format=torch.channels_last)
    bf.broadcast_parameters(model.state_dict(), root_rank=0)
    base = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    opt = bf.DistributedNeighborAllreduceOptimizer(
        base, model, compute_dtype=torch.bfloat16,
        exchange_dtype=torch.bfloat16 if args.exchange_dtype == "bfloat16" else torch.float32)
    sched = one_peer_schedule(bf, size, rank)
    B = args.batch
    g = torch.Generator().manual_seed(rank)
    host_x = torch.randn(B, 3, 224, 224, generator=g).pin_memory()
    host_y = torch.randint(0, 1000, (B,), generator=g).pin_memory()
    # the batch as a data loader delivers it: fp32 NCHW; cast, padding and layout change are the stem kernel's job
    dev_x = host_x.to(dev)
    dev_y = host_y.to(dev)
    loss_fn = make_loss(args)

    def set_weights():
        send, recv = next(sched)
        if size > 1:
            w = 1.0 / (len(recv) + 1)
            opt.dst_weights = list(send)
            opt.src_weights = {r: w for r in recv}
            opt.self_weight = w

    graphed = None
    if not args.no_graphs:
        from bluefog_b200.utils.graphs import GraphedForwardBackward
        graphed = GraphedForwardBackward(model, None, opt, dev_x, dev_y,
                                         forward_loss=lambda x, y: loss_fn(model(x), y))

    def step(x, y):
        set_weights()
        if graphed is not None:
            loss = graphed(x, y)          # zero_grad + forward + loss + backward as one CUDA graph
        else:
            opt.zero_grad()
            loss = loss_fn(model(x), y)
            loss.backward()
        opt.step()
        return loss

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64)
        allv = bf.allgather(t)
        return float(allv.max())

    for _ in range(args.warmup):
        step(dev_x, dev_y)
    torch.cuda.synchronize()
    opt.check()

    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    # device-resident inputs
    bf.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = bf._b.native.kernel_launch_count()
    e0.record()
    for _ in range(args.steps):
        loss = step(dev_x, dev_y)
    e1.record()
    torch.cuda.synchronize()
    launches = bf._b.native.kernel_launch_count() - l0
    if graphed is not None:
        launches += args.steps * graphed.native_launches_per_replay
    ms_dev = max_over_ranks(e0.elapsed_time(e1))
    ms_e2e, loss_val = timed_end_to_end(step, host_x, host_y, dev_x, dev_y, args.steps, bf.barrier)
    ms_e2e = max_over_ranks(ms_e2e)
    clocks = sampler.stop() if rank == 0 else None
    opt.check()
    ok = bool(torch.isfinite(torch.tensor(loss_val)))
    from bluefog_b200.ops import gemm
    if rank == 0:
        value = size * B * args.steps / (ms_dev / 1e3)
        e2e = size * B * args.steps / (ms_e2e / 1e3)
        out = {
            "metric": "ResNet-50 training throughput (img/s), neighbor_allreduce SGD, dynamic one-peer exp2",
            "value": round(value, 2), "unit": "img/s", "n_gpus": size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / (BASELINE_IMG_PER_SEC_PER_GPU * size), 3),
            "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": args.model, "global_batch": B * size, "batch_per_gpu": B, "image": "3x224x224",
                       "parallelism": f"dp{size}", "optimizer": "SGD momentum 0.9 lr 0.1, fp32 master weights",
                       "topology": "ExponentialTwoGraph, dynamic one-peer", "exchange_dtype": args.exchange_dtype,
                       "b200_gemm": args.b200_gemm if gemm.available() else "off",
                       "b200_conv": bool(not args.library_conv and gemm.available()),
                       "loss": "library" if args.library_loss else "fused cross-entropy kernels",
                       "stem": "space-to-depth 4x4" if (args.stem == "s2d") else "7x7 stride 2",
                       "cudnn_benchmark": bool(torch.backends.cudnn.benchmark),
                       "cuda_graph": "forward+backward" if not args.no_graphs else "none",
                       "l2": "inputs plus activations exceed the 126 MB L2 every step; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 2), "unit": "img/s",
                    "h2d_bytes_per_step": int(host_x.numel() * 4 + host_y.numel() * 8),
                    "host_input": "pinned fp32 NCHW images + int64 labels, copied one step ahead on a copy stream", "host_output": "loss of every step copied to pinned memory and read by the host one step later",
                    "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / args.steps, 3)},
            "gpu_launches": int(launches),
            "final_loss": loss_val, "finite": ok,
        }
        print(json.dumps(out), flush=True)
    bf.barrier()
    bf.shutdown()


def main():
    args = parse_args()
    torch.backends.cudnn.benchmark = not args.no_cudnn_benchmark
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0                      # one line per job, printed by rank 0
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference does not install offline: its setup.py needs mpicxx "
                                         "(no MPI on this image), boost/flatbuffers submodules are empty, "
                                         "and it includes TH/THC headers removed from torch 2.x"}), flush=True)
        return 0
    if args.impl == "nccl":
        from benchmarks.nccl_reference_algorithm import run as run_nccl
        return run_nccl(args)
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
