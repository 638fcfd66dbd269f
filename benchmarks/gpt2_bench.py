"""GPT-2 medium data-parallel throughput (tokens/s) with adapt-then-combine AdamW over a ring.

Config: 24 layers, d_model 1024, 16 heads, vocab 50257, sequence 1024, bf16 compute with fp32
master weights, batch 8 sequences per GPU of token ids uniform in [0, 50257) from seed=rank,
RingGraph topology, 64 MiB buckets.

  bfrun -np 8 python benchmarks/gpt2_bench.py --steps 10 --warmup 3
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import json

import torch

import bluefog_b200.torch as bf
from bluefog_b200.models import gpt2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--model", default="gpt2_medium", choices=["gpt2_small", "gpt2_medium"])
    ap.add_argument("--no-b200-gemm", action="store_true")
    ap.add_argument("--exchange-dtype", default="bfloat16", choices=["float32", "bfloat16"],
                    help="format in which neighbors read each other's parameters (the own term and the master "
                         "weights stay fp32)")
    ap.add_argument("--no-graphs", action="store_true", help="drive forward/backward op by op instead of a CUDA graph")
    args = ap.parse_args()
    bf.init()
    rank, size = bf.rank(), bf.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    bf.set_topology(bf.RingGraph(size), is_weighted=True)
    torch.manual_seed(1 + rank)
    model = getattr(gpt2, args.model)(use_b200_gemm=not args.no_b200_gemm).to(dev)
    bf.broadcast_parameters(model.state_dict(), root_rank=0)
    opt = bf.DistributedAdaptThenCombineOptimizer(
        torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1), model,
        compute_dtype=torch.bfloat16, exchange_dtype=getattr(torch, args.exchange_dtype),
        bucket_bytes=64 * 1024 * 1024)
    g = torch.Generator().manual_seed(rank)
    tokens = torch.randint(0, 50257, (args.batch, args.seq + 1), generator=g).to(dev)
    x, y = tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous()

    if args.no_graphs:
        def step():
            opt.zero_grad()
            loss = model(x, y)
            loss.backward()
            opt.step()
            return loss
    else:
        from bluefog_b200.utils.graphs import GraphedForwardBackward
        graphed = GraphedForwardBackward(model, None, opt, x, y, forward_loss=model)

        def step():
            loss = graphed(x, y)
            opt.step()
            return loss

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    opt.check()
    bf.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    opt.check()
    ms = float(bf.allgather(torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)).max())
    if rank == 0:
        toks = size * args.batch * args.seq * args.steps / (ms / 1e3)
        print(json.dumps({"metric": "GPT-2 training throughput (tokens/s), ATC AdamW, ring", "value": round(toks, 1),
                          "unit": "tokens/s", "n_gpus": size, "ms_per_step": round(ms / args.steps, 2),
                          "model": args.model, "batch_per_gpu": args.batch, "seq_len": args.seq, "dtype": "bf16",
                          "exchange_dtype": args.exchange_dtype,
                          "final_loss": float(loss)}), flush=True)
    bf.barrier()
    bf.shutdown()


if __name__ == "__main__":
    main()
