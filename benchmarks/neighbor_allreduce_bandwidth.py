"""neighbor_allreduce / win_put bandwidth sweep (role of the reference's scripts/single_ops_test.py,
extended to the sweep of message sizes and topologies).

  bfrun -np 8 python benchmarks/neighbor_allreduce_bandwidth.py --out sweep.json

For every size (4 KB ... 1 GB, powers of 4), dtype (fp32, bf16) and topology (static exp2,
dynamic one-peer exp2) it times, on the device with CUDA events and as the max over ranks:
  * ours      - bf.neighbor_allreduce (peer-memory pull kernel),
  * nccl      - the reference's algorithm: grouped NCCL send/recv + one mul/add per neighbor,
  * win_put   - bf.win_put into the neighbors' windows (static topology only).
GB/s counts the bytes every rank must receive over NVLink per operation (in-degree x size);
the roofline fraction is against 770 GB/s per direction measured for a peer copy on this pool.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import json
import os

import torch

import bluefog_b200.torch as bf
from bluefog_b200.common import topology_util as tu

NVLINK_GBS = 770.0


def device_time_ms(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    bf.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64)
    return float(bf.allgather(ms).max())


def pipelined_time_ms(issue, iters, warmup):
    """Issues ``iters`` nonblocking operations back to back and waits for all of them; the closing
    event is recorded after the last handle completed, so the figure can only err on the slow side."""
    # as many outputs alive at once as in the timed series, so that the allocator has settled
    for h in [issue(k) for k in range(max(warmup, iters))]:
        bf.synchronize(h)
    torch.cuda.synchronize()
    bf.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    handles = [issue(k) for k in range(iters)]
    outs = [bf.synchronize(h) for h in handles]
    e1.record()
    torch.cuda.synchronize()
    del outs
    ms = e0.elapsed_time(e1) / iters
    return float(bf.allgather(torch.tensor([ms], dtype=torch.float64)).max())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    ap.add_argument("--skip-nccl", action="store_true")
    args = ap.parse_args()
    bf.init()
    rank, size = bf.rank(), bf.size()
    dev = torch.device("cuda", torch.cuda.current_device())
    bf.set_topology(tu.ExponentialTwoGraph(size))
    bf.set_skip_negotiate_stage(True)   # steady-state path: all ranks issue the same ops in order
    nccl = None
    if not args.skip_nccl and size > 1:
        import torch.distributed as dist
        if os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True":
            # under torchrun every rank is a client of the agent's store at MASTER_PORT
            dist.init_process_group("nccl", init_method="env://", rank=rank, world_size=size, device_id=dev)
        else:
            port = int(os.environ.get("MASTER_PORT", "29500")) + 7
            dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=size,
                                    device_id=dev)
        nccl = dist
    results = []
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4
    in_nb, out_nb = bf.in_neighbor_ranks(), bf.out_neighbor_ranks()
    for dtype in (torch.float32, torch.bfloat16):
        esize = 4 if dtype == torch.float32 else 2
        for nbytes in sizes:
            numel = nbytes // esize
            x = (torch.rand(numel, generator=torch.Generator().manual_seed(rank)) * 2 - 1).to(dev).to(dtype)
            for mode in ("static_exp2", "one_peer_exp2"):
                gen = tu.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), rank)

                def ours():
                    if mode == "static_exp2":
                        return bf.neighbor_allreduce(x, name="bw")
                    send, recv = next(gen)
                    w = 1.0 / (len(recv) + 1)
                    return bf.neighbor_allreduce(x, self_weight=w, src_weights={r: w for r in recv},
                                                 dst_weights=send, enable_topo_check=False, name="bw")

                def ours_nonblocking(k):
                    if mode == "static_exp2":
                        return bf.neighbor_allreduce_nonblocking(x, name=f"bw.nb.{k}")
                    send, recv = next(gen)
                    w = 1.0 / (len(recv) + 1)
                    return bf.neighbor_allreduce_nonblocking(x, self_weight=w, src_weights={r: w for r in recv},
                                                             dst_weights=send, enable_topo_check=False,
                                                             name=f"bw.nb.{k}")

                indeg = len(in_nb) if mode == "static_exp2" else 1
                ms = device_time_ms(ours, args.iters, args.warmup)
                row = {"op": "neighbor_allreduce", "impl": "ours", "dtype": str(dtype).split(".")[-1], "bytes": nbytes,
                       "mode": mode, "ms": ms, "gbs": indeg * nbytes / ms / 1e6,
                       "roofline_frac": indeg * nbytes / ms / 1e6 / NVLINK_GBS}
                results.append(row)
                # the same operations issued back to back through the nonblocking API and waited for at the
                # end, which is how the NCCL arm below runs (its wait() only orders streams)
                ms_nb = pipelined_time_ms(ours_nonblocking, args.iters, args.warmup)
                results.append({"op": "neighbor_allreduce", "impl": "ours-nonblocking", "dtype": row["dtype"],
                                "bytes": nbytes, "mode": mode, "ms": ms_nb, "gbs": indeg * nbytes / ms_nb / 1e6,
                                "roofline_frac": indeg * nbytes / ms_nb / 1e6 / NVLINK_GBS})
                if nccl is not None:
                    recv_bufs = [torch.empty_like(x) for _ in range(len(in_nb))]
                    gen2 = tu.GetDynamicOnePeerSendRecvRanks(bf.load_topology(), rank)

                    def ref():
                        if mode == "static_exp2":
                            send, recv = out_nb, in_nb
                        else:
                            send, recv = next(gen2)
                        ops = [nccl.P2POp(nccl.irecv, recv_bufs[j], r) for j, r in enumerate(recv)]
                        ops += [nccl.P2POp(nccl.isend, x, d) for d in send]
                        for req in nccl.batch_isend_irecv(ops):
                            req.wait()
                        w = 1.0 / (len(recv) + 1)
                        out = x * w
                        for j in range(len(recv)):
                            out.add_(recv_bufs[j], alpha=w)
                        return out

                    ms2 = device_time_ms(ref, args.iters, args.warmup)
                    results.append({"op": "neighbor_allreduce", "impl": "nccl-reference-algorithm",
                                    "dtype": row["dtype"], "bytes": nbytes, "mode": mode, "ms": ms2,
                                    "gbs": indeg * nbytes / ms2 / 1e6})
                    del recv_bufs
            # win_put, static topology
            w = torch.zeros_like(x)
            bf.win_create(w, "bw.win", zero_init=True)

            def put():
                bf.win_put(x, "bw.win")

            ms3 = device_time_ms(put, args.iters, args.warmup)
            results.append({"op": "win_put", "impl": "ours", "dtype": str(dtype).split(".")[-1], "bytes": nbytes,
                            "mode": "static_exp2", "ms": ms3, "gbs": len(out_nb) * nbytes / ms3 / 1e6,
                            "roofline_frac": len(out_nb) * nbytes / ms3 / 1e6 / NVLINK_GBS})
            bf.win_free("bw.win")
            del x, w
            torch.cuda.empty_cache()
    if rank == 0:
        for r in results:
            print(json.dumps(r), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump({"n_gpus": size, "results": results}, f, indent=1)
    bf.barrier()
    if nccl is not None:
        nccl.destroy_process_group()
    bf.shutdown()


if __name__ == "__main__":
    main()
