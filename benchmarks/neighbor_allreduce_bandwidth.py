"""Bandwidth sweep of neighbor_allreduce, the window operations and the global collectives (role of the reference's
scripts/single_ops_test.py, extended to the sweep of message sizes and topologies).

  bfrun -np 8 python benchmarks/neighbor_allreduce_bandwidth.py --out sweep.json

For every size (4 KB ... 1 GB, powers of 4), dtype (fp32, bf16) and topology (static exp2,
dynamic one-peer exp2) it times, on the device with CUDA events and as the max over ranks:
  * ours      - bf.neighbor_allreduce (peer-memory pull kernel),
  * nccl      - the reference's algorithm: grouped NCCL send/recv + one mul/add per neighbor,
  * win_put / win_accumulate / win_get / win_update (static topology only),
  * allreduce / broadcast / allgather against torch.distributed's NCCL (bus bandwidth as nccl-tests define it).
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
    ap.add_argument("--registered", action="store_true",
                    help="also time neighbor_allreduce on tensors of bf.symmetric_empty (published in place)")
    ap.add_argument("--registered-min-bytes", type=int, default=0)
    ap.add_argument("--ops", default="neighbor,windows,collectives",
                    help="comma-separated: neighbor (neighbor_allreduce), windows (win_put/accumulate/get/update), "
                         "collectives (allreduce/broadcast/allgather against NCCL)")
    args = ap.parse_args()
    ops = set(args.ops.split(","))
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
            for mode in (("static_exp2", "one_peer_exp2") if "neighbor" in ops else ()):
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
                if args.registered and nbytes >= args.registered_min_bytes:
                    # the same operation on a tensor in symmetric memory: published in place, no copy into the arena
                    xr = bf.symmetric_empty(numel, dtype=dtype)
                    xr.copy_(x)
                    keep, x = x, xr
                    ms_r = device_time_ms(ours, args.iters, args.warmup)
                    x = keep
                    results.append({"op": "neighbor_allreduce", "impl": "ours-registered", "dtype": row["dtype"],
                                    "bytes": nbytes, "mode": mode, "ms": ms_r, "gbs": indeg * nbytes / ms_r / 1e6,
                                    "roofline_frac": indeg * nbytes / ms_r / 1e6 / NVLINK_GBS})
                    del xr
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
            dname = str(dtype).split(".")[-1]
            if "windows" in ops:
                # one-sided operations, static topology: put and accumulate write into every out-neighbor's slot, get
                # reads every in-neighbor's tensor, update folds the slots locally (HBM-bound, no NVLink traffic)
                w = torch.zeros_like(x)
                bf.win_create(w, "bw.win", zero_init=True)
                for op, fn, peers in (("win_put", lambda: bf.win_put(x, "bw.win"), len(out_nb)),
                                      ("win_accumulate", lambda: bf.win_accumulate(x, "bw.win"), len(out_nb)),
                                      ("win_get", lambda: bf.win_get("bw.win"), len(in_nb))):
                    ms3 = device_time_ms(fn, args.iters, args.warmup)
                    results.append({"op": op, "impl": "ours", "dtype": dname, "bytes": nbytes, "mode": "static_exp2",
                                    "ms": ms3, "gbs": peers * nbytes / ms3 / 1e6,
                                    "roofline_frac": peers * nbytes / ms3 / 1e6 / NVLINK_GBS})
                ms4 = device_time_ms(lambda: bf.win_update("bw.win"), args.iters, args.warmup)
                # reads self and every slot, writes self
                results.append({"op": "win_update", "impl": "ours", "dtype": dname, "bytes": nbytes, "mode": "static_exp2",
                                "ms": ms4, "gbs": (len(in_nb) + 2) * nbytes / ms4 / 1e6})
                bf.win_free("bw.win")
                del w
            if "collectives" in ops:
                # bus-bandwidth convention of nccl-tests: allreduce 2(n-1)/n * S / t, allgather (n-1)/n * n*S / t,
                # broadcast S / t
                n = size
                for op, ours, ref, factor in (
                        ("allreduce", lambda: bf.allreduce(x, average=False, name="bw.ar"),
                         (lambda: nccl.all_reduce(xr)) if nccl else None, 2.0 * (n - 1) / n),
                        ("broadcast", lambda: bf.broadcast(x, 0, name="bw.bc"),
                         (lambda: nccl.broadcast(xr, 0)) if nccl else None, 1.0),
                        ("allgather", lambda: bf.allgather(x, name="bw.ag"),
                         (lambda: nccl.all_gather_into_tensor(gather_out, xr)) if nccl else None, float(n - 1))):
                    if op == "allgather" and nbytes * n > (2 << 30):
                        continue
                    xr = x.clone()
                    gather_out = torch.empty(numel * n, dtype=dtype, device=dev) if op == "allgather" else None
                    ms5 = device_time_ms(ours, args.iters, args.warmup)
                    results.append({"op": op, "impl": "ours", "dtype": dname, "bytes": nbytes, "ms": ms5,
                                    "busbw_gbs": factor * nbytes / ms5 / 1e6})
                    if ref is not None:
                        ms6 = device_time_ms(ref, args.iters, args.warmup)
                        results.append({"op": op, "impl": "nccl", "dtype": dname, "bytes": nbytes, "ms": ms6,
                                        "busbw_gbs": factor * nbytes / ms6 / 1e6})
                    del xr, gather_out
            del x
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
