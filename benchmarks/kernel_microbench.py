"""Single-GPU timing of the hand-written kernels against the measured machine peaks.

  python benchmarks/kernel_microbench.py --kernel bucket --numel 67108864
  python benchmarks/kernel_microbench.py --kernel combine --numel 67108864 --dtype bfloat16
  python benchmarks/kernel_microbench.py --kernel gemm --m 8192 --n 8192 --k 8192
  python benchmarks/kernel_microbench.py --kernel conv_layers --batch 64
  python benchmarks/kernel_microbench.py --kernel bn_layers --batch 64

The multi-rank kernels run on a one-process "local world": the peers' buffers are other
buffers of the same GPU, so the numbers are HBM-bound, not NVLink-bound; they show how close
the kernels come to the copy bandwidth of the device.  Inputs are larger than the 126 MB L2.
Timing: CUDA events around `--iters` launches after `--warmup`, reported per launch.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # repository root
import argparse
import json
import os

import torch

from bluefog_b200 import _C

PEAKS = {"hbm_gbs": 6530.6, "bf16_tflops": 1659.0}
_peaks_file = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
if os.path.exists(_peaks_file):
    with open(_peaks_file) as f:
        PEAKS.update({k: v for k, v in json.load(f).items() if k in PEAKS})


def timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def timed_graph(fn, iters, warmup):
    """Device time per call with the host out of the picture: ``iters`` calls captured into one CUDA graph, the graph
    replayed ``warmup`` times untimed and then once between two events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_bucket(args):
    n, W = args.numel, 2
    buckets = _C.Bucket.create_local(W, n, args.exchange, 0)
    master = [torch.randn(n, device="cuda") for _ in range(W)]
    grad = [torch.randn(n, device="cuda").to(torch.bfloat16) for _ in range(W)]
    mom = [torch.zeros(n, device="cuda") for _ in range(W)]
    adam = args.bucket_opt == "adamw"
    second = [torch.zeros(n, device="cuda") for _ in range(W)] if adam else None
    shadow = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    for r in range(W):
        a = _C.BucketStepArgs()
        a.mode, a.master = 4, master[r]
        buckets[r].step(a)
    state = {"first": True}

    def step():
        for r in range(W):
            a = _C.BucketStepArgs()
            a.mode, a.opt = 0, 1
            a.master, a.grad, a.state1, a.shadow = master[r], grad[r], mom[r], shadow[r]
            a.lr, a.momentum, a.first_step = 0.01, 0.9, state["first"]
            if adam:
                a.opt, a.adamw, a.state2 = 2, True, second[r]
                a.beta1, a.beta2, a.eps, a.bias1, a.bias2, a.weight_decay = 0.9, 0.999, 1e-8, 0.5, 0.1, 0.01
            a.self_weight, a.src_ranks, a.src_weights, a.n_readers = 0.5, [1 - r], [0.5], 1
            buckets[r].step(a)
        state["first"] = False

    ms = timed(step, args.iters, args.warmup) / W
    pub = 4 if args.exchange == "float32" else 2
    # per element: master r+w (8), peer published copy r, own published copy w, grad r (2), momentum r+w (8), shadow w (2)
    bytes_per_launch = n * (8 + 2 * pub + 2 + 8 + 2 + (8 if adam else 0))             # AdamW: second moment r+w
    return {"kernel": "bucket_step_kernel (AWC, %s, bf16 grad+shadow)" % ("AdamW" if adam else "SGD momentum"),
            "numel": n, "ms": ms,
            "gbs": bytes_per_launch / ms / 1e6, "frac_of_measured_hbm": bytes_per_launch / ms / 1e6 / PEAKS["hbm_gbs"]}


def bench_combine(args):
    dtype = getattr(torch, args.dtype)
    n, W = args.numel, 2
    esize = torch.empty(0, dtype=dtype).element_size()
    world = _C.LocalWorld(W, n * esize + 4096, 0)
    xs = [torch.randn(n, device="cuda").to(dtype) for _ in range(W)]
    outs = [torch.empty(n, device="cuda", dtype=dtype) for _ in range(W)]

    def step():
        rounds = [world.publish(r, [xs[r]], None, 1) for r in range(W)]
        for r in range(W):
            world.combine(r, rounds[r], [outs[r]], 0.5, [1 - r], [0.5], False, 1.0)

    ms = timed(step, args.iters, args.warmup) / W
    # publish: read x, write arena; combine: read own arena + peer arena, write out
    bytes_per_rank = n * esize * 5
    return {"kernel": "pack_publish_kernel + combine_kernel", "dtype": args.dtype, "numel": n, "ms_per_rank": ms,
            "gbs": bytes_per_rank / ms / 1e6, "frac_of_measured_hbm": bytes_per_rank / ms / 1e6 / PEAKS["hbm_gbs"]}


def bench_gemm(args):
    """--gemm-layout nt: a[M,K] w[N,K]^T (forward);  nn: a[M,K] b[K,N] (input gradient);  tn: a[K,M]^T b[K,N] (weight
    gradient).  M, N, K are the extents of the product in every layout."""
    m, n, k = args.m, args.n, args.k
    if args.gemm_layout == "nt":
        a = (torch.randn(m, k, device="cuda") * 0.1).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
        ours, lib = (lambda: _C.gemm_bf16_nt(a, w, None, 0)), (lambda: torch.matmul(a, w.t()))
    elif args.gemm_layout == "nn":
        a = (torch.randn(m, k, device="cuda") * 0.1).to(torch.bfloat16)
        w = (torch.randn(k, n, device="cuda") * 0.1).to(torch.bfloat16)
        ours, lib = (lambda: _C.gemm_bf16_nn(a, w)), (lambda: torch.matmul(a, w))
    else:
        a = (torch.randn(k, m, device="cuda") * 0.1).to(torch.bfloat16)
        w = (torch.randn(k, n, device="cuda") * 0.1).to(torch.bfloat16)
        ours, lib = (lambda: _C.gemm_bf16_tn(a, w)), (lambda: torch.matmul(a.t(), w))
    ms = timed(ours, args.iters, args.warmup)
    ms_lib = timed(lib, args.iters, args.warmup)
    flops = 2.0 * m * n * k
    nbytes = 2.0 * (m * k + n * k + m * n)     # A, B read once, C written once
    out = {"kernel": "gemm_bf16_nt_persistent_kernel (tcgen05)", "layout": args.gemm_layout, "m": m, "n": n, "k": k,
           "ms": ms, "tflops": flops / ms / 1e9, "frac_of_measured_bf16": flops / ms / 1e9 / PEAKS["bf16_tflops"],
           "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / PEAKS["hbm_gbs"],
           "library_ms": ms_lib, "library_tflops": flops / ms_lib / 1e9}
    if args.gemm_col_stats and args.gemm_layout == "nt" and n % 8 == 0:
        # the epilogue variant that also takes the column statistics of its output, against the separate
        # statistics pass of the BatchNorm kernels over the same [M, N] activation (the sums buffer is cleared
        # inside the timed call in both arms)
        stats = torch.zeros(2 * n, device="cuda")
        y = _C.gemm_bf16_nt(a, w, None, 0)
        out["with_col_stats_ms"] = timed(lambda: (stats.zero_(), _C.gemm_bf16_nt(a, w, None, 0, stats)), args.iters, args.warmup)
        x4 = y.view(1, m, 1, n).permute(0, 3, 1, 2)                   # the NHWC activation a BatchNorm would see
        if _C.bn_supported(x4):
            g, b = torch.ones(n, device="cuda"), torch.zeros(n, device="cuda")
            full = timed(lambda: (stats.zero_(), _C.bn_forward(x4, None, g, b, None, None, 1e-5, 0.1, True, stats, False)),
                         args.iters, args.warmup)
            apply_only = timed(lambda: (stats.zero_(), _C.bn_forward(x4, None, g, b, None, None, 1e-5, 0.1, True, stats, True)),
                               args.iters, args.warmup)
            out["bn_forward_ms"], out["bn_forward_without_statistics_pass_ms"] = full, apply_only
    out["status"] = _C.gemm_status()
    return out


def bench_conv(args):
    n, cin, cout, h, w = args.conv_shape
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.05).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    ms = timed(lambda: _C.conv3x3_nhwc(x, wt), args.iters, args.warmup)
    ms_lib = timed(lambda: torch.nn.functional.conv2d(x, wt, padding=1), args.iters, args.warmup)
    flops = 2.0 * n * h * w * cout * cin * 9
    return {"kernel": "conv3x3_nhwc_kernel (tcgen05 implicit GEMM)", "shape": [n, cin, cout, h, w], "ms": ms,
            "tflops": flops / ms / 1e9, "frac_of_measured_bf16": flops / ms / 1e9 / PEAKS["bf16_tflops"],
            "library_ms": ms_lib, "library_tflops": flops / ms_lib / 1e9, "status": _C.gemm_status()}


# (count in ResNet-50, Cin, Cout, kernel, stride, input height = width) of every convolution of the network
RESNET50_CONVS = [
    (1, 64, 64, 1, 1, 56), (3, 64, 64, 3, 1, 56), (4, 64, 256, 1, 1, 56), (2, 256, 64, 1, 1, 56),
    (1, 256, 128, 1, 1, 56), (1, 128, 128, 3, 2, 56), (4, 128, 512, 1, 1, 28), (1, 256, 512, 1, 2, 56),
    (3, 512, 128, 1, 1, 28), (3, 128, 128, 3, 1, 28),
    (1, 512, 256, 1, 1, 28), (1, 256, 256, 3, 2, 28), (6, 256, 1024, 1, 1, 14), (1, 512, 1024, 1, 2, 28),
    (5, 1024, 256, 1, 1, 14), (5, 256, 256, 3, 1, 14),
    (1, 1024, 512, 1, 1, 14), (1, 512, 512, 3, 2, 14), (3, 512, 2048, 1, 1, 7), (1, 1024, 2048, 1, 2, 14),
    (2, 2048, 512, 1, 1, 7), (2, 512, 512, 3, 1, 7),
]


def bench_conv_layers(args):
    """Forward, input gradient and filter gradient of every convolution shape of ResNet-50 at batch --batch: this
    library's kernels (through the autograd functions the model uses) against the library convolutions with
    ``cudnn.benchmark`` on, each timed as a CUDA graph of --iters calls (no host time in the numbers; the operands of
    one layer fit in L2, as they mostly do between the layers of a step).  One JSON line per shape and a last line with
    the sums weighted by layer count."""
    from bluefog_b200.ops import conv
    torch.backends.cudnn.benchmark = True
    n = args.batch
    aten_bwd = torch.ops.aten.convolution_backward
    total = {"ours": [0.0, 0.0, 0.0], "lib": [0.0, 0.0, 0.0]}
    for count, cin, cout, k, stride, hw in RESNET50_CONVS:
        pad = k // 2
        x = torch.randn(n, cin, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        wt = (torch.randn(cout, cin, k, k, device="cuda") * 0.05).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        ho = (hw + 2 * pad - k) // stride + 1
        dy = torch.randn(n, cout, ho, ho, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        if k == 1 and stride == 1:
            x2d, dy2d, w2d = x.permute(0, 2, 3, 1).reshape(-1, cin), dy.permute(0, 2, 3, 1).reshape(-1, cout), wt.reshape(cout, cin)
            ours_fns = [lambda: _C.gemm_bf16_nt(x2d, w2d, None, 0), lambda: _C.gemm_bf16_nn(dy2d, w2d),
                        lambda: _C.conv_wgrad(dy, x, [0], [0], [0], 1, 1, False)]
        else:
            ours_fns = [lambda: conv.forward_product(x, wt, stride, pad), lambda: conv.input_gradient(dy, wt, x.shape, stride, pad),
                        lambda: conv.filter_gradient(dy, x, k, stride, pad)]
        ours = [timed_graph(f, args.iters, args.warmup) for f in ours_fns]
        conv_args = (None, (stride, stride), (pad, pad), (1, 1), False, (0, 0), 1)
        lib = [timed_graph(lambda: torch.nn.functional.conv2d(x, wt, stride=stride, padding=pad), args.iters, args.warmup),
               timed_graph(lambda: aten_bwd(dy, x, wt, *conv_args, (True, False, False)), args.iters, args.warmup),
               timed_graph(lambda: aten_bwd(dy, x, wt, *conv_args, (False, True, False)), args.iters, args.warmup)]
        flops = 2.0 * n * ho * ho * cout * cin * k * k
        for i in range(3):
            total["ours"][i] += count * ours[i]
            total["lib"][i] += count * lib[i]
        print(json.dumps({"conv": [count, cin, cout, k, stride, hw], "ours_ms_fwd_dgrad_wgrad": [round(v, 4) for v in ours],
                          "library_ms_fwd_dgrad_wgrad": [round(v, 4) for v in lib],
                          "ours_tflops": [round(flops / v / 1e9, 1) for v in ours], "status": _C.gemm_status()}), flush=True)
    return {"kernel": "all ResNet-50 convolutions, batch %d: sum over layers (ms)" % n,
            "ours_fwd_dgrad_wgrad_ms": [round(v, 3) for v in total["ours"]], "ours_total_ms": round(sum(total["ours"]), 3),
            "library_fwd_dgrad_wgrad_ms": [round(v, 3) for v in total["lib"]], "library_total_ms": round(sum(total["lib"]), 3)}


def bench_wgrad(args):
    """One filter gradient (--conv-shape N CIN COUT H W, --ksize, --stride) on the split-K kernel and on the library."""
    from bluefog_b200.ops import conv
    torch.backends.cudnn.benchmark = True
    n, cin, cout, h, w = args.conv_shape
    k, stride = args.ksize, args.stride
    pad = k // 2
    ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    x = torch.randn(n, cin, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wt = torch.zeros(cout, cin, k, k, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    dy = torch.randn(n, cout, ho, wo, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    ms = timed_graph(lambda: conv.filter_gradient(dy, x, k, stride, pad), args.iters, args.warmup)
    conv_args = (None, (stride, stride), (pad, pad), (1, 1), False, (0, 0), 1)
    ms_lib = timed_graph(lambda: torch.ops.aten.convolution_backward(dy, x, wt, *conv_args, (False, True, False)), args.iters, args.warmup)
    flops = 2.0 * n * ho * wo * cout * cin * k * k
    nbytes = 2.0 * (x.numel() + dy.numel() + wt.numel())
    return {"kernel": "conv_wgrad_kernel (tcgen05, split-K)", "shape": [n, cin, cout, h, w], "ksize": k, "stride": stride,
            "ms": ms, "tflops": flops / ms / 1e9, "frac_of_measured_bf16": flops / ms / 1e9 / PEAKS["bf16_tflops"],
            "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / PEAKS["hbm_gbs"],
            "library_ms": ms_lib, "status": _C.gemm_status()}


def bench_ln(args):
    """LayerNorm forward/backward on [rows, 1024] and the bias-gradient column sum on [rows/4, 4096] (both
    134 MB at the default 65536 rows: larger than L2)."""
    rows = args.ln_rows
    x = torch.randn(rows, 1024, device="cuda").to(torch.bfloat16)
    w, b = torch.ones(1024, device="cuda"), torch.zeros(1024, device="cuda")
    dy = torch.randn_like(x)
    wide = torch.randn(max(rows // 4, 8), 4096, device="cuda").to(torch.bfloat16)
    y, mean, rstd = _C.ln_forward(x, w, b, 1e-5)
    nb = x.numel() * 2
    ms_f = timed(lambda: _C.ln_forward(x, w, b, 1e-5), args.iters, args.warmup)
    ms_b = timed(lambda: _C.ln_backward(dy, x, w, mean, rstd), args.iters, args.warmup)
    ms_b2 = timed(lambda: _C.ln_backward(dy, x, w, mean, rstd, y), args.iters, args.warmup)     # + residual term, + column sums
    ms_c = timed(lambda: _C.column_sum(wide), args.iters, args.warmup)
    ms_t = timed(lambda: wide.sum(0, dtype=torch.float32), args.iters, args.warmup)
    ms_tf = timed(lambda: torch.nn.functional.layer_norm(x, (1024,), w.bfloat16(), b.bfloat16()), args.iters, args.warmup)
    peak = PEAKS["hbm_gbs"]
    return {"kernel": "ln_fwd_kernel / ln_bwd_kernel / column_sum_kernel", "rows": rows,
            "ln_fwd_ms": ms_f, "ln_fwd_frac_of_measured_hbm": 2 * nb / ms_f / 1e6 / peak,       # read x, write y
            "ln_bwd_ms": ms_b, "ln_bwd_frac_of_measured_hbm": 3 * nb / ms_b / 1e6 / peak,       # read dy, x, write dx
            "ln_bwd_residual_ms": ms_b2, "ln_bwd_residual_frac_of_measured_hbm": 4 * nb / ms_b2 / 1e6 / peak,
            "column_sum_ms": ms_c, "column_sum_frac_of_measured_hbm": wide.numel() * 2 / ms_c / 1e6 / peak,
            "pytorch_layer_norm_fwd_ms": ms_tf, "pytorch_sum_ms": ms_t}


def bench_bn(args):
    n, c, h, w = args.bn_shape
    x = torch.randn(n, c, h, w, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    res = torch.randn_like(x)
    gamma = torch.ones(c, device="cuda")
    beta = torch.zeros(c, device="cuda")
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    y, mean, rstd, mask = _C.bn_forward(x, res, gamma, beta, rm, rv, 1e-5, 0.1, True)
    dy = torch.randn_like(x)
    ms_f = timed(lambda: _C.bn_forward(x, res, gamma, beta, rm, rv, 1e-5, 0.1, True), args.iters, args.warmup)
    ms_b = timed(lambda: _C.bn_backward(dy, mask, x, mean, rstd, gamma, True, True), args.iters, args.warmup)
    bn = torch.nn.BatchNorm2d(c).cuda()

    bn16 = bn.to(torch.bfloat16)
    ms_tf = timed(lambda: torch.relu(bn16(x) + res), args.iters, args.warmup)
    nbytes = x.numel() * 2
    # forward: stats read x; apply reads x, residual, writes y (+ 1 bit/element).  backward: reduce reads dy, x
    # (+ bits); apply reads dy, x (+ bits) and writes dx, dresidual.
    return {"kernel": "bn_stats+bn_apply / bn_bwd_reduce+bn_bwd_apply (ReLU + residual)", "shape": [n, c, h, w],
            "fwd_ms": ms_f, "fwd_gbs": 4.0625 * nbytes / ms_f / 1e6, "fwd_frac_of_measured_hbm": 4.0625 * nbytes / ms_f / 1e6 / PEAKS["hbm_gbs"],
            "bwd_ms": ms_b, "bwd_gbs": 6.125 * nbytes / ms_b / 1e6, "bwd_frac_of_measured_hbm": 6.125 * nbytes / ms_b / 1e6 / PEAKS["hbm_gbs"],
            "pytorch_fwd_ms (bn, add, relu)": ms_tf}


# (count, channels, height = width, relu, residual) of every BatchNorm of ResNet-50 (stride on the 3x3 convolution)
RESNET50_BNS = [
    (1, 64, 112, True, False),
    (6, 64, 56, True, False), (3, 256, 56, True, True), (1, 256, 56, False, False),
    (1, 128, 56, True, False), (7, 128, 28, True, False), (4, 512, 28, True, True), (1, 512, 28, False, False),
    (1, 256, 28, True, False), (11, 256, 14, True, False), (6, 1024, 14, True, True), (1, 1024, 14, False, False),
    (1, 512, 14, True, False), (5, 512, 7, True, False), (3, 2048, 7, True, True), (1, 2048, 7, False, False),
]


def bench_bn_layers(args):
    """Forward and backward of every BatchNorm(+ReLU, +residual) shape of ResNet-50 at batch --batch, each timed as a
    CUDA graph of --iters calls (statistics workspace cleared once per graph, as the model clears it once per step).
    One JSON line per shape with the traffic each pass has to move and the rate it reached, and a last line with the
    sums weighted by layer count."""
    n = args.batch
    tot_f = tot_b = tot_bytes_f = tot_bytes_b = 0.0
    for count, c, hw, relu, residual in RESNET50_BNS:
        x = torch.randn(n, c, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        res = torch.randn_like(x) if residual else None
        dy = torch.randn_like(x)
        gamma, beta = torch.ones(c, device="cuda"), torch.zeros(c, device="cuda")
        rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        ws = torch.zeros(args.iters + 8, 2 * c if args.bn_two_kernels else _C.bn_workspace_floats(c), device="cuda")
        y, mean, rstd, mask = _C.bn_forward(x, res, gamma, beta, rm, rv, 1e-5, 0.1, relu)
        calls = [0]

        def slot():
            i = calls[0] % (args.iters + 8)
            if i == 0:
                ws.zero_()
            calls[0] += 1
            return ws[i]

        def fwd():
            return _C.bn_forward(x, res, gamma, beta, rm, rv, 1e-5, 0.1, relu, slot())

        def bwd():
            return _C.bn_backward(dy, mask if relu else None, x, mean, rstd, gamma, relu, residual, slot())

        calls[0] = 0
        ms_f = timed_graph(fwd, args.iters, 0)
        calls[0] = 0
        ms_b = timed_graph(bwd, args.iters, 0)
        nb = x.numel() * 2
        bits = 1.0 / 16 if relu else 0.0
        bytes_f = nb * (3 + (1 if residual else 0) + bits)             # read x twice (+ residual), write y (+ bits)
        bytes_b = nb * (5 + (1 if residual else 0) + 2 * bits)         # read dy, x twice (+ bits), write dx (+ dresidual)
        tot_f += count * ms_f
        tot_b += count * ms_b
        tot_bytes_f += count * bytes_f
        tot_bytes_b += count * bytes_b
        print(json.dumps({"bn": [count, c, hw, relu, residual], "mbytes": round(nb / 1e6, 1), "fwd_ms": round(ms_f, 4),
                          "bwd_ms": round(ms_b, 4), "fwd_gbs": round(bytes_f / ms_f / 1e6), "bwd_gbs": round(bytes_b / ms_b / 1e6),
                          "fwd_floor_ms": round(bytes_f / PEAKS["hbm_gbs"] / 1e6, 4),
                          "bwd_floor_ms": round(bytes_b / PEAKS["hbm_gbs"] / 1e6, 4)}), flush=True)
    return {"kernel": "all ResNet-50 BatchNorm layers, batch %d: sum over layers (ms)" % n, "fwd_ms": round(tot_f, 3),
            "bwd_ms": round(tot_b, 3), "fwd_floor_ms_at_measured_hbm": round(tot_bytes_f / PEAKS["hbm_gbs"] / 1e6, 3),
            "bwd_floor_ms_at_measured_hbm": round(tot_bytes_b / PEAKS["hbm_gbs"] / 1e6, 3)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=["bucket", "combine", "gemm", "bn", "bn_layers", "conv", "conv_layers", "wgrad", "ln"])
    ap.add_argument("--ksize", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--bucket-opt", choices=["sgd", "adamw"], default="sgd")
    ap.add_argument("--ln-rows", type=int, default=65536)
    ap.add_argument("--conv-shape", type=int, nargs=5, default=[64, 64, 64, 56, 56], metavar=("N", "CIN", "COUT", "H", "W"))
    ap.add_argument("--bn-shape", type=int, nargs=4, default=[64, 256, 56, 56])
    ap.add_argument("--bn-two-kernels", action="store_true",
                    help="bn_layers: no barrier word behind the sums, so every pass is statistics kernel + apply kernel")
    ap.add_argument("--numel", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--exchange", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--gemm-layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--gemm-col-stats", action="store_true", help="also time the epilogue that takes column statistics")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    out = {"bucket": bench_bucket, "combine": bench_combine, "gemm": bench_gemm, "bn": bench_bn, "bn_layers": bench_bn_layers, "conv": bench_conv, "conv_layers": bench_conv_layers, "wgrad": bench_wgrad,
           "ln": bench_ln}[args.kernel](args)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
