"""CUDA-graph capture of the forward+backward pass.

Batch-64 ResNet-50 on a B200 is bound by kernel-launch latency when it is driven op by op from
Python (hundreds of kernels of a few microseconds each).  ``GraphedForwardBackward`` captures
``zero_grad -> forward -> loss -> backward`` once into a CUDA graph and replays it per step; the
distributed optimizer step (whose neighbor lists, weights and version numbers change from step
to step) stays outside the graph and is launched normally.  It relies on the fused optimizers
keeping ``p.data`` and ``p.grad`` at fixed addresses (views of the flat buckets).
"""
import torch


class GraphedForwardBackward:
    """Usage::

        step = GraphedForwardBackward(model, loss_fn, optimizer, example_x, example_y)
        # or: GraphedForwardBackward(model, None, optimizer, tokens, targets, forward_loss=model)
        for x, y in loader:
            loss = step(x, y)        # copies x, y into the static buffers and replays the graph
            optimizer.step()
    """

    def __init__(self, model, loss_fn, optimizer, example_x, example_y, warmup: int = 3, forward_loss=None):
        """``forward_loss(x, y) -> loss`` replaces ``loss_fn(model(x).float(), y)`` for models that
        compute their own loss (e.g. a language model called with targets)."""
        if not example_x.is_cuda:
            raise ValueError("CUDA graphs need CUDA tensors")
        self.model, self.loss_fn, self.optimizer = model, loss_fn, optimizer
        self.forward_loss = forward_loss
        if hasattr(optimizer, "overlap_backward"):
            # bucket steps launched from backward hooks have per-step arguments: they cannot live in a graph
            optimizer.overlap_backward = False
        self.static_x = example_x.clone()
        self.static_y = example_y.clone()
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):           # lets cuDNN pick algorithms and allocators settle
                self._eager()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from bluefog_b200.common.basics import get_basics
        native = get_basics().native
        before = native.kernel_launch_count()
        with torch.cuda.graph(self.graph):
            self.static_loss = self._eager()
        # kernels of this library inside the graph (each replay launches them again)
        self.native_launches_per_replay = native.kernel_launch_count() - before
        torch.cuda.synchronize()

    def _eager(self):
        self.optimizer.zero_grad()
        if self.forward_loss is not None:
            loss = self.forward_loss(self.static_x, self.static_y)
        else:
            out = self.model(self.static_x)
            loss = self.loss_fn(out.float(), self.static_y)
        loss.backward()
        return loss.detach()

    def __call__(self, x, y):
        self.static_x.copy_(x, non_blocking=True)
        self.static_y.copy_(y, non_blocking=True)
        self.graph.replay()
        return self.static_loss
