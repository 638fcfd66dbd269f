"""Fused bucket engine: the CUDA fast path of the distributed optimizers.

Parameters are re-homed into flat buckets (a bucket is what the reference calls a fusion
group, bluefog/common/operations.cc:990-1008, but permanent: nothing is packed per step).
Per bucket there are: an fp32 master buffer, a table of the parameters' gradient addresses (the
gradients stay where autograd allocates them), flat optimizer-state buffers that ``optimizer.state[p][...]`` aliases, optionally a bf16
shadow that ``p.data`` aliases (bf16 compute with fp32 master weights), and a native
``Bucket`` whose peer-mapped, double-buffered published copy the neighbors read.

One kernel launch per bucket and step (two for adapt-then-combine and gradient allreduce)
pulls the in-neighbors' published copies over NVLink, forms the weighted combine, applies
SGD(momentum/nesterov/weight decay) or Adam/AdamW(amsgrad), and writes master, published copy
and shadow in the same pass.  The maths of the three styles is that of the reference
wrappers (bluefog/torch/optimizers.py:297-319, 485-841, 166-294).
"""

import math
import os
from typing import Dict, Optional

import torch

from bluefog_b200.common.basics import get_basics
from bluefog_b200.ops import collectives as _ops

_b = get_basics()

MODE_AWC, MODE_ADAPT_PUBLISH, MODE_COMBINE_ONLY, MODE_GRAD_REDUCE, MODE_PUBLISH_ONLY = 0, 1, 2, 3, 4
OPT_NONE, OPT_SGD, OPT_ADAM = 0, 1, 2
_ALIGN = 64  # elements; keeps every parameter view 128-byte aligned even in bf16


def supported(optimizer, model, communication_type) -> bool:
    """True when the bucket engine can take over: initialised runtime on a GPU, every
    parameter on that GPU in fp32, optimizer exactly SGD, Adam or AdamW, and a
    communication type other than the hierarchical one."""
    from bluefog_b200.parallel.optimizers import CommunicationType
    if not _b.is_initialized() or _b.device() < 0:
        return False
    if type(optimizer) not in (torch.optim.SGD, torch.optim.Adam, torch.optim.AdamW):
        return False
    if communication_type == CommunicationType.hierarchical_neighbor_allreduce:
        return False
    for g in optimizer.param_groups:
        if g.get("capturable") or g.get("differentiable"):
            return False
        for p in g["params"]:
            if not p.is_cuda or p.dtype != torch.float32 or p.is_sparse:
                return False
    return True


def _same_layout(a, b):
    """True when both tensors order their elements identically in memory (strides of extent-1
    dimensions carry no information and are ignored)."""
    return all(sa == sb for sa, sb, n in zip(a.stride(), b.stride(), a.shape) if n > 1)


class _BucketState:
    """Buffers and metadata of one bucket."""

    def __init__(self, group_index, params, names, device, compute_dtype, pub_dtype, opt_kind, group):
        self.group_index = group_index
        self.params = params
        self.names = names
        offsets, n = [], 0
        for p in params:
            offsets.append(n)
            n += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.offsets = offsets
        self.numel = n
        self.strides = [self._dense_strides(p) for p in params]   # taken before the parameters are re-homed
        self.master = torch.zeros(n, dtype=torch.float32, device=device)
        # gradients stay where autograd puts them; the kernel reads them through a pointer table
        self.seg_start = torch.tensor(offsets, dtype=torch.int64, device=device)
        self.seg_numel = torch.tensor([p.numel() for p in params], dtype=torch.int64, device=device)
        self.grad_ptrs = torch.zeros(len(params), dtype=torch.int64, device=device)
        self.grad_ptr_key = None
        self.grad_bf16 = compute_dtype == torch.bfloat16
        self.shadow = torch.zeros(n, dtype=torch.bfloat16, device=device) if compute_dtype == torch.bfloat16 else None
        self.state1 = self.state2 = self.state3 = None
        if opt_kind == OPT_SGD and group.get("momentum", 0) != 0:
            self.state1 = torch.zeros(n, dtype=torch.float32, device=device)
        if opt_kind == OPT_ADAM:
            self.state1 = torch.zeros(n, dtype=torch.float32, device=device)
            self.state2 = torch.zeros(n, dtype=torch.float32, device=device)
            if group.get("amsgrad", False):
                self.state3 = torch.zeros(n, dtype=torch.float32, device=device)
        self.steps = 0            # optimizer updates applied to this bucket
        self.first_step = True    # SGD momentum buffer not initialised yet
        self.native = _b.native.Bucket.create(n, "bfloat16" if pub_dtype == torch.bfloat16 else "float32")

    @staticmethod
    def _dense_strides(p):
        """Strides the bucket keeps for ``p``: channels_last filters stay channels_last (the
        convolution kernels then read them in place instead of re-laying them out every step);
        everything else is stored row-major."""
        if p.dim() == 4 and not p.is_contiguous() and p.is_contiguous(memory_format=torch.channels_last):
            return tuple(p.stride())
        strides, n = [], 1
        for d in reversed(p.shape):
            strides.append(n)
            n *= d
        return tuple(reversed(strides))

    def view(self, flat, i):
        p = self.params[i]
        return flat.as_strided(p.shape, self.strides[i], self.offsets[i])


class _FusedMixin:
    """Methods grafted in front of the user's optimizer class (see ``build``)."""

    # ------------------------------------------------------------------ construction
    def _bf_init(self, model, style, communication_type, num_steps_per_communication,
                 compute_dtype=None, exchange_dtype=torch.float32, bucket_bytes=None):
        from bluefog_b200.parallel.optimizers import CommunicationType, _check_named_parameters
        named, models = _check_named_parameters(self, model)
        self._models = models
        self._parameter_names = {v: k for k, v in named}
        self._style = style
        self._communication_type = communication_type
        self._num_steps_per_communication = max(1, int(num_steps_per_communication))
        self._local_steps = 0
        self.self_weight = None
        self.src_weights = None
        self.dst_weights = None
        self.src_machine_weights = None
        self.dst_machine_weights = None
        self.enable_topo_check = False
        self._synchronized = False
        self._should_synchronize = True
        self._CommunicationType = CommunicationType
        compute_dtype = compute_dtype or torch.float32
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("compute_dtype must be torch.float32 or torch.bfloat16")
        if exchange_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("exchange_dtype must be torch.float32 or torch.bfloat16")
        self._compute_dtype = compute_dtype
        if bucket_bytes is None:
            bucket_bytes = int(os.environ.get("BLUEFOG_B200_BUCKET_BYTES", 64 * 1024 * 1024))
        self._opt_kind = OPT_SGD if isinstance(self, torch.optim.SGD) else OPT_ADAM
        self._adamw = isinstance(self, torch.optim.AdamW)
        device = torch.device("cuda", _b.device())
        self._buckets = []
        with torch.no_grad():
            for gi, group in enumerate(self.param_groups):
                cur, cur_bytes = [], 0
                for p in group["params"]:
                    if not p.requires_grad:
                        continue
                    nbytes = p.numel() * 4
                    if cur and cur_bytes + nbytes > bucket_bytes:
                        self._add_bucket(gi, cur, device, exchange_dtype, group)
                        cur, cur_bytes = [], 0
                    cur.append(p)
                    cur_bytes += nbytes
                if cur:
                    self._add_bucket(gi, cur, device, exchange_dtype, group)
        self.overlap_backward = os.environ.get("BLUEFOG_B200_OVERLAP_BACKWARD", "1") != "0"
        self._step_recipe = None
        self._armed = False      # set by zero_grad(): the next backward belongs to a regular training step
        self._register_overlap_hooks()
        self._publish_all()

    def _add_bucket(self, gi, params, device, pub_dtype, group):
        names = [self._parameter_names[p] for p in params]
        bk = _BucketState(gi, params, names, device, self._compute_dtype, pub_dtype, self._opt_kind, group)
        for i, p in enumerate(params):
            bk.view(bk.master, i).copy_(p.data)
            if bk.shadow is not None:
                bk.view(bk.shadow, i).copy_(p.data)
                p.data = bk.view(bk.shadow, i)
            else:
                p.data = bk.view(bk.master, i)
            p.grad = None
            st = self.state[p]
            if self._opt_kind == OPT_SGD:
                if bk.state1 is not None:
                    old = st.get("momentum_buffer")
                    if isinstance(old, torch.Tensor):
                        bk.view(bk.state1, i).copy_(old)
                        bk.first_step = False
                    st["momentum_buffer"] = bk.view(bk.state1, i)
            else:
                for key, flat in (("exp_avg", bk.state1), ("exp_avg_sq", bk.state2), ("max_exp_avg_sq", bk.state3)):
                    if flat is None:
                        continue
                    old = st.get(key)
                    if isinstance(old, torch.Tensor):
                        bk.view(flat, i).copy_(old)
                    st[key] = bk.view(flat, i)
                old_step = st.get("step")
                if old_step is not None:
                    bk.steps = int(float(old_step))
                st["step"] = torch.tensor(float(bk.steps))
        self._buckets.append(bk)

    # ------------------------------------------------------------------ helpers
    def _new_args(self, bk, mode):
        a = _b.native.BucketStepArgs()
        a.mode = mode
        a.master = bk.master
        a.shadow = bk.shadow
        return a

    def _fill_opt(self, a, bk):
        g = self.param_groups[bk.group_index]
        a.opt = self._opt_kind
        self._fill_grads(a, bk)
        a.lr = float(g["lr"])
        a.weight_decay = float(g.get("weight_decay", 0.0))
        a.maximize = bool(g.get("maximize", False))
        if self._opt_kind == OPT_SGD:
            a.momentum = float(g.get("momentum", 0.0))
            a.dampening = float(g.get("dampening", 0.0))
            a.nesterov = bool(g.get("nesterov", False))
            a.first_step = bk.first_step
            a.state1 = bk.state1
        else:
            b1, b2 = g["betas"]
            step = bk.steps + 1
            a.beta1, a.beta2, a.eps = float(b1), float(b2), float(g["eps"])
            a.bias1 = 1.0 - b1 ** step
            a.bias2 = 1.0 - b2 ** step
            a.adamw = self._adamw
            a.amsgrad = bool(g.get("amsgrad", False))
            a.state1, a.state2, a.state3 = bk.state1, bk.state2, bk.state3

    def _fill_grads(self, a, bk):
        """Points the kernel at the parameters' current ``.grad`` tensors (no flattening copy)."""
        key = []
        want = torch.bfloat16 if bk.grad_bf16 else torch.float32
        for p in bk.params:
            g = p.grad
            if g is None:
                key.append(0)
                continue
            if g.dtype != want or not _same_layout(g, p):
                # the kernel walks gradient and master in memory order: both must share one layout
                fixed = torch.empty_strided(p.shape, p.stride(), dtype=want, device=g.device)
                fixed.copy_(g)
                g = fixed
                p.grad = g
            key.append(g.data_ptr())
        key = tuple(key)
        if key != bk.grad_ptr_key:     # under a CUDA graph the addresses never change after the first step
            bk.grad_ptrs.copy_(torch.tensor(key, dtype=torch.int64))
            bk.grad_ptr_key = key
        a.grad_ptrs, a.seg_start, a.seg_numel = bk.grad_ptrs, bk.seg_start, bk.seg_numel
        a.grad_table_bf16 = bk.grad_bf16

    def _after_update(self, bk):
        bk.steps += 1
        bk.first_step = False

    def _combine_recipe(self, communicate):
        """(self_weight, src_ranks, src_weights, n_readers) for this step."""
        CT = self._CommunicationType
        if not communicate or self._communication_type == CT.empty or _b.size() == 1:
            return 1.0, [], [], 0
        if self._communication_type == CT.allreduce:
            n = _b.size()
            others = [r for r in range(n) if r != _b.rank()]
            return 1.0 / n, others, [1.0 / n] * len(others), len(others)
        sw, src_ranks, src_w, dst_ranks, dst_w, use_dst, _ = _ops._resolve_neighbor_weights(
            self.self_weight, self.src_weights, self.dst_weights)
        if use_dst:
            raise ValueError("The fused optimizers do not support destination weights other than 1.0; "
                             "fold them into the receivers' src_weights or pass fused=False.")
        return sw, src_ranks, src_w, len(dst_ranks)

    def _publish_all(self):
        for bk in self._buckets:
            a = self._new_args(bk, MODE_PUBLISH_ONLY)
            bk.native.step(a)

    # ------------------------------------------------------------------ public API
    @property
    def communication_type(self):
        return self._communication_type

    @communication_type.setter
    def communication_type(self, value):
        assert isinstance(value, self._CommunicationType)
        self._communication_type = value

    def synchronize(self):
        """Everything is ordered on the CUDA stream; kept for API parity."""
        self._synchronized = True

    from contextlib import contextmanager as _cm

    @_cm
    def skip_synchronize(self):
        self._should_synchronize = False
        try:
            yield
        finally:
            self._should_synchronize = True

    def turn_on_timeline(self):
        self._use_timeline = True

    def turn_off_timeline(self):
        self._use_timeline = False

    def zero_grad(self, set_to_none: bool = True):
        self._armed = True
        for bk in self._buckets:
            bk.remaining = len(bk.params)
            for p in bk.params:
                if p.grad is None:
                    continue
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.detach_()
                    p.grad.zero_()

    def _launch_bucket(self, bk, recipe):
        """Launches the step of one bucket on the current stream."""
        self_w, src_ranks, src_w, n_readers = recipe
        if self._style == "awc":
            a = self._new_args(bk, MODE_AWC)
            self._fill_opt(a, bk)
            a.self_weight, a.src_ranks, a.src_weights, a.n_readers = self_w, src_ranks, src_w, n_readers
            bk.native.step(a)
        elif self._style == "atc":
            a = self._new_args(bk, MODE_ADAPT_PUBLISH)
            self._fill_opt(a, bk)
            bk.native.step(a)
            c = self._new_args(bk, MODE_COMBINE_ONLY)
            c.self_weight, c.src_ranks, c.src_weights, c.n_readers = self_w, src_ranks, src_w, n_readers
            bk.native.step(c)
        else:  # gradient allreduce
            n = _b.size()
            if n > 1:
                pub = self._new_args(bk, MODE_PUBLISH_ONLY)
                pub.master = None
                self._fill_grads(pub, bk)
                bk.native.step(pub)
            a = self._new_args(bk, MODE_GRAD_REDUCE)
            self._fill_opt(a, bk)
            others = [r for r in range(n) if r != _b.rank()]
            if n > 1:
                a.src_ranks, a.src_weights, a.n_readers = others, [1.0] * len(others), len(others)
                a.post_scale = 1.0 / n
                bk.native.step(a)
            else:
                a.mode = MODE_AWC  # single rank: plain local update
                bk.native.step(a)
        self._after_update(bk)

    # -- overlap with backward ------------------------------------------------------------------
    def _register_overlap_hooks(self):
        """When all gradients of a bucket exist, its step is launched on a side stream while
        backward continues with the earlier layers (the role of the reference's per-parameter
        backward hooks, bluefog/torch/optimizers.py:556-599, at bucket granularity).  Not used
        while a CUDA graph is being captured, nor with local gradient accumulation."""
        self._comm_stream = torch.cuda.Stream(device=_b.device(), priority=-1)
        self._early = []        # buckets already launched during this backward
        for bk in self._buckets:
            bk.remaining = len(bk.params)
            for p in bk.params:
                p.register_post_accumulate_grad_hook(self._make_ready_hook(bk))

    def _make_ready_hook(self, bk):
        def hook(_param):
            bk.remaining -= 1
            if bk.remaining != 0:
                return
            if (not self.overlap_backward or not self._armed or self._num_steps_per_communication != 1
                    or torch.cuda.is_current_stream_capturing()):
                return
            with torch.no_grad():
                recipe = self._step_recipe
                if recipe is None:
                    recipe = self._step_recipe = self._combine_recipe(True)
                cur = torch.cuda.current_stream()
                self._comm_stream.wait_stream(cur)
                with torch.cuda.stream(self._comm_stream):
                    self._launch_bucket(bk, recipe)
                self._early.append(bk)
        return hook

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._local_steps += 1
        communicate = self._local_steps % self._num_steps_per_communication == 0
        recipe = self._step_recipe if self._early else None
        if recipe is None:
            recipe = self._combine_recipe(communicate)
        tl = getattr(self, "_use_timeline", False)
        if tl:
            _b.timeline_start_activity("fused.step", "FUSED_" + self._style.upper())
        early = set(id(bk) for bk in self._early)
        for bk in self._buckets:
            if id(bk) not in early:
                self._launch_bucket(bk, recipe)
            bk.remaining = len(bk.params)
        if self._early:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
            self._early = []
        self._step_recipe = None
        self._armed = False
        if tl:
            _b.timeline_end_activity("fused.step")
        self._synchronized = False
        return loss

    def check(self):
        """Raises if a kernel gave up waiting for a peer (call after a stream synchronisation)."""
        for bk in self._buckets:
            bk.native.check()

    # ------------------------------------------------------------------ state / checkpoint
    def master_parameters(self) -> Dict[str, torch.Tensor]:
        """fp32 master value of every parameter, keyed by its model name."""
        out = {}
        for bk in self._buckets:
            for i, name in enumerate(bk.names):
                out[name] = bk.view(bk.master, i)
        return out

    @torch.no_grad()
    def load_master_parameters(self, state: Dict[str, torch.Tensor]):
        for bk in self._buckets:
            for i, name in enumerate(bk.names):
                if name in state:
                    bk.view(bk.master, i).copy_(state[name].to(bk.master.device, torch.float32).reshape(bk.params[i].shape))
            if bk.shadow is not None:
                bk.shadow.copy_(bk.master)
        self._publish_all()

    def state_dict(self):
        if self._opt_kind == OPT_ADAM:
            for bk in self._buckets:
                for p in bk.params:
                    self.state[p]["step"] = torch.tensor(float(bk.steps))
        return self._base_cls.state_dict(self)

    @torch.no_grad()
    def load_state_dict(self, state_dict):
        self._base_cls.load_state_dict(self, state_dict)
        # torch replaced the state tensors by copies: move the values back into the flat buffers
        for bk in self._buckets:
            for i, p in enumerate(bk.params):
                st = self.state[p]
                pairs = (("momentum_buffer", bk.state1),) if self._opt_kind == OPT_SGD else \
                    (("exp_avg", bk.state1), ("exp_avg_sq", bk.state2), ("max_exp_avg_sq", bk.state3))
                for key, flat in pairs:
                    if flat is None:
                        continue
                    val = st.get(key)
                    if isinstance(val, torch.Tensor):
                        bk.view(flat, i).copy_(val)
                        if key == "momentum_buffer":
                            bk.first_step = False
                    st[key] = bk.view(flat, i)
                if "step" in st:
                    bk.steps = int(float(st["step"]))

    @torch.no_grad()
    def broadcast_from(self, root_rank: int = 0):
        """Makes masters, optimizer state and step counters equal to the root's, then republishes."""
        for k, bk in enumerate(self._buckets):
            for tag, flat in (("master", bk.master), ("s1", bk.state1), ("s2", bk.state2), ("s3", bk.state3)):
                if flat is not None:
                    _ops.broadcast_(flat, root_rank, name=f"fused.bucket{k}.{tag}")
            meta = torch.tensor([float(bk.steps), float(bk.first_step)], dtype=torch.float64)
            meta = _ops.broadcast(meta, root_rank, name=f"fused.bucket{k}.meta")
            bk.steps, bk.first_step = int(meta[0].item()), bool(meta[1].item())
            if bk.shadow is not None:
                bk.shadow.copy_(bk.master)
        torch.cuda.current_stream().synchronize()
        self._publish_all()


def build(optimizer, model, style, communication_type, num_steps_per_communication, **kwargs):
    """Returns an instance of ``class <Opt>(_FusedMixin, type(optimizer))`` sharing the given
    optimizer's parameter groups and state."""
    base = optimizer.__class__
    cls = type(base.__name__, (_FusedMixin, base), {"_base_cls": base})
    obj = cls.__new__(cls)
    base.__init__(obj, optimizer.param_groups)
    obj.defaults = dict(optimizer.defaults)
    obj.state = optimizer.state
    obj._bf_init(model, style, communication_type, num_steps_per_communication, **kwargs)
    return obj
