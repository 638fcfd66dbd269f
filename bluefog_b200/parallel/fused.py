"""Fused bucket engine: the CUDA fast path of the distributed optimizers.

Parameters are re-homed into flat buckets (a bucket is what the reference calls a fusion
group, bluefog/common/operations.cc:990-1008, but permanent: nothing is packed per step).
Per bucket there are: an fp32 master buffer, a table of the parameters' gradient addresses (the
gradients stay where autograd allocates them), flat optimizer-state buffers that ``optimizer.state[p][...]`` aliases, optionally a bf16
shadow that ``p.data`` aliases (bf16 compute with fp32 master weights), and a native
``Bucket`` whose peer-mapped, double-buffered published copy the neighbors read.

One kernel launch per bucket and step (two for adapt-then-combine and gradient allreduce)
pulls the in-neighbors' published copies over NVLink, forms the weighted combine, applies
SGD(momentum/nesterov/weight decay), Adam/AdamW(amsgrad), RMSprop(momentum, centered), Adagrad or Adadelta, and writes master, published copy
and shadow in the same pass.  The maths of the three styles is that of the reference
wrappers (bluefog/torch/optimizers.py:297-319, 485-841, 166-294).
"""

import math
import os
import weakref
from typing import Dict, Optional

import torch

from bluefog_b200.common.basics import get_basics
from bluefog_b200.ops import collectives as _ops

_b = get_basics()

MODE_AWC, MODE_ADAPT_PUBLISH, MODE_COMBINE_ONLY, MODE_GRAD_REDUCE, MODE_PUBLISH_ONLY = 0, 1, 2, 3, 4
OPT_NONE, OPT_SGD, OPT_ADAM, OPT_RMSPROP, OPT_ADAGRAD, OPT_ADADELTA = 0, 1, 2, 3, 4, 5
_KINDS = ((torch.optim.SGD, OPT_SGD), (torch.optim.Adam, OPT_ADAM), (torch.optim.AdamW, OPT_ADAM),
          (torch.optim.RMSprop, OPT_RMSPROP), (torch.optim.Adagrad, OPT_ADAGRAD), (torch.optim.Adadelta, OPT_ADADELTA))

_ALIGN = 64  # elements; keeps every parameter view 128-byte aligned even in bf16


_live = weakref.WeakSet()     # fused optimizers of this process


def republish_live():
    """Calls ``republish()`` on every fused optimizer of this process.  The collective helpers that write parameters
    in place on all ranks (``broadcast_parameters``, ``allreduce_parameters``, ``broadcast_optimizer_state``) end
    with this, so that wrapping the optimizer first and broadcasting afterwards - the order of the reference's
    examples (examples/pytorch_resnet.py:213-238) - hands the neighbors the broadcast values, not the initial ones."""
    for opt in list(_live):
        opt.republish()


def supported(optimizer, model, communication_type) -> bool:
    """True when the bucket engine can take over: initialised runtime on a GPU, every
    parameter on that GPU in fp32, optimizer exactly SGD, Adam, AdamW, RMSprop, Adagrad or Adadelta."""
    if not _b.is_initialized() or _b.device() < 0:
        return False
    if type(optimizer) not in tuple(cls for cls, _ in _KINDS):
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
        if opt_kind == OPT_RMSPROP:                  # square_avg, momentum_buffer, grad_avg
            self.state1 = torch.zeros(n, dtype=torch.float32, device=device)
            if group.get("momentum", 0) > 0:
                self.state2 = torch.zeros(n, dtype=torch.float32, device=device)
            if group.get("centered", False):
                self.state3 = torch.zeros(n, dtype=torch.float32, device=device)
        if opt_kind == OPT_ADAGRAD:                  # sum
            self.state1 = torch.full((n,), float(group.get("initial_accumulator_value", 0.0)), dtype=torch.float32,
                                     device=device)
        if opt_kind == OPT_ADADELTA:                 # square_avg, acc_delta
            self.state1 = torch.zeros(n, dtype=torch.float32, device=device)
            self.state2 = torch.zeros(n, dtype=torch.float32, device=device)
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
        self._opt_kind = next(kind for cls, kind in _KINDS if isinstance(self, cls))
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
        _live.add(self)

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
                for key, flat in self._state_pairs(bk):
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
        elif self._opt_kind == OPT_RMSPROP:
            a.beta2, a.eps = float(g["alpha"]), float(g["eps"])
            a.momentum = float(g.get("momentum", 0.0))
            a.amsgrad = bool(g.get("centered", False))          # the kernel's flag for the third state array
            a.state1, a.state2, a.state3 = bk.state1, bk.state2, bk.state3
        elif self._opt_kind == OPT_ADAGRAD:
            a.lr = float(g["lr"]) / (1.0 + bk.steps * float(g.get("lr_decay", 0.0)))
            a.eps = float(g["eps"])
            a.state1 = bk.state1
        elif self._opt_kind == OPT_ADADELTA:
            a.beta2, a.eps = float(g["rho"]), float(g["eps"])
            a.state1, a.state2 = bk.state1, bk.state2
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
        """(self_weight, src_ranks, src_weights, n_readers, dst_weights) for this step; ``dst_weights`` is None or
        one weight per rank of the world (what this rank attaches to the copy each destination pulls)."""
        CT = self._CommunicationType
        if not communicate or self._communication_type == CT.empty or _b.size() == 1:
            return 1.0, [], [], 0, None
        if self._communication_type == CT.allreduce:
            n = _b.size()
            others = [r for r in range(n) if r != _b.rank()]
            return 1.0 / n, others, [1.0 / n] * len(others), len(others), None
        if self._communication_type == CT.hierarchical_neighbor_allreduce:
            return self._hierarchical_recipe()
        sw, src_ranks, src_w, dst_ranks, dst_w, use_dst, _ = _ops._resolve_neighbor_weights(
            self.self_weight, self.src_weights, self.dst_weights)
        dst = None
        if isinstance(self.dst_weights, dict):
            # A dictionary of destination weights switches the weight exchange on for this step (on every rank:
            # readers then wait for their sources' weights), whatever the values are.
            dst = [1.0] * _b.size()
            for r, w in zip(dst_ranks, dst_w):
                dst[r] = float(w)
        return sw, src_ranks, src_w, len(dst_ranks), dst

    def _hierarchical_recipe(self):
        """hierarchical_neighbor_allreduce as one weighted pull (the form the generic operation takes as well):
        every rank of my machine and of the in-neighbor machines is a source, with the machine's weight divided by
        the local size; the readers of my copy are the other ranks of my machine and all ranks of the out-neighbor
        machines.  (reference: bluefog/common/nccl_controller.cc:791-857 does a local allreduce, a neighbor
        allreduce between the local roots and a local broadcast.)"""
        ls = _b.local_size()
        sw, src_machines, dst_machines = _ops._resolve_machine_weights(
            self.self_weight, self.src_machine_weights, self.dst_machine_weights)
        me, my_machine = _b.rank(), _b.machine_rank()
        src_ranks, src_w = [], []
        for r in range(my_machine * ls, (my_machine + 1) * ls):
            if r != me:
                src_ranks.append(r)
                src_w.append(sw / ls)
        # as with dst_weights: a dictionary switches the weight exchange on for every rank of the step
        dst = [1.0] * _b.size() if isinstance(self.dst_machine_weights, dict) else None
        for m in sorted(src_machines):
            for r in range(m * ls, (m + 1) * ls):
                src_ranks.append(r)
                src_w.append(src_machines[m] / ls)
        for m, w in dst_machines.items():
            if dst is not None:
                for r in range(m * ls, (m + 1) * ls):
                    dst[r] = w
        n_readers = (ls - 1) + ls * len(dst_machines)
        return sw / ls, src_ranks, src_w, n_readers, dst

    def _publish_all(self):
        for bk in self._buckets:
            a = self._new_args(bk, MODE_PUBLISH_ONLY)
            bk.native.step(a)

    @torch.no_grad()
    def republish(self):
        """Makes values written into ``p.data`` after construction (a broadcast, ``model.load_state_dict``, a manual
        edit) the values the next step starts from and the neighbors read.  With bf16 compute ``p.data`` is the
        bf16 shadow: where it no longer equals the rounded fp32 master it replaces the master value.  The peer-
        visible copy is then written again.  Collective: every rank must call it the same number of times (the
        published versions advance in lockstep)."""
        for bk in self._buckets:
            if bk.shadow is not None:
                changed = bk.shadow != bk.master.to(torch.bfloat16)
                bk.master.copy_(torch.where(changed, bk.shadow.float(), bk.master))
        self._publish_all()

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
        self_w, src_ranks, src_w, n_readers, dst_w = recipe
        if self._style == "awc":
            a = self._new_args(bk, MODE_AWC)
            self._fill_opt(a, bk)
            a.self_weight, a.src_ranks, a.src_weights, a.n_readers = self_w, src_ranks, src_w, n_readers
            if dst_w is not None:
                a.dst_weights, a.read_dst_weights = dst_w, True
            bk.native.step(a)
        elif self._style == "atc":
            a = self._new_args(bk, MODE_ADAPT_PUBLISH)
            self._fill_opt(a, bk)
            if dst_w is not None:
                a.dst_weights = dst_w
            bk.native.step(a)
            c = self._new_args(bk, MODE_COMBINE_ONLY)
            c.self_weight, c.src_ranks, c.src_weights, c.n_readers = self_w, src_ranks, src_w, n_readers
            c.read_dst_weights = dst_w is not None
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
        # a device-side wait of an earlier step that ran out left its record in pinned host memory: raise it now
        # rather than only when somebody calls check()
        self.check()
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
    def load_master_parameters(self, state: Dict[str, torch.Tensor], publish: bool = True):
        """Loads fp32 master values by model name.  ``publish=False`` leaves the peer-visible copy alone for a caller
        that runs on some ranks only and lets every rank call ``republish()`` or ``broadcast_from()`` afterwards."""
        for bk in self._buckets:
            for i, name in enumerate(bk.names):
                if name in state:
                    bk.view(bk.master, i).copy_(state[name].to(bk.master.device, torch.float32).reshape(bk.params[i].shape))
            if bk.shadow is not None:
                bk.shadow.copy_(bk.master)
        if publish:
            self._publish_all()

    def _state_pairs(self, bk):
        if self._opt_kind == OPT_SGD:
            return (("momentum_buffer", bk.state1),)
        if self._opt_kind == OPT_RMSPROP:
            return (("square_avg", bk.state1), ("momentum_buffer", bk.state2), ("grad_avg", bk.state3))
        if self._opt_kind == OPT_ADAGRAD:
            return (("sum", bk.state1),)
        if self._opt_kind == OPT_ADADELTA:
            return (("square_avg", bk.state1), ("acc_delta", bk.state2))
        return (("exp_avg", bk.state1), ("exp_avg_sq", bk.state2), ("max_exp_avg_sq", bk.state3))

    def state_dict(self):
        if self._opt_kind != OPT_SGD:
            for bk in self._buckets:
                for p in bk.params:
                    self.state[p]["step"] = torch.tensor(float(bk.steps))
        out = self._base_cls.state_dict(self)
        # What the flat buffers cannot say by themselves (whether SGD's momentum buffer has been initialised yet, the
        # update count) travels as one more entry of the first parameter group, so that the dictionary keeps the two
        # top-level keys of every torch optimizer.
        if out["param_groups"]:
            out["param_groups"][0] = dict(out["param_groups"][0])
            out["param_groups"][0]["bluefog_b200"] = {"first_step": [bool(bk.first_step) for bk in self._buckets],
                                                      "steps": [int(bk.steps) for bk in self._buckets]}
        return out

    @torch.no_grad()
    def load_state_dict(self, state_dict):
        """Loads hyper-parameters through the base class and copies the state tensors straight into the fp32 flat
        buffers.  (``torch.optim.Optimizer.load_state_dict`` casts floating state to the parameter's dtype, which
        with bf16 compute is the bf16 shadow: the moments would lose their low mantissa bits on every resume.)"""
        saved_groups = state_dict["param_groups"]
        if len(saved_groups) != len(self.param_groups) or any(
                len(sg["params"]) != len(g["params"]) for sg, g in zip(saved_groups, self.param_groups)):
            raise ValueError("loaded state dict does not match the optimizer's parameter groups")
        by_id = {}
        for sg, g in zip(saved_groups, self.param_groups):
            for old_id, p in zip(sg["params"], g["params"]):
                by_id[old_id] = p
        loaded = {by_id[k]: v for k, v in state_dict["state"].items() if k in by_id}
        extra = saved_groups[0].get("bluefog_b200") if saved_groups else None
        saved_groups = [{k: v for k, v in sg.items() if k != "bluefog_b200"} for sg in saved_groups]
        self._base_cls.load_state_dict(self, {"state": {}, "param_groups": saved_groups})
        for k, bk in enumerate(self._buckets):
            saw_momentum = False
            for i, p in enumerate(bk.params):
                src = loaded.get(p, {})
                st = self.state[p]
                for key, flat in self._state_pairs(bk):
                    if flat is None:
                        continue
                    val = src.get(key)
                    if isinstance(val, torch.Tensor):
                        bk.view(flat, i).copy_(val.to(flat.device, torch.float32).reshape(p.shape))
                        saw_momentum = saw_momentum or key == "momentum_buffer"
                    st[key] = bk.view(flat, i)
                if "step" in src:
                    bk.steps = int(float(src["step"]))
                if self._opt_kind != OPT_SGD:
                    st["step"] = torch.tensor(float(bk.steps))
            if extra is not None and k < len(extra.get("first_step", [])):
                bk.first_step = bool(extra["first_step"][k])
                bk.steps = int(extra["steps"][k])
            elif self._opt_kind == OPT_SGD:
                bk.first_step = not saw_momentum     # a torch.optim.SGD dict has buffers only after its first step

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
