"""Distributed optimizer wrappers.

Every factory returns an object whose class derives from the class of the optimizer it was
given, so ``state_dict()`` keeps the plain torch layout (as in the reference,
bluefog/torch/optimizers.py:1180-1554).  Update styles:

* adapt-with-combine (AWC; ``DistributedAdaptWithCombineOptimizer`` and the older
  ``DistributedNeighborAllreduceOptimizer`` / ``DistributedAllreduceOptimizer`` /
  ``DistributedHierarchicalNeighborAllreduceOptimizer``): the parameter exchange is launched
  from a forward hook and overlaps forward+backward; ``step()`` installs the combined
  parameters and then applies the local gradient:  w+ = Combine(w) - lr * g(w).
* adapt-then-combine (ATC): a per-parameter backward hook applies the local update as soon as
  the gradient exists and then launches the exchange:  w+ = Combine(w - lr * g(w)).
* gradient allreduce (Horovod style), one-sided win_put / pull-get, and push-sum.

On CUDA with SGD, Adam/AdamW, RMSprop, Adagrad or Adadelta the AWC, ATC and gradient-allreduce styles run on the
fused bucket engine (``bluefog_b200.parallel.fused``): parameters live in flat peer-mapped
buckets and one kernel per bucket does combine + update + casts.  Everything else uses the
per-parameter path below, which works for any optimizer class and any device.
"""

import itertools
import os
import warnings
from contextlib import contextmanager
from enum import Enum

import torch

import bluefog_b200.ops.collectives as _ops
import bluefog_b200.ops.windows as _win
from bluefog_b200.common.basics import get_basics

_b = get_basics()


class CommunicationType(Enum):
    neighbor_allreduce = "neighbor.allreduce"
    hierarchical_neighbor_allreduce = "hierarchical.neighbor.allreduce"
    allreduce = "allreduce"
    empty = "empty"


_WARN_STEPS = (
    "Unexpected behavior:\n"
    "  After num_steps_per_communication times of forward computation `y=model(x)` are called,\n"
    "  an optimizer step() function must be called.\n"
    "  It does not matter how many step() functions are called in between.\n"
    "  Please adjust num_step_per_communication to update model parameters locally.\n"
    "  More information can be found in the FAQ page.\n")
_WARN_BACKWARD = (
    "Unexpected behavior:\n"
    "  After num_steps_per_communication times of backward computation `loss.backward()` are called,\n"
    "  an optimizer step() function must be called.\n"
    "  It does not matter how many step() functions are called in between.\n"
    "  Please adjust num_steps_per_communication to accumulate gradients locally.\n"
    "  More information can be found in the FAQ page.\n")
_WARN_DOUBLE_SYNC = (
    "optimizer.step() called without optimizer.skip_synchronize() context after "
    "optimizer.synchronize(). This can cause training slowdown. You may want to consider using "
    "optimizer.skip_synchronize() context if you use optimizer.synchronize() in your code.")


def _named_leaf_module(module, parent_name=None):
    """Yields (qualified name, module) for every module without children."""
    children = list(module.named_children())
    if not children:
        yield parent_name, module
    for name, child in children:
        yield from _named_leaf_module(child, parent_name + "." + name if parent_name else name)


def _check_named_parameters(optimizer, model):
    models = [model] if isinstance(model, torch.nn.Module) else list(model)
    for m in models:
        assert isinstance(m, torch.nn.Module)
    named = list(itertools.chain(*[m.named_parameters() for m in models]))
    seen, dups = set(), set()
    for k, _ in named:
        (dups if k in seen else seen).add(k)
    if dups:
        raise ValueError("Parameter names in named_parameters must be unique. "
                         "Found duplicates: %s" % ", ".join(sorted(dups)))
    opt_ids = {id(v) for g in optimizer.param_groups for v in g["params"]}
    missing = opt_ids - {id(v) for _, v in named}
    if missing:
        raise ValueError("Named parameters provided by model are mismatch with the parameters"
                         "handled by optimizer. Python object ids: %s" % ", ".join(str(i) for i in missing))
    return named, models


def _register_timeline(optimizer, models, parameter_names, parent_name=None):
    """FORWARD and GRADIENT COMPT. spans per parameter, from module and tensor hooks
    (reference: bluefog/torch/optimizers.py:112-163)."""
    handles = []

    def pre_forward(module, *unused):
        for _, p in module.named_parameters(recurse=False):
            if p in parameter_names:
                _b.timeline_start_activity(parameter_names[p], "FORWARD")

    def post_forward(module, *unused):
        for _, p in module.named_parameters(recurse=False):
            if p in parameter_names:
                _b.timeline_end_activity(parameter_names[p])
                _b.timeline_start_activity(parameter_names[p], "GRADIENT COMPT.")

    def make_grad_hook(name):
        def hook(grad):
            _b.timeline_end_activity(name)
        return hook

    for model in models:
        for _, leaf in _named_leaf_module(model):
            handles.append(leaf.register_forward_pre_hook(pre_forward))
            handles.append(leaf.register_forward_hook(post_forward))
    for p, name in parameter_names.items():
        if p.requires_grad:
            handles.append(p.register_hook(make_grad_hook(name)))
    return handles


class _CommonMixin:
    """Pieces shared by all wrappers: timeline switches, skip_synchronize, bookkeeping."""

    def _init_common(self, model, prefix=""):
        named, models = _check_named_parameters(self, model)
        self._models = models
        self._parameter_names = {v: prefix + k for k, v in sorted(named, key=lambda kv: kv[0])}
        self._name_parameters = {k: v for k, v in sorted(named, key=lambda kv: kv[0])}
        self._handles = {}
        self._synchronized = False
        self._should_synchronize = True
        self._timeline_hook_handles = []
        self._use_timeline = False
        self._error_encountered = False
        self._hook_handles = []
        if os.getenv("BLUEFOG_TIMELINE"):
            self.turn_on_timeline()

    def turn_on_timeline(self):
        self._timeline_hook_handles.extend(_register_timeline(self, self._models, self._parameter_names))
        self._use_timeline = True

    def turn_off_timeline(self):
        for h in self._timeline_hook_handles:
            h.remove()
        self._timeline_hook_handles.clear()
        self._use_timeline = False

    @contextmanager
    def skip_synchronize(self):
        """Inside this context ``step()`` does not synchronize; use after an explicit
        ``optimizer.synchronize()`` (e.g. to clip gradients in between)."""
        self._should_synchronize = False
        try:
            yield
        finally:
            self._should_synchronize = True

    def _warn_once(self, msg):
        if not self._error_encountered:
            warnings.warn(msg)
            self._error_encountered = True

    def _base_step(self, closure=None):
        return self._base_cls.step(self, closure)

    def _launch_data_comm(self, p):
        """Starts the parameter exchange configured by communication_type for one parameter."""
        name = self._parameter_names.get(p)
        ct = self._communication_type
        if ct == CommunicationType.allreduce:
            return _ops.allreduce_nonblocking(p.data, average=True, name=name)
        if ct == CommunicationType.neighbor_allreduce:
            return _ops.neighbor_allreduce_nonblocking(
                p.data, name=name, self_weight=self.self_weight, src_weights=self.src_weights,
                dst_weights=self.dst_weights, enable_topo_check=self.enable_topo_check)
        if ct == CommunicationType.hierarchical_neighbor_allreduce:
            return _ops.hierarchical_neighbor_allreduce_nonblocking(
                p.data, name=name, self_weight=self.self_weight,
                src_machine_weights=self.src_machine_weights,
                dst_machine_weights=self.dst_machine_weights, enable_topo_check=self.enable_topo_check)
        if ct == CommunicationType.empty:
            return None
        raise ValueError("Unsuppported CommunicationType encountered.")

    def _init_weight_knobs(self):
        self.self_weight = None
        self.src_weights = None
        self.dst_weights = None
        self.src_machine_weights = None
        self.dst_machine_weights = None
        self.enable_topo_check = False

    @property
    def communication_type(self):
        return self._communication_type

    @communication_type.setter
    def communication_type(self, value):
        assert isinstance(value, CommunicationType)
        self._communication_type = value


# --------------------------------------------------------------------------------------
# gradient allreduce
# --------------------------------------------------------------------------------------
class _DistributedOptimizer(_CommonMixin):
    """Averages gradients with allreduce as they are produced by backward."""

    def _bf_init(self, model, backward_passes_per_step=1):
        self._init_common(model)
        self._requires_update = set()
        self._backward_passes_per_step = backward_passes_per_step
        self._allreduce_delay = {p: backward_passes_per_step for p in self._parameter_names}
        if _b.size() > 1:
            for group in self.param_groups:
                for p in group["params"]:
                    if p.requires_grad:
                        if p.grad is None:
                            p.grad = torch.zeros_like(p.data)
                        self._requires_update.add(p)
                        self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook()))

    def _make_hook(self):
        def hook(p):
            if self._allreduce_delay[p] <= 0:
                self._warn_once(_WARN_BACKWARD)
            self._allreduce_delay[p] -= 1
            if self._allreduce_delay[p] == 0:
                self._handles[p] = self._allreduce_grad_async(p)
        return hook

    def _allreduce_grad_async(self, p):
        return _ops.allreduce_nonblocking(p.grad, average=True, name=self._parameter_names.get(p))

    def synchronize(self):
        for p in self._requires_update - set(self._handles.keys()):
            self._handles[p] = self._allreduce_grad_async(p)
        for p, handle in list(self._handles.items()):
            if handle is None:
                self._handles[p] = self._allreduce_grad_async(p)
        with torch.no_grad():
            for p, handle in self._handles.items():
                output = _ops.synchronize(handle)
                self._allreduce_delay[p] = self._backward_passes_per_step
                p.grad.copy_(output)
        self._handles.clear()
        self._synchronized = True

    def step(self, closure=None):
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn(_WARN_DOUBLE_SYNC)
            self.synchronize()
        self._synchronized = False
        return self._base_step(closure)

    def zero_grad(self, *args, **kwargs):
        if self._handles:
            raise AssertionError(
                "optimizer.zero_grad() was called after loss.backward() but before optimizer.step() "
                "or optimizer.synchronize(). This is prohibited as it can cause a race condition.")
        return self._base_cls.zero_grad(self, *args, **kwargs)


# --------------------------------------------------------------------------------------
# adapt-with-combine
# --------------------------------------------------------------------------------------
class _DistributedReduceOptimizer(_CommonMixin):
    """w+ = Combine(w) - lr * g(w); the exchange starts in a forward hook."""

    def _bf_init(self, model, communication_type, num_steps_per_communication=1):
        self._init_common(model)
        self._init_weight_knobs()
        assert isinstance(communication_type, CommunicationType)
        self._communication_type = communication_type
        self._num_steps_per_communication = num_steps_per_communication
        self._reduce_delay = {p: num_steps_per_communication for p in self._parameter_names}
        if _b.size() > 1:
            for m in self._models:
                self._hook_handles.append(m.register_forward_hook(self._make_hook()))

    def _make_hook(self):
        def hook(model, *unused):
            for parent_name, layer in _named_leaf_module(model):
                if not layer.training:
                    continue
                for name, p in layer.named_parameters(recurse=False):
                    full = (parent_name + "." + name) if parent_name else name
                    if self._name_parameters.get(full) is None or not p.requires_grad:
                        continue
                    if self._reduce_delay[p] <= 0:
                        self._warn_once(_WARN_STEPS)
                    self._reduce_delay[p] -= 1
                    if self._reduce_delay[p] == 0:
                        self._handles[p] = self._launch_data_comm(p)
        return hook

    def synchronize(self):
        with torch.no_grad():
            for p, handle in self._handles.items():
                if handle is not None:
                    p.data.copy_(_ops.synchronize(handle))
                self._reduce_delay[p] = self._num_steps_per_communication
        self._handles.clear()
        self._synchronized = True

    def step(self, closure=None):
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn(_WARN_DOUBLE_SYNC)
            self.synchronize()
        self._synchronized = False
        return self._base_step(closure)


# --------------------------------------------------------------------------------------
# adapt-then-combine
# --------------------------------------------------------------------------------------
class _DistributedAdaptThenCombineOptimizer(_CommonMixin):
    """w+ = Combine(w - lr * g(w)); update and exchange run per parameter inside backward."""

    def _bf_init(self, model, communication_type, backward_passes_per_step=1):
        self._init_common(model)
        self._init_weight_knobs()
        assert isinstance(communication_type, CommunicationType)
        self._communication_type = communication_type
        self._backward_passes_per_step = backward_passes_per_step
        self._reduce_delay = {p: backward_passes_per_step for p in self._parameter_names}
        self._step_func = None
        self._group_of = {p: g for g in self.param_groups for p in g["params"]}
        if _b.size() > 1:
            for group in self.param_groups:
                for p in group["params"]:
                    if p.requires_grad:
                        self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook()))

    def register_step_function(self, step_func):
        """Replaces the local update by ``step_func(self, parameter, gradient, parameter_group)``."""
        import types
        self._step_func = types.MethodType(step_func, self)

    def _local_step(self, p):
        """One optimizer update restricted to parameter ``p`` (any optimizer class works: the
        base class' own ``step`` is run with every other parameter hidden)."""
        if self._step_func is not None:
            with torch.no_grad():
                self._step_func(p, p.grad.data, self._group_of[p])
            return
        saved = [g["params"] for g in self.param_groups]
        try:
            for g in self.param_groups:
                g["params"] = [p] if any(q is p for q in g["params"]) else []
            self._base_cls.step(self)
        finally:
            for g, params in zip(self.param_groups, saved):
                g["params"] = params

    def _make_hook(self):
        def hook(p):
            if self._reduce_delay[p] <= 0:
                self._warn_once(_WARN_BACKWARD)
            self._reduce_delay[p] -= 1
            if self._reduce_delay[p] == 0:
                self._local_step(p)
                self._handles[p] = self._launch_data_comm(p)
        return hook

    def synchronize(self):
        with torch.no_grad():
            for p, handle in self._handles.items():
                if handle is not None:
                    p.data.copy_(_ops.synchronize(handle))
                self._reduce_delay[p] = self._backward_passes_per_step
        self._handles.clear()
        self._synchronized = True

    def step(self, closure=None):
        if _b.size() == 1:
            return self._base_step(closure)
        loss = closure() if closure is not None else None
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn(_WARN_DOUBLE_SYNC)
            self.synchronize()
        self._synchronized = False
        return loss

    def zero_grad(self, *args, **kwargs):
        if self._handles:
            raise AssertionError(
                "optimizer.zero_grad() was called after loss.backward() but before optimizer.step() "
                "or optimizer.synchronize(). This is prohibited as it can cause a race condition.")
        return self._base_cls.zero_grad(self, *args, **kwargs)


# --------------------------------------------------------------------------------------
# one-sided: win_put / pull-get
# --------------------------------------------------------------------------------------
class _WindowBucket:
    """Parameters that travel as one window: a flat tensor holding them back to back."""

    def __init__(self, name, params):
        self.name = name
        self.params = params
        self.offsets, n = [], 0
        for p in params:
            self.offsets.append(n)
            n += p.numel()
        self.numel = n
        self.flat = None
        self.handle = None

    def views(self, flat):
        return [flat[o:o + p.numel()].view(p.shape) for o, p in zip(self.offsets, self.params)]


def _window_bucket_bytes(bucket_bytes):
    if bucket_bytes is None:
        bucket_bytes = int(os.environ.get("BLUEFOG_B200_WINDOW_BUCKET_BYTES", 64 * 1024 * 1024))
    return int(bucket_bytes)


def _make_window_buckets(optimizer, parameter_names, prefix, bucket_bytes):
    """Groups the optimizer's trainable parameters, in order, into buckets of at most ``bucket_bytes`` with one
    dtype and device each.  ``bucket_bytes <= 0``: one bucket per parameter, named after it (the layout of the
    reference, bluefog/torch/optimizers.py:905-922: one window per parameter)."""
    buckets, cur, cur_bytes, key = [], [], 0, None

    def flush():
        nonlocal cur, cur_bytes
        if cur:
            buckets.append(_WindowBucket("%sbucket.%d" % (prefix, len(buckets)), cur))
        cur, cur_bytes = [], 0

    for group in optimizer.param_groups:
        for p in group["params"]:
            if parameter_names.get(p) is None:
                raise KeyError("Cannot find parameter in the _parameter_names dictionary")
            if not p.requires_grad:
                continue
            if bucket_bytes <= 0:
                buckets.append(_WindowBucket(parameter_names[p], [p]))
                continue
            nbytes = p.numel() * p.element_size()
            k = (p.dtype, p.device)
            if cur and (k != key or cur_bytes + nbytes > bucket_bytes):
                flush()
            key = k
            cur.append(p)
            cur_bytes += nbytes
    flush()
    return buckets


class _DistributedWinOptimizer(_CommonMixin):
    """Parameters are windows: a forward hook puts them to (or gets them from) the
    neighbors without waiting for anybody; ``step()`` folds what has arrived.  The parameters are packed into
    buckets (64 MiB by default) and every bucket is ONE window: a step costs one put/get kernel and one update
    kernel per bucket instead of one pair, one mutex and one handle per parameter."""

    def _bf_init(self, model, num_steps_per_communication, window_prefix, pull_style, bucket_bytes=None):
        if pull_style:
            self.src_weights = None   # controls win_get dynamically
        else:
            self.dst_weights = None   # controls win_put dynamically
        self.force_barrier = False
        self.window_prefix = window_prefix + "." if window_prefix is not None else ""
        self._init_common(model, prefix=self.window_prefix)
        self._pull_style = pull_style
        self._num_steps_per_communication = num_steps_per_communication
        self._bluefog_delay = {p: num_steps_per_communication for p in self._parameter_names}
        self._windows_registered = False
        self._owned_windows = {}
        self._bucket_bytes = _window_bucket_bytes(bucket_bytes)
        self._buckets = []
        self._bucket_of = {}
        if _b.size() > 1:
            self._register_window()
            for m in self._models:
                self._hook_handles.append(m.register_forward_hook(self._make_hook()))

    def __del__(self):
        try:
            self.unregister_window()
        except Exception:  # interpreter shutdown
            pass

    def _make_hook(self):
        def hook(model, *unused):
            ready = []
            for _, layer in _named_leaf_module(model):
                if not layer.training:
                    continue
                for _, p in layer.named_parameters(recurse=False):
                    if not p.requires_grad or p not in self._parameter_names:
                        continue
                    if self._bluefog_delay[p] <= 0:
                        self._warn_once(_WARN_STEPS)
                    self._bluefog_delay[p] -= 1
                    if self._bluefog_delay[p] == 0:
                        bk = self._bucket_of.get(p)
                        if bk is not None and bk not in ready:
                            ready.append(bk)
            for bk in ready:
                # a bucket goes out when every one of its parameters has been through its forward passes
                if bk.handle is not None or any(self._bluefog_delay[q] > 0 for q in bk.params):
                    continue
                if self._pull_style:
                    bk.handle = _win.win_get_nonblocking(name=bk.name, src_weights=self.src_weights, require_mutex=True)
                else:
                    bk.handle = _win.win_put_nonblocking(tensor=bk.flat.detach(), name=bk.name, dst_weights=self.dst_weights,
                                                         require_mutex=False)
                self._handles[bk.params[0]] = bk.handle
        return hook

    @torch.no_grad()
    def _register_window(self):
        if _b.size() <= 1 or self._windows_registered:
            return
        self._buckets = _make_window_buckets(self, self._parameter_names, self.window_prefix, self._bucket_bytes)
        for bk in self._buckets:
            if len(bk.params) == 1 and self._bucket_bytes <= 0:
                bk.flat = bk.params[0]                       # the parameter itself is the window tensor
                if not _win.win_create(bk.flat, bk.name):
                    raise ValueError("Cannot allocate window for the parameter {}".format(bk.name))
            else:
                flat = torch.cat([p.data.reshape(-1) for p in bk.params])
                if not _win.win_create(flat, bk.name):
                    raise ValueError("Cannot allocate window for the bucket {}".format(bk.name))
                bk.flat = flat                               # now aliases the window's memory
                for p, v in zip(bk.params, bk.views(flat)):
                    p.data = v
            for p in bk.params:
                self._bucket_of[p] = bk
            self._owned_windows[bk.name] = _win.window_serial(bk.name)
        self._windows_registered = True

    def unregister_window(self):
        """Frees the windows of this optimizer (collective)."""
        if not getattr(self, "_windows_registered", False) or not _b.is_initialized() or _b.size() <= 1:
            return
        for name, serial in sorted(self._owned_windows.items()):
            # only windows this optimizer created and that were not freed or replaced since
            if _win.window_serial(name) == serial:
                if not _win.win_free(name):
                    raise ValueError("Cannot free window for the parameter {}".format(name))
        self._owned_windows.clear()
        self._windows_registered = False

    def synchronize(self):
        with torch.no_grad():
            for bk in self._buckets:
                if bk.handle is None:
                    continue
                _win.win_wait(bk.handle)
                bk.handle = None
                for p in bk.params:
                    self._bluefog_delay[p] = self._num_steps_per_communication
                _win.win_update(name=bk.name, require_mutex=True)
        self._handles.clear()
        self._synchronized = True

    def step(self, closure=None):
        if self.force_barrier:
            _ops.barrier()
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn(_WARN_DOUBLE_SYNC)
            self.synchronize()
        self._synchronized = False
        return self._base_step(closure)


# --------------------------------------------------------------------------------------
# push-sum
# --------------------------------------------------------------------------------------
class _DistributedPushSumOptimizer(_CommonMixin):
    """Every bucket of parameters travels with a scalar weight: ``[x, 1]`` is split between this rank
    (``self_weight``) and its out-neighbors (``dst_weights``, accumulated one-sidedly), the
    arrived shares are collected, and the parameters become ``sum(x) / sum(weight)``."""

    def _bf_init(self, model, num_steps_per_communication, bucket_bytes=None):
        outdegree = len(_b.out_neighbor_ranks())
        self.dst_weights = {r: 1.0 / (outdegree + 1) for r in _b.out_neighbor_ranks()}
        self.self_weight = 1.0 / (outdegree + 1)
        self.force_barrier = True
        self._init_common(model)
        self._num_steps_per_communication = num_steps_per_communication
        self._pushsum_delay = {p: num_steps_per_communication for p in self._parameter_names}
        self._windows_registered = False
        self._owned_windows = {}
        self._bucket_bytes = _window_bucket_bytes(bucket_bytes)
        self._buckets = []
        self._bucket_of = {}
        if _b.size() > 1:
            self._register_window()
            for m in self._models:
                self._hook_handles.append(m.register_forward_hook(self._make_hook()))

    @torch.no_grad()
    def _register_window(self):
        self._buckets = _make_window_buckets(self, self._parameter_names, "", self._bucket_bytes)
        for bk in self._buckets:
            p0 = bk.params[0]
            # the window holds [parameters ..., weight]; the parameters themselves become views of one flat tensor
            # so that filling the window and reading the result back are single copies
            bk.pflat = torch.cat([p.data.reshape(-1) for p in bk.params])
            for p, v in zip(bk.params, bk.views(bk.pflat)):
                p.data = v
            ext = torch.cat((bk.pflat, torch.ones(1, dtype=p0.dtype, device=p0.device)), 0)
            if not _win.win_create(ext, bk.name, zero_init=True):
                raise ValueError("Cannot allocate window for the parameter {}".format(bk.name))
            bk.flat = ext
            for p in bk.params:
                self._bucket_of[p] = bk
            self._owned_windows[bk.name] = _win.window_serial(bk.name)
        self._windows_registered = True

    def unregister_window(self):
        if not getattr(self, "_windows_registered", False) or not _b.is_initialized() or _b.size() <= 1:
            return
        for name, serial in sorted(self._owned_windows.items()):
            if _win.window_serial(name) == serial:
                _win.win_free(name)
        self._owned_windows.clear()
        self._windows_registered = False

    def _make_hook(self):
        def hook(model, *unused):
            ready = []
            for _, layer in _named_leaf_module(model):
                if not layer.training:
                    continue
                for _, p in layer.named_parameters(recurse=False):
                    if not p.requires_grad or p not in self._parameter_names:
                        continue
                    if self._pushsum_delay[p] <= 0:
                        self._warn_once(_WARN_STEPS)
                    self._pushsum_delay[p] -= 1
                    if self._pushsum_delay[p] == 0:
                        bk = self._bucket_of.get(p)
                        if bk is not None and bk not in ready:
                            ready.append(bk)
            for bk in ready:
                if bk.handle is not None or any(self._pushsum_delay[q] > 0 for q in bk.params):
                    continue
                with torch.no_grad():
                    bk.flat[:-1].copy_(bk.pflat)
                    bk.flat[-1] = 1.0
                # The local share is scaled by self_weight after the shares have left.
                bk.handle = _win.win_accumulate_nonblocking(
                    tensor=bk.flat, name=bk.name, self_weight=self.self_weight,
                    dst_weights=self.dst_weights, require_mutex=True)
                self._handles[bk.params[0]] = bk.handle
        return hook

    def synchronize(self):
        with torch.no_grad():
            for bk in self._buckets:
                if bk.handle is None:
                    continue
                _win.win_wait(bk.handle)
                bk.handle = None
                for p in bk.params:
                    self._pushsum_delay[p] = self._num_steps_per_communication
                ext = _win.win_update_then_collect(name=bk.name)
                bk.pflat.copy_(ext[:-1] / ext[-1])
        self._handles.clear()
        self._synchronized = True

    def step(self, closure=None):
        if self.force_barrier:
            _ops.barrier()
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn(_WARN_DOUBLE_SYNC)
            self.synchronize()
        self._synchronized = False
        return self._base_step(closure)


# --------------------------------------------------------------------------------------
# factories
# --------------------------------------------------------------------------------------
def _wrap(optimizer, mixin, *args, **kwargs):
    """Builds ``class <OptName>(mixin, type(optimizer))`` and instantiates it on the same
    parameter groups, so that the result *is* an optimizer of the user's class."""
    base = optimizer.__class__
    cls = type(base.__name__, (mixin, base), {"_base_cls": base})
    obj = cls.__new__(cls)
    base.__init__(obj, optimizer.param_groups)
    # keep hyper-parameter defaults and any existing state of the wrapped instance
    obj.defaults = dict(optimizer.defaults)
    obj.state = optimizer.state
    obj._bf_init(*args, **kwargs)
    return obj


def DistributedPushSumOptimizer(optimizer, model, num_steps_per_communication=1, bucket_bytes=None):
    """Asynchronous push-sum over one-sided windows (column-stochastic weights; the graph
    only needs to be strongly connected). Knobs: ``dst_weights``, ``self_weight``, ``force_barrier``.
    ``bucket_bytes``: parameters per window (default 64 MiB, ``BLUEFOG_B200_WINDOW_BUCKET_BYTES``; 0 = one window
    per parameter as in the reference)."""
    return _wrap(optimizer, _DistributedPushSumOptimizer, model, num_steps_per_communication, bucket_bytes)


def DistributedPullGetOptimizer(optimizer, model, num_steps_per_communication=1, window_prefix=None, bucket_bytes=None):
    """Each step pulls the in-neighbors' parameters with win_get and averages. Knob: ``src_weights``."""
    return _wrap(optimizer, _DistributedWinOptimizer, model, num_steps_per_communication, window_prefix, True,
                 bucket_bytes)


def DistributedWinPutOptimizer(optimizer, model, num_steps_per_communication=1, window_prefix=None, bucket_bytes=None):
    """Each step pushes the parameters to the out-neighbors with win_put and averages what has
    arrived. Knob: ``dst_weights``."""
    return _wrap(optimizer, _DistributedWinOptimizer, model, num_steps_per_communication, window_prefix, False,
                 bucket_bytes)


def _maybe_fused(optimizer, model, style, communication_type, steps, fused, **fused_kwargs):
    from bluefog_b200.parallel import fused as _fused
    if fused is None:
        fused = _fused.supported(optimizer, model, communication_type) and os.environ.get("BLUEFOG_B200_FUSED", "1") != "0"
    if not fused:
        return None
    return _fused.build(optimizer, model, style, communication_type, steps, **fused_kwargs)


def DistributedAdaptWithCombineOptimizer(optimizer, model,
                                         communication_type=CommunicationType.neighbor_allreduce,
                                         num_steps_per_communication=1, fused=None, **fused_kwargs):
    """w+ = Combine(w) - lr * g(w). ``fused=None`` picks the bucket engine when it applies
    (CUDA parameters, SGD/Adam/AdamW/RMSprop/Adagrad/Adadelta, not hierarchical); ``fused_kwargs``: ``compute_dtype``,
    ``exchange_dtype``, ``bucket_bytes``."""
    obj = _maybe_fused(optimizer, model, "awc", communication_type, num_steps_per_communication, fused, **fused_kwargs)
    if obj is not None:
        return obj
    return _wrap(optimizer, _DistributedReduceOptimizer, model, communication_type, num_steps_per_communication)


def DistributedAdaptThenCombineOptimizer(optimizer, model,
                                         communication_type=CommunicationType.neighbor_allreduce,
                                         num_steps_per_communication=1, fused=None, **fused_kwargs):
    """w+ = Combine(w - lr * g(w))."""
    obj = _maybe_fused(optimizer, model, "atc", communication_type, num_steps_per_communication, fused, **fused_kwargs)
    if obj is not None:
        return obj
    return _wrap(optimizer, _DistributedAdaptThenCombineOptimizer, model, communication_type,
                 num_steps_per_communication)


def DistributedGradientAllreduceOptimizer(optimizer, model, num_steps_per_communication=1, fused=None,
                                          **fused_kwargs):
    """Averages gradients over all ranks before the local update (Horovod style)."""
    obj = _maybe_fused(optimizer, model, "grad", CommunicationType.allreduce, num_steps_per_communication, fused,
                       **fused_kwargs)
    if obj is not None:
        return obj
    return _wrap(optimizer, _DistributedOptimizer, model, num_steps_per_communication)


def DistributedAllreduceOptimizer(optimizer, model, num_steps_per_communication=1, **kw):
    """Older name: AWC with global parameter allreduce."""
    return DistributedAdaptWithCombineOptimizer(optimizer, model, CommunicationType.allreduce,
                                                num_steps_per_communication, **kw)


def DistributedNeighborAllreduceOptimizer(optimizer, model, num_steps_per_communication=1, **kw):
    """Older name: AWC with neighbor_allreduce of the parameters."""
    return DistributedAdaptWithCombineOptimizer(optimizer, model, CommunicationType.neighbor_allreduce,
                                                num_steps_per_communication, **kw)


def DistributedHierarchicalNeighborAllreduceOptimizer(optimizer, model, num_steps_per_communication=1, **kw):
    """Older name: AWC with hierarchical_neighbor_allreduce of the parameters."""
    return DistributedAdaptWithCombineOptimizer(optimizer, model, CommunicationType.hierarchical_neighbor_allreduce,
                                                num_steps_per_communication, **kw)
