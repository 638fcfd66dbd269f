"""Parameter and optimizer-state synchronisation helpers.

Same contracts as the reference (bluefog/torch/utility.py:26-216): ``broadcast_parameters``
and ``allreduce_parameters`` accept a ``state_dict()``, ``named_parameters()`` or a list of
(name, tensor) pairs and work in place; ``broadcast_optimizer_state`` makes every rank's
optimizer identical to the root's, including scalar hyper-parameters and step counters.
The scalars travel as one pickled blob over the control plane instead of one wrapped
tensor per scalar.
"""
import collections
import pickle
import warnings

import torch

import bluefog_b200.ops.collectives as _ops
from bluefog_b200.common.basics import get_basics

_b = get_basics()


def _named_tensors(params):
    if isinstance(params, dict):
        items = sorted(params.items())
    elif isinstance(params, list):
        items = list(params)
    else:
        items = list(params)
    if items and not isinstance(items[0], tuple):
        raise ValueError("invalid params of type: %s" % type(params))
    return [(n, t) for n, t in items if isinstance(t, torch.Tensor)]


def broadcast_parameters(params, root_rank):
    """Overwrites every tensor in ``params`` with the root rank's value."""
    handles = []
    for name, p in _named_tensors(params):
        t = p.data if isinstance(p, torch.nn.Parameter) else p
        if not t.is_contiguous():
            tmp = t.contiguous()
            _ops.broadcast_(tmp, root_rank, name="broadcast.param." + name)
            t.copy_(tmp)
            continue
        handles.append(_ops.broadcast_nonblocking_(t, root_rank, name="broadcast.param." + name))
    for h in handles:
        _ops.synchronize(h)
    _republish_fused()


def _republish_fused():
    """Parameters that a fused optimizer keeps in buckets were just written in place on every rank."""
    from bluefog_b200.parallel import fused
    fused.republish_live()


def allreduce_parameters(params):
    """Replaces every tensor in ``params`` by its average over all ranks."""
    handles = []
    for name, p in _named_tensors(params):
        t = p.data if isinstance(p, torch.nn.Parameter) else p
        if not t.is_floating_point():
            continue
        handles.append(_ops.allreduce_nonblocking_(t, average=True, name="allreduce.param." + name))
    for h in handles:
        _ops.synchronize(h)
    _republish_fused()


def _broadcast_object(obj, root_rank, name):
    """Pickles ``obj`` on the root and returns the root's object on every rank."""
    if _b.size() == 1:
        return obj
    payload = pickle.dumps(obj) if _b.rank() == root_rank else b""
    length = torch.tensor([len(payload)], dtype=torch.int64)
    length = _ops.broadcast(length, root_rank, name=name + ".len")
    buf = torch.zeros(int(length.item()), dtype=torch.uint8)
    if _b.rank() == root_rank:
        buf.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    buf = _ops.broadcast(buf, root_rank, name=name + ".data")
    return pickle.loads(buf.numpy().tobytes())


def broadcast_optimizer_state(optimizer, root_rank):
    """Makes ``optimizer.state_dict()`` on every rank equal to the root's."""
    if isinstance(optimizer, torch.optim.LBFGS):
        raise ValueError("cannot broadcast torch.optim.LBFGS state")
    state_dict = optimizer.state_dict()
    # A fresh optimizer has no state: create it with a zero-gradient step so that every rank
    # owns the same set of state tensors (same trick as the reference, utility.py:104-122).
    if len(state_dict["state"]) == 0:
        for group in optimizer.param_groups:
            for p in group["params"]:
                if p.requires_grad and p.grad is None:
                    p.grad = torch.zeros_like(p.data)
        saved = [p.detach().clone() for g in optimizer.param_groups for p in g["params"]]
        base = getattr(optimizer, "_base_cls", None)
        if base is not None:
            base.step(optimizer)
        else:
            optimizer.step()
        with torch.no_grad():
            for p, s in zip([p for g in optimizer.param_groups for p in g["params"]], saved):
                p.copy_(s)
        state_dict = optimizer.state_dict()
    if len(state_dict["state"]) == 0:
        # stateless optimizer (plain SGD): only hyper-parameters to share
        groups = _broadcast_object(state_dict["param_groups"], root_rank, "optimizer.groups")
        for g, src in zip(optimizer.param_groups, groups):
            for k, v in src.items():
                if k != "params":
                    g[k] = v
        return
    scalars = collections.OrderedDict()
    tensors = []
    for pid, st in sorted(state_dict["state"].items()):
        for key, value in sorted(st.items()):
            if isinstance(value, torch.Tensor) and value.numel() > 1:
                tensors.append(("optimizer.state.%s.%s" % (pid, key), value))
            else:
                scalars[(pid, key)] = value.item() if isinstance(value, torch.Tensor) else value
    groups = [{k: v for k, v in g.items() if k != "params"} for g in state_dict["param_groups"]]
    # (the groups of a fused optimizer also carry what it keeps beside its flat buffers: step counts and SGD's
    # first-step flag, under the key "bluefog_b200" of the first group)
    scalars, groups = _broadcast_object((scalars, groups), root_rank, "optimizer.scalars")
    broadcast_parameters(tensors, root_rank)
    for (pid, key), value in scalars.items():
        cur = state_dict["state"][pid].get(key)
        if isinstance(cur, torch.Tensor):
            cur.fill_(value)
        else:
            state_dict["state"][pid][key] = value
    for g, src in zip(state_dict["param_groups"], groups):
        g.update(src)
    optimizer.load_state_dict(state_dict)


def deprecated_function_arg(arg_name: str, fix: str):
    """Decorator that warns when a deprecated keyword argument is used."""
    def decorator(f):
        def wrapper(*args, **kwargs):
            if arg_name in kwargs:
                warnings.warn(f"{arg_name} is deprecated in {f.__name__}. {fix}", DeprecationWarning)
            return f(*args, **kwargs)
        wrapper.__name__ = f.__name__
        wrapper.__doc__ = f.__doc__
        return wrapper
    return decorator
