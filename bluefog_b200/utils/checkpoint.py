"""Checkpoint save / resume.

The file format is the one the reference's ResNet example writes
(examples/pytorch_resnet.py:384-391): ``{"model": model.state_dict(), "optimizer":
optimizer.state_dict()}`` stored with ``torch.save`` by rank 0.  When the optimizer keeps
fp32 master weights beside a bf16 compute copy, the fp32 values are exported under the
usual parameter names.  Resume = load on every rank (or on rank 0) followed by the two
broadcasts, which is how the reference restores consistency at start-up.  What the reference
does not checkpoint (iteration counter of a dynamic schedule, push-sum weights) goes into the
optional ``extra`` entry.
"""
import os

import torch

from bluefog_b200.common.basics import get_basics

_b = get_basics()


def _model_state(model, optimizer):
    state = model.state_dict()
    export = getattr(optimizer, "master_parameters", None)
    if export is not None:
        masters = export()
        for name in list(state.keys()):
            if name in masters:
                state[name] = masters[name].detach().clone().reshape(state[name].shape)
    return {k: v.detach().cpu() if isinstance(v, torch.Tensor) else v for k, v in state.items()}


def save_checkpoint(path, model, optimizer, extra=None, all_ranks=False):
    """Writes ``path`` on rank 0 (or ``path.format(rank=...)`` on every rank with ``all_ranks``)."""
    if not all_ranks and _b.is_initialized() and _b.rank() != 0:
        return None
    if all_ranks and _b.is_initialized():
        path = path.format(rank=_b.rank())
    payload = {"model": _model_state(model, optimizer), "optimizer": optimizer.state_dict()}
    if extra is not None:
        payload["extra"] = extra
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)
    return path


def load_checkpoint(path, model, optimizer=None, root_rank=0, broadcast=True, map_location="cpu"):
    """Loads ``path`` where it exists and makes all ranks consistent with ``root_rank``: parameters (fp32 masters of
    a fused optimizer), optimizer state, the model's buffers (BatchNorm running statistics and counters) and the
    ``extra`` entry, which is returned on every rank (None when the file has none).  Collective: every rank calls it."""
    from bluefog_b200.parallel.utility import _broadcast_object, broadcast_optimizer_state, broadcast_parameters
    extra = None
    have = os.path.exists(path)
    fused = getattr(optimizer, "load_master_parameters", None) is not None
    if have:
        payload = torch.load(path, map_location=map_location, weights_only=False)
        if fused:
            # no publish here: this branch runs only where the file is, the peer-visible copies advance in lockstep
            optimizer.load_master_parameters(payload["model"], publish=False)
            other = {k: v for k, v in payload["model"].items() if k not in dict(model.named_parameters())}
            model.load_state_dict(other, strict=False)
        else:
            model.load_state_dict(payload["model"])
        if optimizer is not None and "optimizer" in payload:
            optimizer.load_state_dict(payload["optimizer"])
        extra = payload.get("extra")
    distributed = broadcast and _b.is_initialized() and _b.size() > 1
    if distributed:
        if fused:
            optimizer.broadcast_from(root_rank)           # masters, optimizer state, step counters; republishes
            buffers = dict(model.named_buffers())
            if buffers:
                broadcast_parameters(buffers, root_rank)
        else:
            broadcast_parameters(model.state_dict(), root_rank)
            if optimizer is not None:
                broadcast_optimizer_state(optimizer, root_rank)
        extra = _broadcast_object(extra, root_rank, "checkpoint.extra")
    elif fused:
        optimizer.republish()
    return extra
