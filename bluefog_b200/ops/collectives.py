"""Collective and neighbor operations (blocking, ``_nonblocking`` and in-place forms).

Argument rules, defaults and results follow the reference's Python API
(bluefog/torch/mpi_ops.py:82-1005): ``neighbor_allreduce`` computes
``self_weight * x + sum_j src_weights[j] * (dst_weight_{j->me} * x_j)``; ``self_weight`` and
``src_weights`` come together or not at all; giving ``dst_weights`` switches to a dynamic
topology and then requires them; a list of destinations means weights of 1.0.  Every op
is turned into one generic ``OpSpec`` (who reads whom, with which coefficients) that the
native runtime executes over TCP for host tensors and with peer-memory kernels for CUDA
tensors, so that allreduce, pair gossip and the hierarchical variant are all instances of
the same weighted pull-combine.
"""

import itertools
import os
from typing import Dict, List, Optional, Union

import numpy as np
import torch

from bluefog_b200.common.basics import get_basics, logger
from bluefog_b200.common.topology_util import GetRecvWeights

_b = get_basics()

OP_ALLREDUCE, OP_ALLGATHER, OP_BROADCAST, OP_NEIGHBOR_ALLREDUCE, OP_NEIGHBOR_ALLGATHER = 0, 1, 2, 3, 4
OP_WIN_CREATE, OP_WIN_FREE, OP_WIN_PUT, OP_WIN_GET, OP_WIN_ACCUMULATE, OP_BARRIER, OP_PAIR_GOSSIP = 5, 6, 7, 8, 9, 10, 11

# handle -> (input, output, finish_fn): keeps tensors alive until synchronize()
_handle_map = {}
_noname_counter = itertools.count()

_REDUCE_TYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
_ALLREDUCE_TYPES = _REDUCE_TYPES + (torch.int32, torch.int64)
_COPY_TYPES_CPU = _ALLREDUCE_TYPES + (torch.uint8, torch.int8, torch.int16, torch.bool)


def _ops_on_cpu() -> bool:
    return os.environ.get("BLUEFOG_OPS_ON_CPU", "0") not in ("0", "", "false", "False")


def _check_tensor(tensor: torch.Tensor, allowed, op: str):
    if not isinstance(tensor, torch.Tensor):
        raise ValueError(f"{op} expects a torch.Tensor.")
    if tensor.dtype not in allowed:
        raise ValueError(f"Tensor type {tensor.type()} is not supported by {op}.")
    if not tensor.is_contiguous():
        raise ValueError(f"{op} requires a contiguous tensor; call .contiguous() first.")


def _full_name(prefix: str, name: Optional[str]) -> str:
    if name:
        return f"{prefix}.{name}"
    return f"{prefix}.noname.{next(_noname_counter)}"


def _submit(spec, tensor, output, finish=None) -> int:
    handle = _b.native.enqueue(spec)
    _handle_map[handle] = (tensor, output, finish)
    return handle


def _new_spec(op: int, name: str):
    _b._require_init()
    spec = _b.native.OpSpec()
    spec.type = op
    spec.name = name
    return spec


def _stage(tensor: torch.Tensor):
    """Optionally move a CUDA tensor to the host (BLUEFOG_OPS_ON_CPU=1)."""
    if tensor.is_cuda and _ops_on_cpu():
        return tensor.detach().cpu(), tensor.device
    return tensor, None


# --------------------------------------------------------------------------------------
# allreduce
# --------------------------------------------------------------------------------------
def _allreduce_nonblocking(tensor, output, average, is_hierarchical_local, name):
    _check_tensor(tensor, _ALLREDUCE_TYPES, "allreduce")
    if is_hierarchical_local:
        base = _b.machine_rank() * _b.local_size()
        group = list(range(base, base + _b.local_size()))
    else:
        group = list(range(_b.size()))
    others = [r for r in group if r != _b.rank()]
    spec = _new_spec(OP_ALLREDUCE, _full_name("allreduce", name))
    staged, dev = _stage(tensor)
    out = output if dev is None else torch.empty_like(staged)
    spec.input, spec.output = staged, out
    spec.src_ranks, spec.src_weights = others, [1.0] * len(others)
    spec.dst_ranks, spec.dst_weights = others, [1.0] * len(others)
    spec.self_weight = 1.0
    spec.post_scale = 1.0 / len(group) if (average and tensor.is_floating_point()) else 1.0
    spec.is_hierarchical = bool(is_hierarchical_local)
    finish = None if dev is None else (lambda: output.copy_(out))
    return _submit(spec, tensor, output, finish)


def allreduce_nonblocking(tensor: torch.Tensor, average: bool = True,
                          name: Optional[str] = None, is_hierarchical_local: bool = False) -> int:
    """Starts an average (or sum) of ``tensor`` over all ranks, or over the ranks of this
    machine when ``is_hierarchical_local``. The input is not modified. Returns a handle."""
    output = torch.empty_like(tensor)
    return _allreduce_nonblocking(tensor, output, average, is_hierarchical_local, name)


def allreduce(tensor: torch.Tensor, average: bool = True,
              name: Optional[str] = None, is_hierarchical_local: bool = False) -> torch.Tensor:
    return synchronize(allreduce_nonblocking(tensor, average, name, is_hierarchical_local))


def allreduce_nonblocking_(tensor: torch.Tensor, average: bool = True,
                           name: Optional[str] = None, is_hierarchical_local: bool = False) -> int:
    """In-place variant: the result overwrites ``tensor``."""
    return _allreduce_nonblocking(tensor, tensor, average, is_hierarchical_local, name)


def allreduce_(tensor: torch.Tensor, average: bool = True,
               name: Optional[str] = None, is_hierarchical_local: bool = False) -> torch.Tensor:
    return synchronize(allreduce_nonblocking_(tensor, average, name, is_hierarchical_local))


# --------------------------------------------------------------------------------------
# broadcast
# --------------------------------------------------------------------------------------
def _check_rank(rank_: int):
    if not isinstance(rank_, (int, np.integer)) or rank_ < 0 or rank_ >= _b.size():
        raise ValueError(f"Rank should be an integer between 0 and {_b.size() - 1}, got {rank_}.")


def _broadcast_nonblocking(tensor, output, root_rank, name):
    allowed = _ALLREDUCE_TYPES if tensor.is_cuda else _COPY_TYPES_CPU
    _check_tensor(tensor, allowed, "broadcast")
    _check_rank(root_rank)
    spec = _new_spec(OP_BROADCAST, _full_name("broadcast", name))
    staged, dev = _stage(output)
    spec.output = staged
    spec.root_rank = int(root_rank)
    others = [r for r in range(_b.size()) if r != root_rank]
    if _b.rank() == root_rank:
        spec.dst_ranks, spec.dst_weights = others, [1.0] * len(others)
    else:
        spec.src_ranks, spec.src_weights = [int(root_rank)], [1.0]
    finish = None if dev is None else (lambda: output.copy_(staged))
    return _submit(spec, tensor, output, finish)


def broadcast_nonblocking(tensor: torch.Tensor, root_rank: int, name: Optional[str] = None) -> int:
    """Every rank receives the root's value in a new tensor; the input is not modified."""
    output = tensor.clone()
    return _broadcast_nonblocking(tensor, output, root_rank, name)


def broadcast(tensor: torch.Tensor, root_rank: int, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(broadcast_nonblocking(tensor, root_rank, name))


def broadcast_nonblocking_(tensor, root_rank, name=None) -> int:
    return _broadcast_nonblocking(tensor, tensor, root_rank, name)


def broadcast_(tensor, root_rank, name=None) -> torch.Tensor:
    return synchronize(broadcast_nonblocking_(tensor, root_rank, name))


# --------------------------------------------------------------------------------------
# allgather / neighbor_allgather
# --------------------------------------------------------------------------------------
def allgather_nonblocking(tensor: torch.Tensor, name: Optional[str] = None) -> int:
    """Concatenates the tensors of all ranks along dimension 0 (first dimensions may differ)."""
    allowed = _ALLREDUCE_TYPES if tensor.is_cuda else _COPY_TYPES_CPU
    _check_tensor(tensor, allowed, "allgather")
    if tensor.dim() == 0:
        raise ValueError("allgather requires a tensor with at least one dimension.")
    spec = _new_spec(OP_ALLGATHER, _full_name("allgather", name))
    staged, dev = _stage(tensor)
    out = staged.new_empty((0,) + tuple(staged.shape[1:]))
    spec.input, spec.output = staged, out
    others = [r for r in range(_b.size()) if r != _b.rank()]
    spec.src_ranks, spec.src_weights = others, [1.0] * len(others)
    spec.dst_ranks, spec.dst_weights = others, [1.0] * len(others)
    holder = {}
    finish = None if dev is None else (lambda: holder.setdefault("out", out.to(dev)))
    handle = _submit(spec, tensor, out, finish)
    if dev is not None:
        _handle_map[handle] = (tensor, holder, finish)
    return handle


def allgather(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(allgather_nonblocking(tensor, name))


def neighbor_allgather_nonblocking(tensor: torch.Tensor, *,
                                   src_ranks: Optional[List[int]] = None,
                                   dst_ranks: Optional[List[int]] = None,
                                   enable_topo_check: bool = True,
                                   name: Optional[str] = None) -> int:
    """Concatenates the in-neighbors' tensors (self excluded) in sorted in-neighbor order, or
    in the order of ``src_ranks`` when a dynamic pattern is given."""
    allowed = _ALLREDUCE_TYPES if tensor.is_cuda else _COPY_TYPES_CPU
    _check_tensor(tensor, allowed, "neighbor_allgather")
    if tensor.dim() == 0:
        raise ValueError("neighbor_allgather requires a tensor with at least one dimension.")
    if (src_ranks is None) != (dst_ranks is None):
        raise ValueError("Arguments src_ranks and dst_ranks should be presented at the same time.")
    dynamic = src_ranks is not None
    if dynamic:
        if len(set(src_ranks)) != len(src_ranks) or len(set(dst_ranks)) != len(dst_ranks):
            raise ValueError("src_ranks and dst_ranks should only contain unique ranks.")
        for r in list(src_ranks) + list(dst_ranks):
            _check_rank(r)
            if r == _b.rank():
                raise ValueError("src_ranks and dst_ranks should not contain the self rank.")
    else:
        src_ranks, dst_ranks = _b.in_neighbor_ranks(), _b.out_neighbor_ranks()
    spec = _new_spec(OP_NEIGHBOR_ALLGATHER, _full_name("neighbor.allgather", name))
    staged, dev = _stage(tensor)
    out = staged.new_empty((0,) + tuple(staged.shape[1:]))
    spec.input, spec.output = staged, out
    spec.src_ranks, spec.src_weights = [int(r) for r in src_ranks], [1.0] * len(src_ranks)
    spec.dst_ranks, spec.dst_weights = [int(r) for r in dst_ranks], [1.0] * len(dst_ranks)
    spec.enable_topo_check = bool(enable_topo_check and dynamic)
    holder = {}
    finish = None if dev is None else (lambda: holder.setdefault("out", out.to(dev)))
    handle = _submit(spec, tensor, out, finish)
    if dev is not None:
        _handle_map[handle] = (tensor, holder, finish)
    return handle


def neighbor_allgather(tensor: torch.Tensor, *, src_ranks=None, dst_ranks=None,
                       enable_topo_check: bool = True, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(neighbor_allgather_nonblocking(
        tensor, src_ranks=src_ranks, dst_ranks=dst_ranks, enable_topo_check=enable_topo_check, name=name))


# --------------------------------------------------------------------------------------
# neighbor_allreduce
# --------------------------------------------------------------------------------------
def _resolve_neighbor_weights(self_weight, src_weights, dst_weights):
    """Applies the argument rules and returns
    (self_weight, src_ranks, src_w, dst_ranks, dst_w, use_dst_weight, dynamic)."""
    if dst_weights is None:
        dynamic, use_dst = False, False
        dst_map = {r: 1.0 for r in _b.out_neighbor_ranks()}
    else:
        if len(set(dst_weights)) != len(dst_weights):
            raise ValueError("Argument dst_weights should only contain the unique ranks.")
        if self_weight is None or src_weights is None:
            raise ValueError("Arguments self_weight and src_weights should be presented if "
                             "enabling dynamic topology.")
        dynamic = True
        if isinstance(dst_weights, list):
            dst_map, use_dst = {int(d): 1.0 for d in dst_weights}, False
        else:
            dst_map = {int(k): float(v) for k, v in dst_weights.items()}
            # same tolerance as numpy.allclose(values, 1.0), without the array round trip on the hot path
            use_dst = any(abs(v - 1.0) > 1e-8 + 1e-5 for v in dst_map.values())
    if self_weight is None and src_weights is None:
        if _b.is_topo_weighted():
            self_weight, src_map = GetRecvWeights(_b.load_topology(), _b.rank())
        else:
            w = 1.0 / (len(_b.in_neighbor_ranks()) + 1)
            self_weight, src_map = w, {r: w for r in _b.in_neighbor_ranks()}
    elif self_weight is not None and src_weights is not None:
        if not isinstance(src_weights, dict):
            raise ValueError("Argument src_weights has to be a dictionary map from the "
                             "(in-)neighbor rank to the weights.")
        if not isinstance(self_weight, float):
            raise ValueError("Argument self_weight has to be a float for self rank.")
        if not dynamic and not set(src_weights.keys()).issubset(set(_b.in_neighbor_ranks())):
            raise ValueError("The key of weights should only contain the ranks that belong to "
                             " in-neighbors and self rank.")
        src_map = {int(k): float(v) for k, v in src_weights.items()}
        if not dynamic:
            # Static topology: every in-neighbor publishes for this rank, so every one of them is
            # read (with weight 0 when it was left out) to keep the reader accounting balanced.
            src_map = {r: src_map.get(r, 0.0) for r in _b.in_neighbor_ranks()}
    else:
        raise ValueError("Arguments self_weight and src_weights have to be presented at "
                         "the same time")
    for r in list(src_map) + list(dst_map):
        _check_rank(r)
        if r == _b.rank():
            raise ValueError("Neighbor lists should not contain the self rank.")
    src_ranks = sorted(src_map)
    dst_ranks = sorted(dst_map)
    return (float(self_weight), src_ranks, [src_map[r] for r in src_ranks], dst_ranks,
            [dst_map[r] for r in dst_ranks], use_dst, dynamic)


def _neighbor_allreduce_nonblocking(tensor, output, self_weight, src_weights, dst_weights,
                                    enable_topo_check, name):
    _check_tensor(tensor, _REDUCE_TYPES, "neighbor_allreduce")
    sw, src_ranks, src_w, dst_ranks, dst_w, use_dst, dynamic = _resolve_neighbor_weights(
        self_weight, src_weights, dst_weights)
    spec = _new_spec(OP_NEIGHBOR_ALLREDUCE, _full_name("neighbor.allreduce", name))
    staged, dev = _stage(tensor)
    out = output if dev is None else torch.empty_like(staged)
    spec.input, spec.output = staged, out
    spec.self_weight = sw
    spec.src_ranks, spec.src_weights = src_ranks, src_w
    spec.dst_ranks, spec.dst_weights = dst_ranks, dst_w
    spec.use_dst_weight = use_dst
    spec.enable_topo_check = bool(enable_topo_check and dynamic)
    finish = None if dev is None else (lambda: output.copy_(out))
    return _submit(spec, tensor, output, finish)


def neighbor_allreduce_nonblocking(tensor: torch.Tensor, *,
                                   self_weight: Optional[float] = None,
                                   src_weights: Optional[Dict[int, float]] = None,
                                   dst_weights: Optional[Union[Dict[int, float], List[int]]] = None,
                                   enable_topo_check: bool = True,
                                   name: Optional[str] = None,
                                   neighbor_weights=None, send_neighbors=None) -> int:
    """Starts a weighted average with the in-neighbors. With no weights the static topology
    decides (its edge weights if the topology was set as weighted, uniform otherwise)."""
    if neighbor_weights is not None:  # deprecated spelling
        logger.warning("neighbor_weights is deprecated. Use src_weights instead")
        src_weights = neighbor_weights
    if send_neighbors is not None:
        logger.warning("send_neighbors is deprecated. Use dst_weights instead")
        dst_weights = send_neighbors
    output = torch.empty_like(tensor)
    return _neighbor_allreduce_nonblocking(tensor, output, self_weight, src_weights, dst_weights,
                                           enable_topo_check, name)


def neighbor_allreduce(tensor: torch.Tensor, *,
                       self_weight: Optional[float] = None,
                       src_weights: Optional[Dict[int, float]] = None,
                       dst_weights: Optional[Union[Dict[int, float], List[int]]] = None,
                       enable_topo_check: bool = True,
                       name: Optional[str] = None,
                       neighbor_weights=None, send_neighbors=None) -> torch.Tensor:
    """``self_weight * x + sum_j src_weights[j] * dst_weight_{j->me} * x_j`` over the in-neighbors."""
    return synchronize(neighbor_allreduce_nonblocking(
        tensor, self_weight=self_weight, src_weights=src_weights, dst_weights=dst_weights,
        enable_topo_check=enable_topo_check, name=name, neighbor_weights=neighbor_weights,
        send_neighbors=send_neighbors))


# --------------------------------------------------------------------------------------
# registered tensors
# --------------------------------------------------------------------------------------
def symmetric_empty(*shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """An uninitialised CUDA tensor in symmetric memory: memory of this rank's GPU that is mapped into every other
    rank of the machine.  ``neighbor_allreduce`` publishes such a tensor in place - it raises a flag instead of copying
    the tensor into its staging arena, and the neighbors pull it from where it is - and returns once they have.

    Collective: every rank calls it, in the same order, with the same shape and dtype; every rank then passes its tensor
    (or the same slice of it) to an operation, or none does.  The memory is released at ``shutdown()``.  Without a GPU
    (CPU ranks, a single process) the result is an ordinary ``torch.empty`` and nothing changes.
    The reference has no counterpart: its GPU path hands every tensor to NCCL or copies it into a fusion buffer first
    (bluefog/common/nccl_controller.cc:1013-1204)."""
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    native = _b.native
    if (native is None or not hasattr(native, "symmetric_alloc") or not torch.cuda.is_available()
            or not _b.is_initialized() or _b.size() == 1 or _b.device() < 0):
        device = "cuda" if torch.cuda.is_available() and _b.is_initialized() and _b.device() >= 0 else "cpu"
        return torch.empty(*shape, dtype=dtype, device=device)
    numel = int(np.prod(shape)) if len(shape) else 1
    nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 16)
    raw = native.symmetric_alloc(nbytes)
    return raw[:numel * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)


def is_symmetric(tensor: torch.Tensor) -> bool:
    """Whether ``tensor`` lies in memory of ``symmetric_empty`` (and starts on a 16-byte boundary), i.e. whether
    ``neighbor_allreduce`` will publish it in place."""
    native = _b.native
    return bool(native is not None and hasattr(native, "is_symmetric") and tensor.is_cuda and _b.is_initialized()
                and native.is_symmetric(tensor))


# --------------------------------------------------------------------------------------
# hierarchical_neighbor_allreduce
# --------------------------------------------------------------------------------------
def _resolve_machine_weights(self_weight, src_machine_weights, dst_machine_weights):
    """Argument rules of the hierarchical operation (reference bluefog/torch/mpi_ops.py:790-864): all three given,
    or none (then the machine topology supplies them).  Returns (self_weight, {machine: weight}, {machine: weight})."""
    if self_weight is None and src_machine_weights is None and dst_machine_weights is None:
        topo = _b.load_machine_topology()
        if topo is None:
            raise RuntimeError("Machine topology must be set before the use of hierarchical "
                               "neighbor allreduce")
        if _b.is_machine_topo_weighted():
            self_weight, src_machine_weights = GetRecvWeights(topo, _b.machine_rank())
        else:
            w = 1.0 / (len(_b.in_neighbor_machine_ranks()) + 1)
            self_weight = w
            src_machine_weights = {m: w for m in _b.in_neighbor_machine_ranks()}
        dst_map = {m: 1.0 for m in _b.out_neighbor_machine_ranks()}
    elif self_weight is not None and src_machine_weights is not None and dst_machine_weights is not None:
        if not isinstance(src_machine_weights, dict):
            raise ValueError("Argument src_machine_weights has to be a dictionary map from the "
                             "(in-)neighbor rank to the weights.")
        if not isinstance(self_weight, float):
            raise ValueError("Argument self_weight has to be a float for self rank.")
        if len(set(dst_machine_weights)) != len(dst_machine_weights):
            raise ValueError("Argument dst_machine_weights should only contain the unique ranks.")
        dst_map = {int(d): 1.0 for d in dst_machine_weights} if isinstance(dst_machine_weights, list) \
            else {int(k): float(v) for k, v in dst_machine_weights.items()}
    else:
        raise ValueError("Arguments self_weight, src_machine_weights, dst_machine_weights have to "
                         "be presented at the same time.")
    my_machine = _b.machine_rank()
    for m in list(src_machine_weights) + list(dst_map):
        if m < 0 or m >= _b.machine_size() or m == my_machine:
            raise ValueError("Machine ids must be other machines between 0 and machine_size-1.")
    return float(self_weight), {int(m): float(w) for m, w in src_machine_weights.items()}, dst_map


def hierarchical_neighbor_allreduce_nonblocking(
        tensor: torch.Tensor, *,
        self_weight: Optional[float] = None,
        src_machine_weights: Optional[Dict[int, float]] = None,
        dst_machine_weights: Optional[Union[Dict[int, float], List[int]]] = None,
        enable_topo_check: bool = False,
        name: Optional[str] = None,
        neighbor_machine_weights=None, send_neighbor_machines=None) -> int:
    """Machines are the nodes of the topology: the result on every rank of machine M is
    ``self_weight * mean_M(x) + sum_m w_m * mean_m(x)``.  On an NVSwitch box every rank pulls
    the contributing ranks' tensors directly, so the local allreduce, the leader exchange
    and the local broadcast of the reference collapse into one weighted pull."""
    if neighbor_machine_weights is not None:
        src_machine_weights = neighbor_machine_weights
    if send_neighbor_machines is not None:
        dst_machine_weights = send_neighbor_machines
    assert _b.is_homogeneous(), \
        "hierarchical_neighbor_allreduce should be used under homogeneous environment only"
    assert _b.local_size() > 1, "If local size is 1, you should use neighbor allreduce directly."
    _check_tensor(tensor, _REDUCE_TYPES, "hierarchical_neighbor_allreduce")
    self_weight, src_machine_weights, dst_map = _resolve_machine_weights(self_weight, src_machine_weights,
                                                                         dst_machine_weights)
    L, me, my_machine = _b.local_size(), _b.rank(), _b.machine_rank()
    src, dst = {}, {}
    for r in range(my_machine * L, (my_machine + 1) * L):
        if r != me:
            src[r] = float(self_weight) / L
            dst[r] = 1.0
    for m, w in src_machine_weights.items():
        for r in range(int(m) * L, (int(m) + 1) * L):
            src[r] = float(w) / L
    for m, w in dst_map.items():
        for r in range(m * L, (m + 1) * L):
            dst[r] = w
    use_dst = any(abs(v - 1.0) > 1e-8 + 1e-5 for v in dst_map.values())
    spec = _new_spec(OP_NEIGHBOR_ALLREDUCE, _full_name("neighbor.allreduce", name))
    buf, dev = _stage(tensor.detach().clone())
    output = torch.empty_like(tensor)
    out = output if dev is None else torch.empty_like(buf)
    spec.input, spec.output = buf, out
    spec.self_weight = float(self_weight) / L
    spec.src_ranks = sorted(src)
    spec.src_weights = [src[r] for r in spec.src_ranks]
    spec.dst_ranks = sorted(dst)
    spec.dst_weights = [dst[r] for r in spec.dst_ranks]
    spec.use_dst_weight = use_dst
    spec.enable_topo_check = bool(enable_topo_check)
    spec.is_hierarchical = True
    finish = None if dev is None else (lambda: output.copy_(out))
    return _submit(spec, buf, output, finish)


def hierarchical_neighbor_allreduce(tensor: torch.Tensor, *,
                                    self_weight: Optional[float] = None,
                                    src_machine_weights: Optional[Dict[int, float]] = None,
                                    dst_machine_weights: Optional[Union[Dict[int, float], List[int]]] = None,
                                    enable_topo_check: bool = False,
                                    name: Optional[str] = None,
                                    neighbor_machine_weights=None, send_neighbor_machines=None) -> torch.Tensor:
    return synchronize(hierarchical_neighbor_allreduce_nonblocking(
        tensor, self_weight=self_weight, src_machine_weights=src_machine_weights,
        dst_machine_weights=dst_machine_weights, enable_topo_check=enable_topo_check, name=name,
        neighbor_machine_weights=neighbor_machine_weights, send_neighbor_machines=send_neighbor_machines))


# --------------------------------------------------------------------------------------
# pair_gossip
# --------------------------------------------------------------------------------------
def pair_gossip_nonblocking(tensor: torch.Tensor, target_rank: int, self_weight: float = None,
                            pair_weight: float = None, name: str = None) -> int:
    """Averages (or weighted-averages) with exactly one other rank, which must call
    ``pair_gossip`` towards this rank at the same time."""
    _check_tensor(tensor, _REDUCE_TYPES, "pair_gossip")
    _check_rank(target_rank)
    if target_rank == _b.rank():
        raise ValueError("pair_gossip target must be another rank.")
    if pair_weight is None and self_weight is None:
        self_weight, pair_weight = 0.5, 0.5
    elif pair_weight is None or self_weight is None:
        raise ValueError("self_weight and pair_weight have to be set at same time.")
    spec = _new_spec(OP_PAIR_GOSSIP, _full_name("pair.gossip", name))
    spec.negotiate = False  # only two ranks take part
    # CUDA tensors travel over a two-rank peer-memory channel that the partners set up between themselves
    staged, dev = _stage(tensor)
    output = torch.empty_like(tensor)
    out = output if dev is None else torch.empty_like(staged)
    spec.input, spec.output = staged, out
    spec.self_weight = float(self_weight)
    spec.src_ranks, spec.src_weights = [int(target_rank)], [float(pair_weight)]
    spec.dst_ranks, spec.dst_weights = [int(target_rank)], [1.0]
    finish = None if dev is None else (lambda: output.copy_(out))
    return _submit(spec, tensor, output, finish)


def pair_gossip(tensor: torch.Tensor, target_rank: int, self_weight: float = None,
                pair_weight: float = None, name: str = None) -> torch.Tensor:
    return synchronize(pair_gossip_nonblocking(tensor, target_rank, self_weight, pair_weight, name))


# --------------------------------------------------------------------------------------
# handles
# --------------------------------------------------------------------------------------
def poll(handle: int) -> bool:
    """True once the operation behind ``handle`` has finished; ``synchronize`` then returns at once."""
    return bool(_b.native.poll(handle))


def synchronize(handle: int) -> torch.Tensor:
    """Waits for the operation and returns its output tensor."""
    if handle not in _handle_map:
        raise ValueError("Cannot find handle to synchronize")
    try:
        _b.native.wait(handle)
    finally:
        _, output, finish = _handle_map.pop(handle)
    if finish is not None:
        finish()
    if isinstance(output, dict):
        return output["out"]
    return output


def wait(handle: int) -> torch.Tensor:
    return synchronize(handle)


def barrier():
    """Returns once every rank has reached the barrier."""
    _b._require_init()
    if _b.get_skip_negotiate_stage():
        _b.native.barrier_now()
        return
    spec = _new_spec(OP_BARRIER, "barrier")
    handle = _b.native.enqueue(spec)
    _b.native.wait(handle)
