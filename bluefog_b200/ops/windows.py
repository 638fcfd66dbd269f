"""One-sided window operations.

Semantics follow the reference (bluefog/torch/mpi_ops.py:1010-1503,
bluefog/torch/mpi_win_ops.cc:83-426): ``win_create`` registers a tensor and one receive
slot per in-neighbor (initialised with a copy of the tensor unless ``zero_init``);
``win_put``/``win_accumulate`` write ``dst_weights[d] * tensor`` into the caller's slot at
every destination and then scale the local tensor by ``self_weight``; ``win_get`` pulls the
in-neighbors' registered tensors into the local slots; ``win_update`` folds the slots into
the registered tensor (optionally zeroing them) and clears the version counters; every
transfer bumps the per-source version counter of the receiver, and with associated-p
turned on a scalar push-sum weight travels alongside the data.

Difference to the reference: the registered tensor is re-homed into shared memory (POSIX
shm for host tensors, CUDA-IPC device memory for CUDA tensors) so that neighbors can
reach it without this rank's help; ``win_create`` therefore rebinds ``tensor.data``.
"""

from contextlib import contextmanager
from typing import Dict, List, Optional

import torch

from bluefog_b200.common.basics import get_basics, logger
from bluefog_b200.common.topology_util import GetRecvWeights
from bluefog_b200.ops import collectives as _c

_b = get_basics()

_WIN_TYPES = (torch.float32, torch.float64, torch.int32, torch.int64, torch.bfloat16, torch.float16)

_win_map: Dict[str, torch.Tensor] = {}
# name -> serial number of the window currently registered under that name; lets an owner
# check that a window is still the one it created before freeing it
_win_serial: Dict[str, int] = {}
_serial_counter = [0]
_win_handle_map: Dict[int, tuple] = {}


def _in_neighbors_of(rank: int) -> List[int]:
    topo = _b.load_topology()
    return sorted(int(r) for r in topo.predecessors(rank) if r != rank)


def _slot_index_at(dst: int) -> int:
    """Index of this rank's slot inside rank ``dst``'s window."""
    return _in_neighbors_of(dst).index(_b.rank())


def win_create(tensor: torch.Tensor, name: str, zero_init: bool = False) -> bool:
    """Collectively creates window ``name`` from ``tensor`` (same shape and dtype on all ranks).
    After the call ``tensor`` aliases the window's memory."""
    _c._check_tensor(tensor, _WIN_TYPES, "win_create")
    if name in _win_map:
        return False
    topo = _b.load_topology()
    spec = _c._new_spec(_c.OP_WIN_CREATE, f"win_create.{name}")
    spec.win_name = name
    spec.input = tensor.detach()
    spec.zero_init = bool(zero_init)
    spec.in_neighbors = _b.in_neighbor_ranks()
    spec.num_slots = max(len([p for p in topo.predecessors(r) if p != r]) for r in range(_b.size()))
    handle = _b.native.enqueue(spec)
    try:
        _b.native.wait(handle)
    except (ValueError, RuntimeError) as exc:
        logger.error("win_create(%s) failed: %s", name, exc)
        return False
    view = _b.native.win_self_view(name)
    tensor.data = view
    _win_map[name] = tensor
    _serial_counter[0] += 1
    _win_serial[name] = _serial_counter[0]
    return True


def window_serial(name: str) -> int:
    """Serial number of the window registered as ``name`` (0 if there is none)."""
    return _win_serial.get(name, 0)


def win_free(name: Optional[str] = None) -> bool:
    """Collectively frees one window, or all windows when ``name`` is None."""
    if name is None:
        if not _win_map and _b.native.win_count() == 0:
            return True
        _win_map.clear()
        _win_serial.clear()
        target = ""
    else:
        if name not in _win_map:
            return False
        _win_map.pop(name)
        _win_serial.pop(name, None)
        target = name
    spec = _c._new_spec(_c.OP_WIN_FREE, f"win_free.{target if target else '__all__'}")
    spec.win_name = target
    handle = _b.native.enqueue(spec)
    try:
        _b.native.wait(handle)
    except (ValueError, RuntimeError) as exc:
        logger.error("win_free failed: %s", exc)
        return False
    return True


def win_update(name: str,
               self_weight: Optional[float] = None,
               neighbor_weights: Optional[Dict[int, float]] = None,
               reset: bool = False, clone: bool = False,
               require_mutex: bool = False) -> torch.Tensor:
    """``x = self_weight * x + sum_j neighbor_weights[j] * slot_j``; returns the registered tensor
    (or a fresh tensor when ``clone``). ``reset`` zeroes the slots that were combined."""
    if name not in _win_map:
        raise ValueError(f"{name} is not found in the registered window object.")
    tensor = _win_map[name]
    if neighbor_weights is not None and self_weight is not None:
        if not isinstance(neighbor_weights, dict):
            raise ValueError("Argument neighbor_weights has to be a dictionary map from the "
                             "(in-)neighbor rank to the weights.")
        if not isinstance(self_weight, float):
            raise ValueError("Argument self_weight has to be a float for self rank.")
        if not set(neighbor_weights.keys()).issubset(set(_b.in_neighbor_ranks())):
            raise ValueError("The key of weights should only contain the ranks that belong to "
                             " in-neighbors and self rank.")
    elif neighbor_weights is None and self_weight is None:
        if _b.is_topo_weighted():
            self_weight, neighbor_weights = GetRecvWeights(_b.load_topology(), _b.rank())
        else:
            w = 1.0 / (len(_b.in_neighbor_ranks()) + 1)
            self_weight, neighbor_weights = w, {r: w for r in _b.in_neighbor_ranks()}
    else:
        raise ValueError("Arguments self_weight and neighbor_weights have to be presented at "
                         "the same time")
    ranks = sorted(int(r) for r in neighbor_weights)
    out = torch.empty_like(tensor) if clone else None
    try:
        _b.native.win_update(name, out, float(self_weight), ranks,
                             [float(neighbor_weights[r]) for r in ranks], bool(reset), bool(require_mutex))
    except (ValueError, RuntimeError) as exc:
        raise RuntimeError("Cannot apply win_update on " + name) from exc
    return out if clone else tensor


def win_update_then_collect(name: str, require_mutex: bool = True) -> torch.Tensor:
    """Sum of the tensor and all slots, then the slots are zeroed (used by push-sum)."""
    weights = {r: 1.0 for r in _b.in_neighbor_ranks()}
    return win_update(name, 1.0, weights, reset=True, require_mutex=require_mutex)


def _transfer(op: int, tensor: torch.Tensor, name: str, self_weight, dst_weights, require_mutex, accumulate):
    _c._check_tensor(tensor, _WIN_TYPES, "win_put")
    if name not in _win_map:
        raise ValueError(f"{name} is not found in the registered window object.")
    dst_weights = {r: 1.0 for r in _b.out_neighbor_ranks()} if dst_weights is None else dst_weights
    if self_weight is None:
        self_weight = 1.0
    if not set(dst_weights.keys()).issubset(set(_b.out_neighbor_ranks())):
        raise ValueError("The key of dst_weights should only contain ranks that "
                         " belong to out-neighbors (self-rank is not allowed).")
    kind = "win_accumulate" if accumulate else "win_put"
    spec = _c._new_spec(op, _c._full_name(f"{kind}.{name}", None))
    spec.negotiate = False
    spec.win_name = name
    spec.input = tensor
    spec.self_weight = float(self_weight)
    spec.dst_ranks = sorted(int(r) for r in dst_weights)
    spec.dst_weights = [float(dst_weights[r]) for r in spec.dst_ranks]
    spec.slot_index = [_slot_index_at(d) for d in spec.dst_ranks]
    spec.require_mutex = bool(require_mutex)
    spec.accumulate = bool(accumulate)
    handle = _b.native.enqueue(spec)
    _win_handle_map[handle] = (name, tensor)
    return handle


def neighbor_win_put_nonblocking(tensor: torch.Tensor, name: str,
                                 self_weight: Optional[float] = None,
                                 dst_weights: Optional[Dict[int, float]] = None,
                                 require_mutex: bool = False) -> int:
    """Writes ``dst_weights[d] * tensor`` into this rank's slot at every destination ``d`` (all
    out-neighbors by default), then scales ``tensor`` by ``self_weight`` in place."""
    return _transfer(_c.OP_WIN_PUT, tensor, name, self_weight, dst_weights, require_mutex, False)


def neighbor_win_put(tensor, name, self_weight=None, dst_weights=None, require_mutex=False) -> bool:
    return win_wait(neighbor_win_put_nonblocking(tensor, name, self_weight, dst_weights, require_mutex))


def neighbor_win_accumulate_nonblocking(tensor: torch.Tensor, name: str,
                                        self_weight: Optional[float] = None,
                                        dst_weights: Optional[Dict[int, float]] = None,
                                        require_mutex: bool = False) -> int:
    """Like ``win_put`` but adds into the destination slots instead of overwriting them."""
    return _transfer(_c.OP_WIN_ACCUMULATE, tensor, name, self_weight, dst_weights, require_mutex, True)


def neighbor_win_accumulate(tensor, name, self_weight=None, dst_weights=None, require_mutex=False) -> bool:
    return win_wait(neighbor_win_accumulate_nonblocking(tensor, name, self_weight, dst_weights, require_mutex))


def neighbor_win_get_nonblocking(name: str, src_weights: Optional[Dict[int, float]] = None,
                                 require_mutex: bool = False) -> int:
    """Copies ``src_weights[s] *`` (the registered tensor of in-neighbor ``s``) into the local slot of ``s``."""
    if name not in _win_map:
        raise ValueError(f"{name} is not found in the registered window object.")
    src_weights = {r: 1.0 for r in _b.in_neighbor_ranks()} if src_weights is None else src_weights
    if not set(src_weights.keys()).issubset(set(_b.in_neighbor_ranks())):
        raise ValueError("The key of src_weights should only containranks that "
                         " belong to in-neighbors.")
    spec = _c._new_spec(_c.OP_WIN_GET, _c._full_name(f"win_get.{name}", None))
    spec.negotiate = False
    spec.win_name = name
    spec.src_ranks = sorted(int(r) for r in src_weights)
    spec.src_weights = [float(src_weights[r]) for r in spec.src_ranks]
    mine = _b.in_neighbor_ranks()
    spec.slot_index = [mine.index(s) for s in spec.src_ranks]
    spec.require_mutex = bool(require_mutex)
    handle = _b.native.enqueue(spec)
    _win_handle_map[handle] = (name, None)
    return handle


def neighbor_win_get(name: str, src_weights: Optional[Dict[int, float]] = None,
                     require_mutex: bool = False) -> bool:
    return win_wait(neighbor_win_get_nonblocking(name, src_weights, require_mutex))


win_accumulate = neighbor_win_accumulate
win_get = neighbor_win_get
win_put = neighbor_win_put
win_accumulate_nonblocking = neighbor_win_accumulate_nonblocking
win_get_nonblocking = neighbor_win_get_nonblocking
win_put_nonblocking = neighbor_win_put_nonblocking


def win_poll(handle: int) -> bool:
    return bool(_b.native.poll(handle))


def win_wait(handle: int) -> bool:
    if handle not in _win_handle_map:
        logger.warning("Win wait is called but the handle is not found in the _win_handle_map.")
        return False
    try:
        _b.native.wait(handle)
    finally:
        _win_handle_map.pop(handle)
    return True


def get_current_created_window_names() -> List[str]:
    return sorted(_win_map.keys())


def get_win_version(name: str) -> Dict[int, int]:
    """Transfers received from each in-neighbor since the last ``win_update``."""
    versions = _b.native.win_versions(name)
    return {r: int(versions[r]) for r in _b.in_neighbor_ranks()}


@contextmanager
def win_lock(name: str):
    """Kept for API parity (an MPI access epoch in the reference): windows here are coherent
    shared memory, so entering and leaving the context only validates the name."""
    if name not in _win_map:
        raise ValueError(f"{name} is not found in the registered window object.")
    yield


@contextmanager
def win_mutex(name: str, for_self: bool = False, ranks: Optional[List[int]] = None):
    """Holds the mutexes that guard this rank's slots at ``ranks`` (default: out-neighbors), or,
    with ``for_self``, the mutexes of this rank's own slots for ``ranks``."""
    _ranks = _b.out_neighbor_ranks() if ranks is None else list(ranks)
    _b.native.win_mutex_acquire(name, _ranks, bool(for_self))
    try:
        yield
    finally:
        _b.native.win_mutex_release(name, _ranks, bool(for_self))


def win_associated_p(name: str) -> float:
    """The push-sum weight associated with window ``name`` on this rank (starts at 1.0)."""
    return float(_b.native.win_get_p(name))


def turn_on_win_ops_with_associated_p():
    _b.native.win_set_with_p(True)


def turn_off_win_ops_with_associated_p():
    _b.native.win_set_with_p(False)
