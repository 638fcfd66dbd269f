"""Process-level state: init/shutdown, rank and size queries, virtual topology.

Behaviour follows the reference's ``BlueFogBasics`` (bluefog/common/basics.py:37-568):
``init`` installs ``ExponentialGraph(size)`` unless a topology function is given,
``set_topology`` refuses (returns False) while windows exist, is a no-op for an equivalent
topology, and keeps sorted neighbor lists without the self loop; the machine topology only
lives in Python.  What differs is the plumbing: ranks are separate processes started by
``bfrun``/``torchrun`` (RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT), they find each
other through a TCP key-value store and then talk over the native TCP mesh and, on GPUs,
CUDA-IPC peer memory; there is no MPI.
"""

import atexit
import contextlib
import datetime
import logging
import os
import socket
from typing import Callable, List, Optional

import networkx
import torch

from bluefog_b200.common import topology_util

logger = logging.getLogger("bluefog")
logger.setLevel(logging.INFO)
if not logger.handlers:
    _ch = logging.StreamHandler()
    _ch.setLevel(logging.INFO)
    _ch.setFormatter(logging.Formatter("%(asctime)-15s %(levelname)s  %(message)s"))
    logger.addHandler(_ch)
    logger.propagate = False


def _load_native():
    try:
        from bluefog_b200 import _C  # noqa: WPS433
    except ImportError as exc:  # pragma: no cover - build problem
        raise ImportError(
            "bluefog_b200._C is not built. Run `python setup.py build_ext --inplace` "
            "in the repository root (needs nvcc and PyTorch headers).") from exc
    return _C


class BlueFogBasics:
    """Wrapper holding rank/size, topologies and the handle to the native runtime."""

    def __init__(self):
        self._C = None
        self._topology = None
        self._machine_topology = None
        self._is_topo_weighted = False
        self._is_machine_topo_weighted = False
        self._rank = 0
        self._size = 1
        self._local_rank = 0
        self._local_size = 1
        self._device = -1
        self._store = None
        self._in_neighbors: List[int] = []
        self._out_neighbors: List[int] = []
        self._atexit_registered = False

    # ------------------------------------------------------------------ lifecycle
    @property
    def native(self):
        if self._C is None:
            self._C = _load_native()
        return self._C

    def is_initialized(self) -> bool:
        return self._C is not None and self._C.is_initialized()

    def _require_init(self):
        if not self.is_initialized():
            raise ValueError("BlueFog has not been initialized; use bf.init().")

    def init(self, topology_fn: Optional[Callable[[int], networkx.DiGraph]] = None,
             is_weighted: bool = False):
        """Start the runtime of this rank and install the default topology.

        Args:
          topology_fn: callable ``size -> DiGraph``; default ``ExponentialGraph``.
          is_weighted: use the edge weights of the topology for the neighbor averages
            instead of uniform ``1/(in_degree+1)``.
        """
        C = self.native
        if C.is_initialized():
            return
        env = os.environ
        rank = int(env.get("BLUEFOG_RANK", env.get("RANK", "0")))
        size = int(env.get("BLUEFOG_SIZE", env.get("WORLD_SIZE", "1")))
        local_rank = int(env.get("BLUEFOG_LOCAL_RANK", env.get("LOCAL_RANK", str(rank))))
        local_size = int(env.get("BLUEFOG_LOCAL_SIZE", env.get("LOCAL_WORLD_SIZE", str(size))))
        fake = env.get("BLUEFOG_NODES_PER_MACHINE")
        if fake:  # pretend that every `fake` consecutive ranks share a machine
            local_size = int(fake)
            if size % local_size != 0:
                raise ValueError("BLUEFOG_NODES_PER_MACHINE must divide the number of ranks.")
            local_rank = rank % local_size
        bind = env.get("BLUEFOG_BIND_ADDR", "127.0.0.1")
        port = C.listen(bind)
        endpoints = [f"{bind}:{port}"]
        if size > 1:
            addr = env.get("MASTER_ADDR", "127.0.0.1")
            mport = int(env.get("MASTER_PORT", "29500"))
            use_agent = env.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
            timeout = datetime.timedelta(seconds=float(env.get("BLUEFOG_START_TIMEOUT", "600")))
            import torch.distributed as dist
            store = dist.TCPStore(addr, mport, size, rank == 0 and not use_agent, timeout,
                                  wait_for_workers=False, multi_tenant=True)
            self._store = dist.PrefixStore(f"bfb200/{env.get('TORCHELASTIC_RESTART_COUNT', '0')}", store)
            host = bind if bind != "0.0.0.0" else socket.gethostbyname(socket.gethostname())
            self._store.set(f"ep/{rank}", f"{host}:{port}")
            endpoints = [self._store.get(f"ep/{r}").decode() for r in range(size)]
        device = -1
        if torch.cuda.is_available() and env.get("BLUEFOG_B200_FORCE_CPU", "0") != "1":
            device = local_rank % torch.cuda.device_count()
            torch.cuda.set_device(device)
            torch.cuda.current_stream(device)  # creates the context on the calling thread
        C.init(rank, size, local_rank, local_size, endpoints, device)
        self._rank, self._size = rank, size
        self._local_rank, self._local_size = local_rank, local_size
        self._device = device
        self._topology = None
        self._machine_topology = None
        topo = topology_fn(size) if topology_fn else topology_util.ExponentialGraph(size)
        self.set_topology(topo, is_weighted)
        if not self._atexit_registered:
            atexit.register(self.shutdown)
            self._atexit_registered = True

    def shutdown(self) -> None:
        if self._C is not None and self._C.is_initialized():
            self._C.shutdown()
        self._topology = None
        self._machine_topology = None
        self._store = None

    # ------------------------------------------------------------------ identity
    def size(self) -> int:
        self._require_init()
        return self._size

    def local_size(self) -> int:
        self._require_init()
        return self._local_size

    def rank(self) -> int:
        self._require_init()
        return self._rank

    def local_rank(self) -> int:
        self._require_init()
        return self._local_rank

    def machine_rank(self) -> int:
        self._require_init()
        assert self.is_homogeneous(), "Only supported in homogeneous environment"
        return self._rank // self._local_size

    def machine_size(self) -> int:
        self._require_init()
        assert self.is_homogeneous(), "Only supported in homogeneous environment"
        return self._size // self._local_size

    def device(self) -> int:
        """CUDA device index of this rank, -1 on a CPU-only rank."""
        return self._device

    def is_homogeneous(self) -> bool:
        self._require_init()
        return self._size % self._local_size == 0

    def nccl_built(self) -> bool:
        """True when the GPU data path is available (kept under the reference's name; the
        path is peer-memory kernels, NCCL is only used by the baseline benchmark)."""
        return torch.cuda.is_available()

    def mpi_threads_supported(self) -> bool:
        """Kept for API parity: the TCP mesh is safe to use from the runtime's threads."""
        self._require_init()
        return True

    def unified_mpi_window_model_supported(self) -> bool:
        """Windows are coherent shared memory (host) or peer-mapped device memory."""
        self._require_init()
        return True

    # ------------------------------------------------------------------ topology
    def is_topo_weighted(self) -> bool:
        return self._is_topo_weighted

    def is_machine_topo_weighted(self) -> bool:
        return self._is_machine_topo_weighted

    def load_topology(self) -> networkx.DiGraph:
        return self._topology

    def load_machine_topology(self) -> networkx.DiGraph:
        return self._machine_topology

    def in_neighbor_ranks(self) -> List[int]:
        if self._topology is None:
            return []
        return list(self._in_neighbors)

    def out_neighbor_ranks(self) -> List[int]:
        if self._topology is None:
            return []
        return list(self._out_neighbors)

    def in_neighbor_machine_ranks(self) -> List[int]:
        if self._machine_topology is None:
            return []
        m = self.machine_rank()
        return sorted(r for r in self._machine_topology.predecessors(m) if r != m)

    def out_neighbor_machine_ranks(self) -> List[int]:
        if self._machine_topology is None:
            return []
        m = self.machine_rank()
        return sorted(r for r in self._machine_topology.successors(m) if r != m)

    def set_topology(self, topology: Optional[networkx.DiGraph] = None,
                     is_weighted: bool = False) -> bool:
        """Install a new virtual topology. Returns False (and keeps the old one) when the
        graph is invalid or a window exists; True otherwise."""
        self._require_init()
        if topology is None:
            topology = topology_util.ExponentialGraph(self._size)
            is_weighted = False
        if not isinstance(topology, networkx.DiGraph):
            raise TypeError("topology must be a networkx.DiGraph object.")
        if topology.number_of_nodes() != self._size:
            raise TypeError("topology must be a networkx.DiGraph object with same number of nodes as bf.size().")
        if topology_util.IsTopologyEquivalent(topology, self._topology):
            if self._is_topo_weighted != is_weighted:
                self._is_topo_weighted = is_weighted
            return True
        if self.native.win_count() > 0:
            logger.error("Cannot set the topology while windows exist; call bf.win_free() first.")
            return False
        self._topology = topology
        self._is_topo_weighted = is_weighted
        r = self._rank
        self._in_neighbors = sorted(int(x) for x in topology.predecessors(r) if x != r)
        self._out_neighbors = sorted(int(x) for x in topology.successors(r) if x != r)
        return True

    def set_machine_topology(self, topology: Optional[networkx.DiGraph],
                             is_weighted: bool = False) -> bool:
        self._require_init()
        if topology is None:
            raise ValueError("Machine topology shall not be None.")
        if not isinstance(topology, networkx.DiGraph):
            raise TypeError("Machine topology must be a networkx.DiGraph object.")
        if not self.is_homogeneous():
            raise RuntimeError("Beefog should be run under homogeneous environment to set machine topology.")
        if topology.number_of_nodes() != self.machine_size():
            raise TypeError("topology must be a networkx.DiGraph object with same number of nodes as "
                            "bf.machine_size().")
        if topology_util.IsTopologyEquivalent(topology, self._machine_topology):
            self._is_machine_topo_weighted = is_weighted
            return True
        self._machine_topology = topology
        self._is_machine_topo_weighted = is_weighted
        return True

    # ------------------------------------------------------------------ runtime toggles
    def set_skip_negotiate_stage(self, value: bool) -> None:
        """Skip the coordinator round trip: operations run in local program order. All ranks
        must then issue the same collectives in the same order."""
        self._require_init()
        self.native.set_skip_negotiate_stage(bool(value))

    def get_skip_negotiate_stage(self) -> bool:
        self._require_init()
        return self.native.get_skip_negotiate_stage()

    def suspend(self):
        """Pause the background thread (interactive sessions)."""
        self._require_init()
        self.native.suspend()

    def resume(self):
        self._require_init()
        self.native.resume()

    # ------------------------------------------------------------------ timeline
    def timeline_start_activity(self, tensor_name: str, activity_name: str) -> bool:
        if self._C is None:
            return False
        return self._C.timeline_start_activity(tensor_name, activity_name)

    def timeline_end_activity(self, tensor_name: str) -> bool:
        if self._C is None:
            return False
        return self._C.timeline_end_activity(tensor_name)

    @contextlib.contextmanager
    def timeline_context(self, tensor_name: str, activity_name: str):
        self.timeline_start_activity(tensor_name, activity_name)
        try:
            yield
        finally:
            self.timeline_end_activity(tensor_name)

    def runtime_stats(self) -> dict:
        """Counters of this rank since ``init()``: operations enqueued per type (``enqueued.NEIGHBOR_ALLREDUCE``, ...),
        ``input_bytes``, ``issued_on_calling_thread`` (operations that skipped the background loop),
        ``responses_executed`` and ``tensors_in_fused_responses`` (negotiated path), ``operations_failed`` and
        ``kernel_launches`` of this library's kernels.  The reference has no counterpart (its observability is the
        log and the timeline)."""
        self._require_init()
        return dict(self.native.runtime_stats())


_basics = BlueFogBasics()


def get_basics() -> BlueFogBasics:
    return _basics
