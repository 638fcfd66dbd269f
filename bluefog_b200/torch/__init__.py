"""``import bluefog_b200.torch as bf`` - the public API, name for name the surface of the
reference's ``bluefog.torch`` (bluefog/torch/__init__.py:34-110)."""

from bluefog_b200.common.basics import get_basics as _get_basics

_b = _get_basics()

init = _b.init
shutdown = _b.shutdown
size = _b.size
local_size = _b.local_size
rank = _b.rank
local_rank = _b.local_rank
machine_size = _b.machine_size
machine_rank = _b.machine_rank
load_topology = _b.load_topology
set_topology = _b.set_topology
load_machine_topology = _b.load_machine_topology
set_machine_topology = _b.set_machine_topology
in_neighbor_ranks = _b.in_neighbor_ranks
out_neighbor_ranks = _b.out_neighbor_ranks
in_neighbor_machine_ranks = _b.in_neighbor_machine_ranks
out_neighbor_machine_ranks = _b.out_neighbor_machine_ranks
mpi_threads_supported = _b.mpi_threads_supported
unified_mpi_window_model_supported = _b.unified_mpi_window_model_supported
nccl_built = _b.nccl_built
is_homogeneous = _b.is_homogeneous
is_topo_weighted = _b.is_topo_weighted
is_machine_topo_weighted = _b.is_machine_topo_weighted
suspend = _b.suspend
resume = _b.resume
set_skip_negotiate_stage = _b.set_skip_negotiate_stage
get_skip_negotiate_stage = _b.get_skip_negotiate_stage
timeline_start_activity = _b.timeline_start_activity
timeline_end_activity = _b.timeline_end_activity
timeline_context = _b.timeline_context
runtime_stats = _b.runtime_stats

from bluefog_b200.ops.collectives import (  # noqa: E402
    allreduce, allreduce_nonblocking, allreduce_, allreduce_nonblocking_,
    allgather, allgather_nonblocking,
    broadcast, broadcast_nonblocking, broadcast_, broadcast_nonblocking_,
    neighbor_allgather, neighbor_allgather_nonblocking,
    neighbor_allreduce, neighbor_allreduce_nonblocking,
    hierarchical_neighbor_allreduce, hierarchical_neighbor_allreduce_nonblocking,
    pair_gossip, pair_gossip_nonblocking,
    poll, synchronize, wait, barrier,
    symmetric_empty, is_symmetric,
)
from bluefog_b200.ops.windows import (  # noqa: E402
    win_create, win_free, win_update, win_update_then_collect,
    neighbor_win_put_nonblocking, neighbor_win_put,
    neighbor_win_get_nonblocking, neighbor_win_get,
    neighbor_win_accumulate_nonblocking, neighbor_win_accumulate,
    win_put_nonblocking, win_put, win_get_nonblocking, win_get,
    win_accumulate_nonblocking, win_accumulate,
    win_wait, win_poll, win_mutex, win_lock,
    get_win_version, get_current_created_window_names,
    win_associated_p, turn_on_win_ops_with_associated_p, turn_off_win_ops_with_associated_p,
)
from bluefog_b200.common.topology_util import (  # noqa: E402
    GetRecvWeights, GetSendWeights, IsRegularGraph, IsTopologyEquivalent,
    ExponentialTwoGraph, ExponentialGraph, FullyConnectedGraph, MeshGrid2DGraph,
    RingGraph, StarGraph, SymmetricExponentialGraph,
    GetDynamicOnePeerSendRecvRanks, GetExp2DynamicSendRecvMachineRanks,
    GetInnerOuterRingDynamicSendRecvRanks, GetInnerOuterExpo2DynamicSendRecvRanks,
)
from bluefog_b200.torch.topology_util import (  # noqa: E402
    InferSourceFromDestinationRanks, InferDestinationFromSourceRanks,
)
from bluefog_b200.parallel.utility import (  # noqa: E402
    broadcast_optimizer_state, broadcast_parameters, allreduce_parameters,
)
from bluefog_b200.parallel.optimizers import (  # noqa: E402
    CommunicationType,
    DistributedAdaptThenCombineOptimizer, DistributedAdaptWithCombineOptimizer,
    DistributedGradientAllreduceOptimizer, DistributedWinPutOptimizer,
    DistributedPullGetOptimizer, DistributedPushSumOptimizer,
    DistributedAllreduceOptimizer, DistributedNeighborAllreduceOptimizer,
    DistributedHierarchicalNeighborAllreduceOptimizer,
)
from bluefog_b200.utils.checkpoint import save_checkpoint, load_checkpoint  # noqa: E402
from bluefog_b200.common.util import check_extension  # noqa: E402
