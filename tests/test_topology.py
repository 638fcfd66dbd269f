"""Topology library: closed-form properties of the graphs and generators."""
import numpy as np
import networkx as nx
import pytest

from bluefog_b200.common import topology_util as tu


@pytest.mark.parametrize("n", [1, 2, 3, 4, 7, 8, 12, 16])
def test_static_graphs_are_row_and_column_stochastic(n):
    for g in (tu.ExponentialTwoGraph(n), tu.ExponentialGraph(n), tu.SymmetricExponentialGraph(n),
              tu.RingGraph(n), tu.FullyConnectedGraph(n), tu.MeshGrid2DGraph(n), tu.StarGraph(n)):
        w = nx.to_numpy_array(g)
        assert w.shape == (n, n)
        assert np.allclose(w.sum(axis=1), 1.0)
        assert np.allclose(w.sum(axis=0), 1.0)


def test_exponential_two_edges():
    g = tu.ExponentialTwoGraph(12)
    assert sorted(g.successors(0)) == [0, 1, 2, 4, 8]
    assert sorted(g.predecessors(0)) == [0, 4, 8, 10, 11]
    w = nx.to_numpy_array(g)
    assert np.isclose(w[0, 1], 0.2) and np.isclose(w[3, 3], 0.2)
    assert tu.IsRegularGraph(g)
    assert tu.IsTopologyEquivalent(tu.ExponentialGraph(12, base=2), g)
    assert not tu.IsTopologyEquivalent(tu.ExponentialGraph(12, base=3), g)
    assert not tu.IsTopologyEquivalent(g, None)


def test_ring_styles_and_weights():
    assert sorted(tu.RingGraph(5, 0).successors(0)) == [0, 1, 4]
    assert sorted(tu.RingGraph(5, 1).successors(0)) == [0, 4]
    assert sorted(tu.RingGraph(5, 2).successors(0)) == [0, 1]
    sw, nw = tu.GetRecvWeights(tu.RingGraph(5, 2), 2)
    assert sw == 0.5 and nw == {1: 0.5}
    sw, nw = tu.GetSendWeights(tu.RingGraph(5, 2), 2)
    assert sw == 0.5 and nw == {3: 0.5}


def test_meshgrid_hastings_weights():
    g = tu.MeshGrid2DGraph(6)          # 2 x 3
    w = nx.to_numpy_array(g)
    # corner 0 has 2 neighbours (3 with itself); edge node 1 has 3 (4 with itself)
    assert np.isclose(w[0, 1], 1 / 4) and np.isclose(w[0, 3], 1 / 3)
    assert np.isclose(w[0, 0], 1 - 1 / 4 - 1 / 3)
    assert w[0, 2] == 0 and np.allclose(w, w.T)
    with pytest.raises(AssertionError):
        tu.MeshGrid2DGraph(6, shape=(4, 2))


def test_star_and_symmetric_exponential():
    w = nx.to_numpy_array(tu.StarGraph(4, center_rank=1))
    assert np.isclose(w[0, 1], 0.25) and np.isclose(w[1, 0], 0.25) and w[0, 2] == 0
    g = tu.SymmetricExponentialGraph(12, base=4)
    assert sorted(g.successors(0)) == [0, 1, 4, 8, 11]


@pytest.mark.parametrize("n", [4, 8, 16])
def test_one_peer_exp2_send_recv_are_consistent_and_reach_exact_average(n):
    topo = tu.ExponentialTwoGraph(n)
    gens = [tu.GetDynamicOnePeerSendRecvRanks(topo, r) for r in range(n)]
    x = np.arange(n, dtype=np.float64)
    for k in range(int(np.log2(n))):
        rounds = [next(g) for g in gens]
        for r, (send, recv) in enumerate(rounds):
            assert send == [(r + 2 ** k) % n]
            assert recv == [(r - 2 ** k) % n]
        x = np.array([(x[r] + sum(x[s] for s in rounds[r][1])) / (len(rounds[r][1]) + 1) for r in range(n)])
    assert np.allclose(x, (n - 1) / 2)


def test_one_peer_on_irregular_graph_matches_transpose():
    topo = tu.StarGraph(5)
    gens = [tu.GetDynamicOnePeerSendRecvRanks(topo, r) for r in range(5)]
    for _ in range(6):
        rounds = [next(g) for g in gens]
        for r, (send, recv) in enumerate(rounds):
            for s in send:
                assert r in rounds[s][1]
            for s in recv:
                assert rounds[s][0] == [r]


def test_machine_and_inner_outer_generators():
    g = tu.GetExp2DynamicSendRecvMachineRanks(world_size=16, local_size=2, self_rank=5, local_rank=1)
    assert [next(g) for _ in range(4)] == [([3], [1]), ([4], [0]), ([6], [6]), ([3], [1])]
    for gen_fn in (tu.GetInnerOuterRingDynamicSendRecvRanks, tu.GetInnerOuterExpo2DynamicSendRecvRanks):
        world, local = 12, 4
        gens = [gen_fn(world, local, r) for r in range(world)]
        for _ in range(9):
            rounds = [next(g) for g in gens]
            for r, (send, recv) in enumerate(rounds):
                assert len(send) == 1 and len(recv) == 1
                assert rounds[send[0]][1] == [r], (gen_fn.__name__, r, rounds)
    with pytest.raises(AssertionError):
        next(tu.GetInnerOuterRingDynamicSendRecvRanks(8, 2, 0))



def test_every_public_name_of_the_reference_package_exists():
    """``import bluefog.torch as bf`` -> ``import bluefog_b200.torch as bf`` must not lose a name
    (list read from bluefog/torch/__init__.py:34-110 of the reference)."""
    import bluefog_b200.torch as bf
    names = """
    init shutdown size local_size rank local_rank machine_size machine_rank load_topology set_topology
    load_machine_topology set_machine_topology in_neighbor_ranks out_neighbor_ranks in_neighbor_machine_ranks
    out_neighbor_machine_ranks mpi_threads_supported unified_mpi_window_model_supported nccl_built is_homogeneous
    suspend resume check_extension
    allreduce allreduce_nonblocking allreduce_ allreduce_nonblocking_ allgather allgather_nonblocking
    broadcast broadcast_nonblocking broadcast_ broadcast_nonblocking_ neighbor_allgather neighbor_allgather_nonblocking
    neighbor_allreduce neighbor_allreduce_nonblocking hierarchical_neighbor_allreduce
    hierarchical_neighbor_allreduce_nonblocking poll synchronize wait barrier
    win_create win_free win_update win_update_then_collect win_put_nonblocking win_put win_get_nonblocking win_get
    win_accumulate_nonblocking win_accumulate win_wait win_poll win_mutex get_win_version
    get_current_created_window_names win_associated_p turn_on_win_ops_with_associated_p
    turn_off_win_ops_with_associated_p set_skip_negotiate_stage get_skip_negotiate_stage
    timeline_start_activity timeline_end_activity timeline_context
    neighbor_win_put neighbor_win_put_nonblocking neighbor_win_get neighbor_win_get_nonblocking
    neighbor_win_accumulate neighbor_win_accumulate_nonblocking
    broadcast_parameters allreduce_parameters broadcast_optimizer_state
    CommunicationType DistributedAdaptThenCombineOptimizer DistributedAdaptWithCombineOptimizer
    DistributedGradientAllreduceOptimizer DistributedWinPutOptimizer DistributedAllreduceOptimizer
    DistributedNeighborAllreduceOptimizer DistributedHierarchicalNeighborAllreduceOptimizer
    DistributedPullGetOptimizer DistributedPushSumOptimizer
    GetRecvWeights GetSendWeights IsRegularGraph IsTopologyEquivalent ExponentialGraph ExponentialTwoGraph
    SymmetricExponentialGraph MeshGrid2DGraph StarGraph RingGraph FullyConnectedGraph
    GetDynamicOnePeerSendRecvRanks GetExp2DynamicSendRecvMachineRanks GetInnerOuterRingDynamicSendRecvRanks
    GetInnerOuterExpo2DynamicSendRecvRanks InferSourceFromDestinationRanks InferDestinationFromSourceRanks
    pair_gossip pair_gossip_nonblocking
    """.split()
    missing = [n for n in names if not hasattr(bf, n)]
    assert not missing, missing
    bf.check_extension("bluefog_b200")          # the extension of this checkout is built


# ---- randomised properties (hypothesis) ---------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st  # noqa: E402

_STATIC = [tu.ExponentialTwoGraph, tu.ExponentialGraph, tu.SymmetricExponentialGraph, tu.MeshGrid2DGraph, tu.StarGraph,
           tu.RingGraph, tu.FullyConnectedGraph]


@settings(max_examples=60, deadline=None)
@given(n=st.integers(min_value=1, max_value=48), which=st.integers(min_value=0, max_value=len(_STATIC) - 1))
def test_any_static_graph_gives_every_rank_weights_that_sum_to_one(n, which):
    topo = _STATIC[which](n)
    assert topo.number_of_nodes() == n and tu.IsTopologyEquivalent(topo, topo)
    for r in range(n):
        self_w, src = tu.GetRecvWeights(topo, r)
        assert abs(self_w + sum(src.values()) - 1.0) < 1e-9, (which, n, r)
        assert r not in src and all(0 <= s < n for s in src)
        _, dst = tu.GetSendWeights(topo, r)
        # what r says it sends to d is what d says it receives from r
        for d in dst:
            assert r in tu.GetRecvWeights(topo, d)[1]


@settings(max_examples=40, deadline=None)
@given(n=st.integers(min_value=2, max_value=24), which=st.integers(min_value=0, max_value=len(_STATIC) - 1),
       rounds=st.integers(min_value=1, max_value=12))
def test_one_peer_schedule_is_a_matching_of_sends_and_receives_on_any_graph(n, which, rounds):
    topo = _STATIC[which](n)
    gens = [tu.GetDynamicOnePeerSendRecvRanks(topo, r) for r in range(n)]
    for _ in range(rounds):
        step = [next(g) for g in gens]
        for r, (send, recv) in enumerate(step):
            assert len(send) == 1 and topo.has_edge(r, send[0])
            assert r in step[send[0]][1]                      # my destination expects me
            for s in recv:
                assert step[s][0] == [r]                      # everyone I expect sends to me
        # averaging with these lists preserves the mean when every rank weighs what it has uniformly only on
        # regular patterns; what always holds is that nothing is sent twice or dropped:
        assert sum(len(recv) for _, recv in step) == n


@settings(max_examples=30, deadline=None)
@given(machines=st.integers(min_value=2, max_value=6), local=st.integers(min_value=3, max_value=6),
       rounds=st.integers(min_value=1, max_value=10))
def test_inner_outer_schedules_pair_every_send_with_a_receive(machines, local, rounds):
    world = machines * local
    for gen_fn in (tu.GetInnerOuterRingDynamicSendRecvRanks, tu.GetInnerOuterExpo2DynamicSendRecvRanks):
        gens = [gen_fn(world, local, r) for r in range(world)]
        for _ in range(rounds):
            step = [next(g) for g in gens]
            for r, (send, recv) in enumerate(step):
                assert len(send) == 1 and len(recv) == 1 and send[0] != r
                assert step[send[0]][1] == [r], (gen_fn.__name__, machines, local, r)
