"""Virtual topologies and dynamic send/recv schedules.

Every static constructor returns a weighted ``networkx.DiGraph`` whose adjacency
matrix ``W`` uses the convention ``W[i, j]`` = weight that rank ``i`` *sends to*
rank ``j`` (so column ``j`` holds the weights rank ``j`` applies when it combines
what it received).  The graphs, their weights and the generator contracts match
the behaviour documented for the reference in
``bluefog/common/topology_util.py:23-554``; the construction here is by explicit
edge enumeration rather than by rolled circulant rows.
"""

from typing import Dict, Iterator, List, Optional, Tuple

import math

import networkx as nx
import numpy as np

__all__ = [
    "IsTopologyEquivalent", "GetRecvWeights", "GetSendWeights",
    "ExponentialTwoGraph", "ExponentialGraph", "SymmetricExponentialGraph",
    "MeshGrid2DGraph", "StarGraph", "RingGraph", "FullyConnectedGraph",
    "IsRegularGraph", "GetDynamicOnePeerSendRecvRanks",
    "GetExp2DynamicSendRecvMachineRanks", "GetInnerOuterRingDynamicSendRecvRanks",
    "GetInnerOuterExpo2DynamicSendRecvRanks", "isPowerOf",
]


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def _graph_from_matrix(weights: np.ndarray) -> nx.DiGraph:
    return nx.from_numpy_array(np.asarray(weights, dtype=np.float64), create_using=nx.DiGraph)


def _circulant(size: int, offsets: List[int]) -> nx.DiGraph:
    """Graph where rank i sends to (i + d) % size for every d in ``offsets``
    (0 = self loop), all edges weighted 1/len(offsets)."""
    offsets = sorted(set(o % size for o in offsets))
    w = 1.0 / len(offsets)
    mat = np.zeros((size, size))
    for i in range(size):
        for d in offsets:
            mat[i, (i + d) % size] = w
    return _graph_from_matrix(mat)


def isPowerOf(x: int, base: int) -> bool:
    assert isinstance(base, int), "Base has to be a integer."
    assert base > 1, "Base has to a interger larger than 1."
    assert x > 0
    p = 1
    while p < x:
        p *= base
    return p == x


def IsTopologyEquivalent(topo1: nx.DiGraph, topo2: nx.DiGraph) -> bool:
    """Two topologies are equivalent when their weighted adjacency matrices are
    identical (no isomorphism test)."""
    if topo1 is None or topo2 is None:
        return False
    if topo1.number_of_nodes() != topo2.number_of_nodes():
        return False
    if topo1.number_of_edges() != topo2.number_of_edges():
        return False
    a1 = nx.to_numpy_array(topo1)
    a2 = nx.to_numpy_array(topo2)
    return bool((a1 == a2).all())


def GetRecvWeights(topo: nx.DiGraph, rank: int) -> Tuple[float, Dict[int, float]]:
    """(self_weight, {in-neighbor: weight}) used by ``rank`` when it combines."""
    w = nx.to_numpy_array(topo)
    self_weight = 0.0
    neighbor_weights = {}
    for src in topo.predecessors(rank):
        if src == rank:
            self_weight = float(w[src, rank])
        else:
            neighbor_weights[int(src)] = float(w[src, rank])
    return self_weight, neighbor_weights


def GetSendWeights(topo: nx.DiGraph, rank: int) -> Tuple[float, Dict[int, float]]:
    """(self_weight, {out-neighbor: weight}) attached to what ``rank`` sends."""
    w = nx.to_numpy_array(topo)
    self_weight = 0.0
    neighbor_weights = {}
    for dst in topo.successors(rank):
        if dst == rank:
            self_weight = float(w[rank, dst])
        else:
            neighbor_weights[int(dst)] = float(w[rank, dst])
    return self_weight, neighbor_weights


# --------------------------------------------------------------------------- #
# static graphs
# --------------------------------------------------------------------------- #
def ExponentialTwoGraph(size: int) -> nx.DiGraph:
    """Rank i sends to i + 2^k (mod size) for every 2^k < size, plus itself."""
    assert size > 0
    offsets = [0]
    d = 1
    while d < size:
        offsets.append(d)
        d *= 2
    return _circulant(size, offsets)


def ExponentialGraph(size: int, base: int = 2) -> nx.DiGraph:
    """Rank i sends to i + base^k (mod size) for every base^k < size, plus itself."""
    assert size > 0
    offsets = [0] + [d for d in range(1, size) if isPowerOf(d, base)]
    return _circulant(size, offsets)


def SymmetricExponentialGraph(size: int, base: int = 4) -> nx.DiGraph:
    """Exponential graph whose offsets are mirrored around size/2, so that the
    edge set is symmetric."""
    assert size > 0
    offsets = [0]
    for d in range(1, size):
        folded = d if d <= size // 2 else size - d
        if isPowerOf(folded, base):
            offsets.append(d)
    return _circulant(size, offsets)


def MeshGrid2DGraph(size: int, shape: Optional[Tuple[int, int]] = None) -> nx.DiGraph:
    """2-D grid (no wrap-around) with Metropolis-Hastings weights:
    w_ij = 1 / max(deg_i, deg_j) where deg counts the node itself, and the
    self weight takes the remainder so that every row sums to one."""
    assert size > 0
    if shape is None:
        nrow = int(math.isqrt(size))
        while size % nrow != 0:
            nrow -= 1
        shape = (nrow, size // nrow)
    nrow, ncol = shape
    assert size == nrow * ncol, "The shape doesn't match the size provided."
    neigh = [{i} for i in range(size)]
    for i in range(size):
        r, c = divmod(i, ncol)
        if c + 1 < ncol:
            neigh[i].add(i + 1)
            neigh[i + 1].add(i)
        if r + 1 < nrow:
            neigh[i].add(i + ncol)
            neigh[i + ncol].add(i)
    mat = np.zeros((size, size))
    for i in range(size):
        for j in neigh[i]:
            if j != i:
                mat[i, j] = 1.0 / max(len(neigh[i]), len(neigh[j]))
        mat[i, i] = 1.0 - mat[i].sum()
    return _graph_from_matrix(mat)


def StarGraph(size: int, center_rank: int = 0) -> nx.DiGraph:
    """Bidirectional star around ``center_rank``; every spoke weighs 1/size."""
    assert size > 0
    mat = np.zeros((size, size))
    for i in range(size):
        mat[i, i] = 1.0 - 1.0 / size
        mat[center_rank, i] = 1.0 / size
        mat[i, center_rank] = 1.0 / size
    return _graph_from_matrix(mat)


def RingGraph(size: int, connect_style: int = 0) -> nx.DiGraph:
    """Ring. connect_style 0: both neighbours (weights 1/3), 1: send to the left
    neighbour (i-1) only, 2: send to the right neighbour (i+1) only (weights 1/2)."""
    assert size > 0
    assert 0 <= connect_style <= 2, \
        "connect_style has to be int between 0 and 2, where 0 " \
        "for bi-connection, 1 for left connection, 2 for right connection."
    if size == 1:
        return _graph_from_matrix(np.array([[1.0]]))
    if size == 2:
        return _graph_from_matrix(np.array([[0.5, 0.5], [0.5, 0.5]]))
    if connect_style == 0:
        return _circulant(size, [0, 1, size - 1])
    if connect_style == 1:
        return _circulant(size, [0, size - 1])
    return _circulant(size, [0, 1])


def FullyConnectedGraph(size: int) -> nx.DiGraph:
    assert size > 0
    return _graph_from_matrix(np.full((size, size), 1.0 / size))


def IsRegularGraph(topo: nx.DiGraph) -> bool:
    """True when every node has the same (in+out) degree."""
    degree = topo.degree(0)
    return all(topo.degree(r) == degree for r in range(1, topo.number_of_nodes()))


# --------------------------------------------------------------------------- #
# dynamic schedules: generators of ([send_ranks], [recv_ranks])
# --------------------------------------------------------------------------- #
def _clockwise_out_neighbors(topo: nx.DiGraph, rank: int, size: int) -> List[int]:
    out = [r for r in topo.successors(rank) if r != rank]
    return sorted(out, key=lambda r: (r - rank) % size)


def GetDynamicOnePeerSendRecvRanks(
        topo: nx.DiGraph, self_rank: int) -> Iterator[Tuple[List[int], List[int]]]:
    """At round k every rank sends to the (k mod out-degree)-th of its
    out-neighbours taken clockwise; the recv list is whoever picks this rank in
    the same round."""
    size = topo.number_of_nodes()
    send_table = [_clockwise_out_neighbors(topo, r, size) for r in range(size)]
    index = 0
    while True:
        mine = send_table[self_rank]
        send_rank = mine[index % len(mine)]
        recv_ranks = [r for r in range(size)
                      if r != self_rank and send_table[r]
                      and send_table[r][index % len(send_table[r])] == self_rank]
        yield [send_rank], recv_ranks
        index += 1


def GetExp2DynamicSendRecvMachineRanks(
        world_size: int, local_size: int, self_rank: int, local_rank: int
) -> Iterator[Tuple[List[int], List[int]]]:
    """One-peer exponential-2 schedule over *machine* ids (for
    hierarchical_neighbor_allreduce)."""
    assert (self_rank % local_size) == local_rank, \
        "It should be used under homogeneous environment only."
    assert (world_size % local_size) == 0, \
        "It should be used under homogeneous environment only."
    assert world_size > local_size, \
        "It should be used under at least two machines case."
    machine_id = self_rank // local_size
    machine_size = world_size // local_size
    n_dist = (int(np.log2(machine_size - 1)) if machine_size > 1 else 0) + 1
    index = 0
    while True:
        dist = 2 ** (index % n_dist)
        yield [(machine_id + dist) % machine_size], [(machine_id - dist) % machine_size]
        index += 1


def GetInnerOuterRingDynamicSendRecvRanks(
        world_size: int, local_size: int, self_rank: int
) -> Iterator[Tuple[List[int], List[int]]]:
    """Round k: local rank (k mod local_size) of every machine talks to the same
    local rank of the next/previous machine; the remaining local ranks form a
    ring inside the machine that skips the outgoing one."""
    num_machines = world_size // local_size
    npm = local_size
    assert world_size % local_size == 0, "It should be used under homogeneous environment only."
    assert local_size > 2, "Do no support the case where nodes_per_machine is equal or " \
        "less than 2. Consider use hierarchical_neighbor_allreduce or GetDynamicOnePeerSendRecvRanks."
    machine_id, local_id = divmod(self_rank, npm)
    index = 0
    while True:
        outgoing = index % npm
        if outgoing == local_id:
            send_rank = ((machine_id + 1) % num_machines) * npm + local_id
            recv_rank = ((machine_id - 1) % num_machines) * npm + local_id
        else:
            nxt = (local_id + 1) % npm
            if nxt == outgoing:
                nxt = (nxt + 1) % npm
            prv = (local_id - 1) % npm
            if prv == outgoing:
                prv = (prv - 1) % npm
            send_rank = machine_id * npm + nxt
            recv_rank = machine_id * npm + prv
        yield [send_rank], [recv_rank]
        index += 1


def GetInnerOuterExpo2DynamicSendRecvRanks(
        world_size: int, local_size: int, self_rank: int
) -> Iterator[Tuple[List[int], List[int]]]:
    """Like the inner/outer ring schedule, but both the inter-machine hop and the
    intra-machine hop walk exponential-2 distances."""
    num_machines = world_size // local_size
    npm = local_size
    assert world_size % local_size == 0, "It should be used under homogeneous environment only."
    assert local_size > 2, "Do no support the case where nodes_per_machine is equal or " \
        "less than 2. Consider use hierarchical_neighbor_allreduce or GetDynamicOnePeerSendRecvRanks."
    n_out = int(np.log2(num_machines - 1)) + 1
    n_in = (0 if npm == 2 else int(np.log2(npm - 2))) + 1
    machine_id, local_id = divmod(self_rank, npm)
    index = 0
    while True:
        outgoing = index % npm
        if outgoing == local_id:
            dist = 2 ** (index % n_out)
            send_rank = ((machine_id + dist) % num_machines) * npm + local_id
            recv_rank = ((machine_id - dist) % num_machines) * npm + local_id
        else:
            fwd = 2 ** (index % n_in)
            if fwd >= (outgoing - local_id) % npm:
                fwd += 1  # hop over the rank that is talking to another machine
            bwd = 2 ** (index % n_in)
            if bwd >= (local_id - outgoing) % npm:
                bwd += 1
            send_rank = machine_id * npm + (local_id + fwd) % npm
            recv_rank = machine_id * npm + (local_id - bwd) % npm
        yield [send_rank], [recv_rank]
        index += 1
