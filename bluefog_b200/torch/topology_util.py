"""Collective inference of the reverse neighbor lists.

Each rank knows only whom it sends to (or receives from); two allgathers assemble the full
edge list so that every rank can read off the other direction.  Same contract as the
reference (bluefog/torch/topology_util.py:22-108), including the optional
receive-normalised adjacency matrix.
"""
import collections
from typing import Any, List, Tuple, Union

import numpy as np
import torch

from bluefog_b200.common.basics import get_basics
from bluefog_b200.ops.collectives import allgather

_b = get_basics()


def _validate(ranks: List[Any], what: str):
    problem = None
    if any(not isinstance(r, (int, np.integer)) for r in ranks):
        problem = "contain element that is not integer."
    elif any(r < 0 or r >= _b.size() for r in ranks):
        problem = "contain element that is not between 0 and size-1."
    elif len(set(ranks)) != len(ranks):
        problem = "contain duplicated elements."
    elif _b.rank() in ranks:
        problem = "contain self rank."
    assert problem is None, f"The format of {what} is wrong: {problem}"


def _gather_edges(ranks: List[int]):
    degrees = allgather(torch.tensor([len(ranks)], dtype=torch.int32)).tolist()
    flat = allgather(torch.tensor(list(ranks), dtype=torch.int32)).tolist()
    edges, pos = {}, 0
    for r, d in enumerate(degrees):
        edges[r] = sorted(int(x) for x in flat[pos:pos + d])
        pos += d
    return edges


def _infer(ranks: List[int], transpose: bool, construct_adjacency_matrix: bool):
    edges = _gather_edges(ranks)
    reverse = collections.defaultdict(list)
    for r, adj in edges.items():
        for v in adj:
            reverse[v].append(r)
    mine = reverse.get(_b.rank(), [])
    if not construct_adjacency_matrix:
        return mine
    w = np.eye(_b.size())
    for r, adj in edges.items():
        w[r, adj] = 1
    if transpose:
        w = w.T
    return mine, w / w.sum(axis=1)


def InferSourceFromDestinationRanks(
        dst_ranks: List[int], construct_adjacency_matrix: bool = False,
) -> Union[List[int], Tuple[List[int], np.ndarray]]:
    """Collective: given everybody's destination list, returns this rank's source list (and,
    optionally, the adjacency matrix W with W[i, j] = weight of i -> j)."""
    _validate(dst_ranks, "dst_ranks")
    return _infer(dst_ranks, False, construct_adjacency_matrix)


def InferDestinationFromSourceRanks(
        src_ranks: List[int], construct_adjacency_matrix: bool = False,
) -> Union[List[int], Tuple[List[int], np.ndarray]]:
    """Collective: given everybody's source list, returns this rank's destination list."""
    _validate(src_ranks, "src_ranks")
    return _infer(src_ranks, True, construct_adjacency_matrix)
