"""Placement of independent compressed tensors on the ranks of one node.

The codec has no exchange step: every tensor (and every unit inside it) is
compressed and decoded on its own (reference: one cache entry per name,
cuda/high_level.cu:126-129).  Sharding is therefore a pure assignment problem;
no collective touches the data path.
"""
from __future__ import annotations

from typing import List, Sequence


def owner_of_layer(layer: int, world_size: int) -> int:
    """Layer-set `layer` lives on rank layer mod world_size."""
    return layer % world_size


def layers_of_rank(n_layers: int, rank: int, world_size: int) -> List[int]:
    return [l for l in range(n_layers) if owner_of_layer(l, world_size) == rank]


def balance_by_bytes(sizes: Sequence[int], world_size: int) -> List[List[int]]:
    """Greedy longest-first assignment of tensors to ranks by byte size; returns
    the tensor indices of each rank.  Deterministic (ties go to the lower rank)."""
    order = sorted(range(len(sizes)), key=lambda i: (-sizes[i], i))
    loads = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += sizes[i]
    return [sorted(v) for v in out]
