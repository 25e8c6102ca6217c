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


# ---------------------------------------------------------------------------
# Tensor parallelism of the converted Linears.
#
# The reference converts every nn.Linear whole (neuzip/utils.py:57-68) and has no
# tensor parallelism.  With `Manager.convert(model, tp_rank=r, tp_world=t)` each rank
# compresses only its block of every Linear named in the plan:
#   "column"  the rank's contiguous rows of W[out, in] (and of the bias): the output is
#             the rank's slice of the features, no communication;
#   "row"     the rank's contiguous columns, stored as its own contiguous
#             [out, in / t] matrix; the outputs of the ranks are partial sums, added by
#             one all-reduce after the Linear (the bias is added on rank 0 only).
# The default plan is the Llama / Mistral naming: q, k, v, gate, up are column-parallel,
# o and down row-parallel, so one all-reduce follows the attention output projection and
# one the MLP.  The codec itself never communicates.

LLAMA_TP_PLAN = {
    "q_proj": "column", "k_proj": "column", "v_proj": "column",
    "gate_proj": "column", "up_proj": "column",
    "o_proj": "row", "down_proj": "row",
}


def tp_mode(name: str, plan=None):
    """'column', 'row' or None for a child module called `name`."""
    plan = LLAMA_TP_PLAN if plan is None else plan
    return plan.get(name)


def shard_bounds(size: int, rank: int, world_size: int):
    if size % world_size:
        raise ValueError(f"a dimension of {size} does not split over {world_size} ranks")
    step = size // world_size
    return rank * step, (rank + 1) * step


def shard_linear_weight(weight, bias, mode: str, rank: int, world_size: int):
    """The rank's block of a Linear's weight [out, in] (a contiguous copy) and bias."""
    out_f, in_f = weight.shape
    if mode == "column":
        lo, hi = shard_bounds(out_f, rank, world_size)
        return weight[lo:hi].contiguous(), (None if bias is None else bias[lo:hi].contiguous())
    if mode == "row":
        lo, hi = shard_bounds(in_f, rank, world_size)
        return weight[:, lo:hi].contiguous(), (bias if rank == 0 else None)
    raise ValueError(f"unknown tensor-parallel mode {mode!r}")
