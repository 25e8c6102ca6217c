"""Peer-visible buffers for the tensor-parallel all-reduce that is fused into the linear
kernel's epilogue (``nz_linear_allreduce_bf16``).

One process per GPU of one node.  Every rank allocates two buffer sets (a workspace for the
fp32 partial sums of all ranks and a few arrival counters), exports them as inter-process
handles, gathers the peers' handles over the given process group (host side, any backend) and
maps them.  Calls alternate between the two sets: a set is written again by the call after
next at the earliest, by which time every rank has read it (a rank's call k+2 starts after its
own reduction of call k+1, which waited for every peer's kernel of call k+1, which follows
that peer's reduction of call k in stream order).

The reference has no tensor parallelism; nothing here has a counterpart in it.
"""
import ctypes
from typing import List, Optional, Tuple

import torch

from . import _lib

_SETS = 2
_COUNTER_BYTES = 256


class PeerReducer:
    """Two peer-mapped buffer sets of `workspace_bytes` each for the ranks of `group`."""

    def __init__(self, group=None, workspace_bytes: int = 64 << 20, lib=None,
                 device: Optional[int] = None) -> None:
        """`lib` and `device` default to the CUDA library and the current device (tests pass
        stand-ins to exercise the bookkeeping without a GPU)."""
        import torch.distributed as dist
        self._lib = lib if lib is not None else _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError(f"a peer group has 2 to 8 ranks, got {self.world}")
        self.workspace_bytes = (int(workspace_bytes) + 255) // 256 * 256
        self.device = torch.cuda.current_device() if device is None else int(device)
        self._own: List[Tuple[int, int]] = []
        self._mapped: List[int] = []
        mine = []
        for _ in range(_SETS):
            pair = []
            for nbytes in (self.workspace_bytes, _COUNTER_BYTES):
                ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                _lib.check(self._lib.nz_peer_alloc(nbytes, ctypes.byref(ptr), handle))
                pair.append((ptr.value, handle.raw))
            self._own.append((pair[0][0], pair[1][0]))
            mine.append((pair[0][1], pair[1][1]))
        everyone: List[Optional[list]] = [None] * self.world
        dist.all_gather_object(everyone, (self.device, mine), group=group)
        devices = [d for d, _ in everyone]
        if len(set(devices)) != self.world:
            raise RuntimeError(f"the ranks of a peer group need one GPU each, got devices {devices}")
        self._groups = []
        for s in range(_SETS):
            g = _lib.PeerGroup()
            g.world, g.rank, g.workspace_bytes = self.world, self.rank, self.workspace_bytes
            for q, (_, handles) in enumerate(everyone):
                if q == self.rank:
                    g.workspace[q], g.arrivals[q] = self._own[s]
                    continue
                for field, handle in ((g.workspace, handles[s][0]), (g.arrivals, handles[s][1])):
                    ptr = ctypes.c_void_p()
                    _lib.check(self._lib.nz_peer_open(handle, ctypes.byref(ptr)))
                    self._mapped.append(ptr.value)
                    field[q] = ptr.value
            self._groups.append(g)
        self._arrivals = [0] * _SETS
        self._turn = 0
        # every rank has mapped every buffer before anybody's kernel stores into one
        dist.barrier(group=group)

    def fits(self, need_bytes: int) -> bool:
        return need_bytes <= self.workspace_bytes

    def next_set(self):
        """(struct nz_peer_group, arrivals so far) of the set this call uses; give the call's
        *arrivals_after to `advance`."""
        s = self._turn
        return s, self._groups[s], self._arrivals[s]

    def advance(self, s: int, arrivals_after: int) -> None:
        self._arrivals[s] = int(arrivals_after)
        self._turn = (s + 1) % _SETS

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Collective: every rank of the group
        calls it.  Each rank first waits for its own stream (its last reduction has then seen
        every peer's stores and arrivals, so nobody still writes here), unmaps what it
        imported, and only after a barrier -- when no rank holds a mapping any more -- frees
        what it exported."""
        if self._lib is None:
            return
        import torch.distributed as dist
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for ptr in self._mapped:
            self._lib.nz_peer_close(ptr)
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for ws, arr in self._own:
            self._lib.nz_peer_free(ws)
            self._lib.nz_peer_free(arr)
        self._mapped, self._own, self._lib = [], [], None
