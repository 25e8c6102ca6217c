"""World-size-2 run on CPU (gloo) of the host side of the fused linear + all-reduce: the
exchange of memory handles and the bookkeeping of buffer sets and arrival counts
(neuzip_b200.tpcomm.PeerReducer) against a stand-in for the CUDA library that hands out
fake pointers.  What the kernels do with the buffers is covered on two GPUs
(tests/test_gpu_tp_allreduce.py)."""
import ctypes
import os
import socket

import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class FakeLib:
    """nz_peer_* of the C ABI: pointers are rank * 2^32 + a running number, a handle holds the
    pointer it stands for, opening a handle gives that pointer + 2^48 (a mapping elsewhere)."""

    def __init__(self, rank):
        self.rank, self.count = rank, 0
        self.opened, self.closed, self.freed = [], [], []

    def nz_peer_alloc(self, nbytes, ptr_ref, handle):
        self.count += 1
        value = (self.rank + 1) * (1 << 32) + self.count * 4096
        ptr_ref._obj.value = value
        handle.raw = value.to_bytes(8, "little") + bytes(56)
        return 0

    def nz_peer_open(self, handle, ptr_ref):
        value = int.from_bytes(bytes(handle)[:8], "little") + (1 << 48)
        ptr_ref._obj.value = value
        self.opened.append(value)
        return 0

    def nz_peer_close(self, ptr):
        self.closed.append(ptr)
        return 0

    def nz_peer_free(self, ptr):
        self.freed.append(ptr)
        return 0


def _worker(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from neuzip_b200.tpcomm import PeerReducer
    lib = FakeLib(rank)
    red = PeerReducer(None, workspace_bytes=1000, lib=lib, device=rank)
    sets = []
    for call in range(5):
        s, group, before = red.next_set()
        sets.append((s, before, [group.workspace[q] for q in range(world)],
                     [group.arrivals[q] for q in range(world)], group.world, group.rank,
                     group.workspace_bytes))
        red.advance(s, before + 10 * (call + 1))
    fits = (red.fits(1024), red.fits(1025))
    red.close()
    out_q.put((rank, sets, fits, lib.opened, lib.closed, lib.freed))
    dist.barrier()
    dist.destroy_process_group()


def test_peer_reducer_exchanges_handles_and_alternates_buffer_sets():
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out_q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, sets, fits, opened, closed, freed in results:
        peer = 1 - rank
        assert fits == (True, False)                       # 1000 bytes round up to 1024
        assert [s for s, *_ in sets] == [0, 1, 0, 1, 0]    # two sets in turn
        # a set's arrival count is what the previous call on that set reported
        assert [before for _, before, *_ in sets] == [0, 0, 10, 20, 40]
        for s, _, ws, arr, world, grank, nbytes in sets:
            assert (world, grank, nbytes) == (2, rank, 1024)
            # own buffers: local pointers; the peer's: mappings of the peer's allocations
            own_ws = (rank + 1) * (1 << 32) + (2 * s + 1) * 4096
            own_arr = (rank + 1) * (1 << 32) + (2 * s + 2) * 4096
            assert (ws[rank], arr[rank]) == (own_ws, own_arr)
            assert ws[peer] == (peer + 1) * (1 << 32) + (2 * s + 1) * 4096 + (1 << 48)
            assert arr[peer] == (peer + 1) * (1 << 32) + (2 * s + 2) * 4096 + (1 << 48)
        assert len(opened) == 4 and sorted(closed) == sorted(opened)
        assert len(freed) == 4 and all(p >> 32 == rank + 1 for p in freed)
