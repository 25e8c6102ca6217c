"""World-size-2 run on CPU (gloo): each rank owns the layer sets the sharding
rule gives it, compresses and decodes them independently (oracle codec standing
in for the GPU), and only a checksum travels between ranks."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neuzip_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_layers, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    mine = sharding.layers_of_rank(n_layers, rank, world)
    total = 0
    stored = 0
    for layer in mine:
        for j, shape in enumerate([(64, 64), (176, 64)]):
            g = torch.Generator().manual_seed(1000 + 7 * layer + j)
            w = (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16)
            bits = w.view(torch.int16).numpy().view(np.uint16).reshape(-1)
            cont, frac = O.compress_bf16(bits, 7)
            back = O.decompress_bf16(cont, frac, bits.size, 7)
            assert np.array_equal(back, bits)
            total += int(O.crc32(back))
            stored += cont.size + frac.size
    t = torch.tensor([total, stored, len(mine)], dtype=torch.int64)
    dist.all_reduce(t)            # bookkeeping only: no tensor data crosses ranks
    if rank == 0:
        out_q.put(t.tolist())
    dist.destroy_process_group()


def test_layers_shard_without_overlap_and_checksums_agree():
    n_layers, world = 6, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_layers, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-process reference
    from oracle import oracle as O
    total = 0
    for layer in range(n_layers):
        for j, shape in enumerate([(64, 64), (176, 64)]):
            g = torch.Generator().manual_seed(1000 + 7 * layer + j)
            w = (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16)
            total += int(O.crc32(w.view(torch.int16).numpy().view(np.uint16).reshape(-1)))
    assert got[0] == total and got[2] == n_layers and got[1] > 0


def test_sharding_rules():
    assert sharding.layers_of_rank(32, 3, 8) == [3, 11, 19, 27]
    parts = [sharding.layers_of_rank(32, r, 8) for r in range(8)]
    assert sorted(sum(parts, [])) == list(range(32))
    sizes = [16, 16, 16, 16, 45, 45, 45]
    split = sharding.balance_by_bytes(sizes, 2)
    assert sorted(split[0] + split[1]) == list(range(7))
    loads = [sum(sizes[i] for i in part) for part in split]
    assert abs(loads[0] - loads[1]) <= 45
