"""Two ranks on two GPUs (four on four, where the box has them): the fused linear whose epilogue
adds the ranks' partial outputs over peer memory (nz_linear_allreduce_bf16) against an fp64
product of the unsharded weight.  Checks: all ranks obtain the same bits; the error stays within bf16 rounding of an fp32
sum; a sequence of calls on alternating buffer sets and different shapes keeps working (the
arrival counters only grow); the bias given on rank 0 is added once; the status word stays 0.
Host side over gloo; no library collective touches the GPUs here.  Skipped with fewer than
two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

SHAPES = [(640, 4096), (384, 8192), (4096, 4096)]     # (out, in) of the unsharded weights
ROWS = [1, 16, 128, 16, 100, 128, 7]                   # tokens of the successive calls


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import neuzip
    from neuzip_b200.sharding import shard_bounds
    manager = neuzip.Manager(precision=7)
    gen = torch.Generator().manual_seed(5)
    layers, dense = [], []
    for i, (out_f, in_f) in enumerate(SHAPES):
        lin = torch.nn.Linear(in_f, out_f, bias=(i == 0), dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_((torch.randn(out_f, in_f, generator=gen) * 0.02).to(torch.bfloat16))
            if lin.bias is not None:
                lin.bias.copy_(torch.randn(out_f, generator=gen).to(torch.bfloat16))
        dense.append((lin.weight.detach().double(),
                      None if lin.bias is None else lin.bias.detach().double()))
        layers.append(neuzip.nn.Linear(manager, lin.cuda(), tp=("row", rank, world, None)))
    manager.fuse_tp_allreduce(None, max_rows=256)
    report = []
    with torch.no_grad():
        for call, m in enumerate(ROWS):
            k = call % len(SHAPES)
            out_f, in_f = SHAPES[k]
            x = (torch.randn(m, in_f, generator=gen)).to(torch.bfloat16)
            lo, hi = shard_bounds(in_f, rank, world)
            y = layers[k](x[:, lo:hi].contiguous().cuda())
            torch.cuda.synchronize()
            want = x.double() @ dense[k][0].t()
            if dense[k][1] is not None:
                want = want + dense[k][1]
            got = y.cpu()
            err = (got.double() - want).abs().max().item()
            scale = want.abs().max().item()
            both = [None] * world
            dist.all_gather_object(both, got.view(torch.int16).numpy().tobytes())
            report.append((call, m, err, scale, all(b == both[0] for b in both)))
    status = manager._be.status()
    dist.barrier()
    manager.fuse_tp_allreduce(None, max_rows=0)
    dist.barrier()
    out_q.put((rank, status, report))
    dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", (2, 4))
def test_fused_linear_allreduce_over_peer_memory(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=500) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, status, report in results:
        assert status == 0, f"rank {rank}: status {status:#x}"
        assert len(report) == len(ROWS)
        for call, m, err, scale, same in report:
            assert same, f"rank {rank} call {call}: the ranks' outputs differ"
            # one rounding to bf16 of an fp32 sum: half an ulp of the largest output
            assert err <= scale * 2.0 ** -8 + 1e-6, (rank, call, m, err, scale)
