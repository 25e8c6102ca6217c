"""World-size-2 run on CPU (gloo) of the data-parallel gradient path of
CompressedAdamW: two micro-batches per step, with and without no_sync, must give
sum over ranks and micro-batches of the weight gradient -- the value a single
process computes from all four micro-batches."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _micro_batch(rank, mb):
    g = torch.Generator().manual_seed(100 + 10 * rank + mb)
    return torch.randn(4, 32, generator=g).to(torch.bfloat16)


def _weight():
    g = torch.Generator().manual_seed(7)
    return (torch.randn(16, 32, generator=g) * 0.1).to(torch.bfloat16)


def _grad_of(x, w):
    """dW of loss = sum(x @ W^T) as the autograd function computes it (bf16 matmul)."""
    y = torch.nn.functional.linear(x, w)
    return torch.mm(torch.ones_like(y).t(), x)


def _worker(rank, world, port, use_no_sync, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import neuzip
    from neuzip_b200.optim import CompressedAdamW
    from tests.fakes import cpu_manager
    m = cpu_manager(7)
    lin = torch.nn.Linear(32, 16, bias=False).to(torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(_weight())
    layer = neuzip.nn.Linear(m, lin)
    opt = CompressedAdamW(layer.parameters(), lr=1e-3)
    assert opt.world == 2 and len(opt._hooks) == 1
    for mb in range(2):
        x = _micro_batch(rank, mb).requires_grad_(True)
        if use_no_sync and mb == 0:
            with opt.no_sync():
                layer(x).sum().backward()
            assert not opt._pending          # nothing in flight inside no_sync
        else:
            layer(x).sum().backward()
    total = opt._reduced_gradient(layer._p)
    out_q.put((rank, total.float().tolist()))
    dist.barrier()
    dist.destroy_process_group()


def _run(use_no_sync):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, use_no_sync, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = _weight()
    pieces = [[_grad_of(_micro_batch(r, mb), w) for mb in range(2)] for r in range(world)]
    if use_no_sync:
        # each rank adds its two micro-batches in bf16, then the ranks are summed
        local = [pieces[r][0].clone().add_(pieces[r][1]) for r in range(world)]
        expect = local[0] + local[1]
    else:
        # each micro-batch is summed over the ranks, then the two sums are added
        expect = (pieces[0][0] + pieces[1][0]).add_(pieces[0][1] + pieces[1][1])
    for r in range(world):
        assert torch.equal(torch.tensor(got[r]), expect.float()), r
    assert got[0] == got[1]                  # replicas agree bit for bit


def test_two_micro_batches_are_each_reduced():
    _run(use_no_sync=False)


def test_no_sync_accumulates_locally_and_reduces_once():
    _run(use_no_sync=True)
