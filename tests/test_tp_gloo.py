"""World-size-2 run on CPU (gloo) of the tensor-parallel conversion: every rank
builds the same small Llama, converts it with Manager.convert(tp_rank, tp_world) (CPU
stand-in backend), and the tensor-parallel logits must match the dense model's within
bf16 tolerance; the slices must be the ones the sharding rules name and the stored
bytes must split evenly."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neuzip_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model():
    import transformers
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128,
                                   num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).eval()


def _worker(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import neuzip
    from tests.fakes import cpu_manager
    model = _model()
    ids = torch.randint(0, 128, (2, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model(ids).logits.float()
    dense_q = model.model.layers[0].self_attn.q_proj.weight.data.clone()
    dense_down = model.model.layers[1].mlp.down_proj.weight.data.clone()
    m = cpu_manager(7)
    m.convert(model, tp_rank=rank, tp_world=world)
    layer0, layer1 = model.model.layers[0], model.model.layers[1]
    q, down = layer0.self_attn.q_proj, layer1.mlp.down_proj
    assert isinstance(q, neuzip.nn.Linear) and (q.out_features, q.in_features) == (32, 64)
    assert (down.out_features, down.in_features) == (64, 64) and down.reduce_output
    assert not q.reduce_output
    assert torch.equal(q._p(), dense_q[32 * rank:32 * (rank + 1)])
    assert torch.equal(down._p(), dense_down[:, 64 * rank:64 * (rank + 1)])
    with torch.no_grad():
        got = model(ids).logits.float()
    # the same tokens come out of every rank (the all-reduce leaves identical sums)
    gathered = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(gathered, got)
    assert all(torch.equal(g, gathered[0]) for g in gathered)
    stored = torch.tensor([m.total_size()], dtype=torch.int64)
    sizes = [torch.zeros_like(stored) for _ in range(world)]
    dist.all_gather(sizes, stored)
    if rank == 0:
        out_q.put((float((got - ref).abs().max()), float(ref.abs().max()),
                   [int(s) for s in sizes]))
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_conversion_matches_the_dense_model():
    pytest.importorskip("transformers")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    err, scale, sizes = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # partial sums are rounded to bf16 before they are added: a few bf16 steps of the logits
    assert err <= 2.0 ** -5 * max(scale, 1.0)
    assert abs(sizes[0] - sizes[1]) <= 0.02 * sizes[0]


def test_sharding_helpers():
    w = torch.arange(24, dtype=torch.float32).reshape(4, 6)
    b = torch.arange(4, dtype=torch.float32)
    col, cb = sharding.shard_linear_weight(w, b, "column", 1, 2)
    assert torch.equal(col, w[2:4]) and torch.equal(cb, b[2:4]) and col.is_contiguous()
    row, rb = sharding.shard_linear_weight(w, b, "row", 1, 2)
    assert torch.equal(row, w[:, 3:6]) and rb is None and row.is_contiguous()
    assert sharding.shard_linear_weight(w, b, "row", 0, 2)[1] is b
    assert sharding.tp_mode("o_proj") == "row" and sharding.tp_mode("lm_head") is None
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 0, 3)
