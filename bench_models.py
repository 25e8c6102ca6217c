#!/usr/bin/env python
"""Model-level legs of the benchmark: Llama-shaped models, dense vs compressed.

Imported by bench.py (`model` sub-object: shortened 7B-shape decode and 1.3B-shape
training on one GPU) and runnable on its own for the full configurations:

    python bench_models.py decode --layers 32                     # config 3 (7B shape)
    python bench_models.py train --layers 24                      # config 4 (1.3B shape)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        bench_models.py tp --layers 80 --precision 3              # config 5 (70B shape, TP)

Weights are random (N(0, 0.02)), prompts uniform random tokens: synthetic stand-ins for
the Llama checkpoints and datasets the reference's scripts load.

The decode legs use a small Llama-architecture module of their own (RMSNorm, rotary
attention over a static key/value cache, SwiGLU) whose single-token step takes its
position from a device tensor, so that the whole step can be captured in a CUDA graph:
the eager loop of a general-purpose model class is bound by kernel-launch overhead at
batch 1, which hides the cost of decoding the weights; the graphed loop does not.  Both
are reported, for the dense and for the compressed model.
"""
import argparse
import json
import os
import time

import torch
import torch.nn.functional as F

SHAPES = {
    "7b": dict(d=4096, heads=32, kv_heads=32, ffn=11008, vocab=32000, layers=32),
    "1.3b": dict(d=2048, heads=16, kv_heads=16, ffn=5504, vocab=32000, layers=24),
    "70b": dict(d=8192, heads=64, kv_heads=8, ffn=28672, vocab=32000, layers=80),
    "tiny": dict(d=1024, heads=8, kv_heads=4, ffn=2048, vocab=1024, layers=2),
}


def _linear(out_f, in_f, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    lin = torch.nn.Linear(in_f, out_f, bias=False, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(out_f, in_f, generator=g, device="cuda") * 0.02).to(torch.bfloat16))
    return lin


def _rope(x, cos, sin):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class Block(torch.nn.Module):
    """One decoder layer.  The projections are built whole and named as in Llama, so that
    Manager.convert(..., tp_rank, tp_world) finds and shards them."""

    def __init__(self, cfg, layer):
        super().__init__()
        d, hd = cfg["d"], cfg["d"] // cfg["heads"]
        self.hd = hd
        s = 1000 * layer
        self.q_proj = _linear(cfg["heads"] * hd, d, s + 1)
        self.k_proj = _linear(cfg["kv_heads"] * hd, d, s + 2)
        self.v_proj = _linear(cfg["kv_heads"] * hd, d, s + 3)
        self.o_proj = _linear(d, cfg["heads"] * hd, s + 4)
        self.gate_proj = _linear(cfg["ffn"], d, s + 5)
        self.up_proj = _linear(cfg["ffn"], d, s + 6)
        self.down_proj = _linear(d, cfg["ffn"], s + 7)
        self.norm1 = torch.nn.RMSNorm(d, eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.norm2 = torch.nn.RMSNorm(d, eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.k_cache = None
        self.v_cache = None

    def forward(self, x, cos, sin, pos_idx, mask):
        B, T, _ = x.shape
        h = self.norm1(x)
        q = self.q_proj(h).view(B, T, -1, self.hd).transpose(1, 2)
        k = self.k_proj(h).view(B, T, -1, self.hd).transpose(1, 2)
        v = self.v_proj(h).view(B, T, -1, self.hd).transpose(1, 2)
        if self.k_cache is None or self.k_cache.shape[1] != k.shape[1]:
            raise RuntimeError("key/value cache not allocated for this head count")
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        self.k_cache.index_copy_(2, pos_idx, k)
        self.v_cache.index_copy_(2, pos_idx, v)
        att = F.scaled_dot_product_attention(q, self.k_cache, self.v_cache, attn_mask=mask,
                                             enable_gqa=q.shape[1] != k.shape[1])
        x = x + self.o_proj(att.transpose(1, 2).reshape(B, T, -1))
        h = self.norm2(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class MiniLlama(torch.nn.Module):
    def __init__(self, cfg, n_layers, max_len, batch):
        super().__init__()
        self.cfg, self.max_len, self.batch = cfg, max_len, batch
        g = torch.Generator(device="cuda").manual_seed(7)
        self.embed = (torch.randn(cfg["vocab"], cfg["d"], generator=g, device="cuda") * 0.02
                      ).to(torch.bfloat16)
        self.lm_head = _linear(cfg["vocab"], cfg["d"], 8)      # never converted (as in the reference)
        self.norm = torch.nn.RMSNorm(cfg["d"], eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.layers = torch.nn.ModuleList([Block(cfg, l) for l in range(n_layers)])
        hd = cfg["d"] // cfg["heads"]
        inv = 1.0 / (10000 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
        fr = torch.outer(torch.arange(max_len, device="cuda").float(), inv)
        self.cos, self.sin = fr.cos().to(torch.bfloat16), fr.sin().to(torch.bfloat16)
        self.positions = torch.arange(max_len, device="cuda")
        self.allocate_cache(cfg["kv_heads"])

    def allocate_cache(self, kv_heads):
        hd = self.cfg["d"] // self.cfg["heads"]
        for layer in self.layers:
            layer.k_cache = torch.zeros(self.batch, kv_heads, self.max_len, hd, device="cuda",
                                        dtype=torch.bfloat16)
            layer.v_cache = torch.zeros_like(layer.k_cache)

    @torch.no_grad()
    def forward(self, ids, pos_idx):
        """ids [B, T]; pos_idx LongTensor[T] on the device: the positions of these tokens."""
        x = self.embed[ids]
        cos, sin = self.cos.index_select(0, pos_idx), self.sin.index_select(0, pos_idx)
        mask = self.positions[None, :] <= pos_idx[:, None]            # [T, max_len]
        for layer in self.layers:
            x = layer(x, cos, sin, pos_idx, mask)
        return self.lm_head(self.norm(x[:, -1:]))


class Decoder:
    """Greedy decoding with device-side state: eager, or one CUDA graph replay per token."""

    def __init__(self, model, prompt, new_tokens):
        self.model, self.prompt, self.new = model, prompt, new_tokens
        B = prompt.shape[0]
        self.tok = torch.zeros(B, 1, dtype=torch.long, device="cuda")
        self.pos = torch.zeros(1, dtype=torch.long, device="cuda")
        self.step_no = torch.zeros(1, dtype=torch.long, device="cuda")
        self.out = torch.zeros(B, new_tokens, dtype=torch.long, device="cuda")

    def prefill(self):
        T = self.prompt.shape[1]
        logits = self.model(self.prompt, self.model.positions[:T])
        self.tok.copy_(logits.argmax(-1).view(-1, 1))
        self.pos.fill_(T)
        self.step_no.zero_()
        self.out.zero_()
        self.out.index_copy_(1, self.step_no, self.tok)
        self.step_no.add_(1)

    def step(self):
        logits = self.model(self.tok, self.pos)
        self.tok.copy_(logits.argmax(-1).view(-1, 1))
        self.out.index_copy_(1, self.step_no, self.tok)
        self.pos.add_(1)
        self.step_no.add_(1)

    def run(self, graph=False):
        """Returns (tokens [B, new], seconds per generated token after the first)."""
        with torch.no_grad():
            self.prefill()
            runner = self.step
            if graph:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.step()                     # warm-up outside the capture
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                self.prefill()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.step()
                torch.cuda.synchronize()
                self.prefill()                      # the captured step ran once: start over
                runner = g.replay
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(self.new - 1):
                runner()
            e1.record()
            torch.cuda.synchronize()
        return self.out.clone(), e0.elapsed_time(e1) * 1e-3 / max(1, self.new - 1)


def decode_leg(n_layers=8, full_layers=32, shape="7b", prompt_len=128, new_tokens=64, batch=1,
               precision=7):
    """Configuration 3 (shortened when n_layers < full_layers): greedy decode, batch 1."""
    import neuzip
    from neuzip_b200 import layerwise
    cfg = SHAPES[shape]
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg["vocab"], (batch, prompt_len), generator=g).cuda()
    model = MiniLlama(cfg, n_layers, prompt_len + new_tokens + 8, batch)
    res = {"workload": f"config 3 shape ({shape}: d_model {cfg['d']}, FFN {cfg['ffn']}, vocab "
                       f"{cfg['vocab']}), {n_layers} of {full_layers} layers, batch {batch}, "
                       f"{prompt_len}-token random prompt, {new_tokens} greedy tokens, precision "
                       f"{precision}; own Llama-architecture loop with a static key/value cache",
           "layers": n_layers, "of_layers": full_layers}
    dec = Decoder(model, prompt, new_tokens)
    dec.run()                                                       # warm-up
    ref, t = dec.run()
    res["dense_eager_tok_s"] = batch / t
    _, t = dec.run(graph=True)
    res["dense_graph_tok_s"] = batch / t

    manager = neuzip.Manager(precision=precision)
    t0 = time.perf_counter()
    for layer in model.layers:
        manager.convert(layer)
    torch.cuda.synchronize()
    res["convert_s"] = round(time.perf_counter() - t0, 2)
    manager._be.settle_all()
    manager._be.release_scratch()
    torch.cuda.empty_cache()
    dense_bytes = sum(int(torch.Size(s).numel()) * 2 for s in manager.meta_dict.values())
    res["ratio_converted_weights"] = round(manager.total_size() / dense_bytes, 5)
    dec.run()
    out, t = dec.run()                                              # one decode per Linear
    res["neuzip_per_linear_eager_tok_s"] = batch / t
    res["tokens_identical"] = bool(torch.equal(out, ref))
    hooks = layerwise.attach(model, manager)
    dec.run()
    out, t = dec.run()
    res["neuzip_layerwise_eager_tok_s"] = batch / t
    res["layerwise_tokens_identical"] = bool(torch.equal(out, ref))
    out, t = dec.run(graph=True)
    res["neuzip_layerwise_graph_tok_s"] = batch / t
    res["layerwise_graph_tokens_identical"] = bool(torch.equal(out, ref))
    for h in hooks:
        h.remove()
    manager.fuse_linear(256)        # prompt and single-token steps decode into tensor-core tiles
    dec.run()
    out, t = dec.run()
    res["neuzip_fused_linear_eager_tok_s"] = batch / t
    out, t = dec.run(graph=True)
    res["neuzip_fused_linear_graph_tok_s"] = batch / t
    res["fused_linear_tokens_equal_fraction"] = float((out == ref).float().mean().item())
    manager.check()
    res["ratio_vs_dense_eager"] = round(res["neuzip_layerwise_eager_tok_s"] / res["dense_eager_tok_s"], 3)
    res["ratio_vs_dense_graph"] = round(res["neuzip_layerwise_graph_tok_s"] / res["dense_graph_tok_s"], 3)
    for k, v in list(res.items()):
        if k.endswith("tok_s"):
            res[k] = round(v, 2)
    del model, dec
    torch.cuda.empty_cache()
    return res


def train_leg(n_layers=6, full_layers=24, shape="1.3b", batch=8, seq=1024, steps=3, precision=7):
    """Configuration 4 (shortened when n_layers < full_layers): AdamW lr 1e-4 with lossless
    compressed weights, per-layer decode in forward and backward, on this rank's GPU; under
    torch.distributed the replicas' weight gradients are all-reduced."""
    import torch.distributed as dist
    import transformers
    import neuzip
    from neuzip_b200.optim import CompressedAdamW
    cfg = SHAPES[shape]
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    hf = transformers.LlamaConfig(vocab_size=cfg["vocab"], hidden_size=cfg["d"],
                                  intermediate_size=cfg["ffn"], num_hidden_layers=n_layers,
                                  num_attention_heads=cfg["heads"], num_key_value_heads=cfg["kv_heads"],
                                  max_position_embeddings=4096, rms_norm_eps=1e-5)

    def build():
        torch.manual_seed(0)
        with torch.device("cuda"):
            return transformers.LlamaForCausalLM(hf).to(torch.bfloat16)

    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, cfg["vocab"], (batch, seq), generator=g).cuda()

    def run(model, opt, warmup=2):
        times = []
        for it in range(warmup + steps):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            loss = model(ids, labels=ids).loss
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            e1.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1) * 1e-3)
        t = sum(times) / len(times)
        if world > 1:
            tt = torch.tensor([t], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t, float(loss.item())

    tokens = world * batch * seq
    res = {"workload": f"config 4 shape ({shape}: d_model {cfg['d']}, FFN {cfg['ffn']}), {n_layers} of "
                       f"{full_layers} layers, batch {batch} x {seq} random tokens per GPU, AdamW lr "
                       f"1e-4, precision {precision}, {world} GPU(s); Hugging Face LlamaForCausalLM",
           "layers": n_layers, "of_layers": full_layers, "n_gpus": world}
    dense = build()
    wrapped = (torch.nn.parallel.DistributedDataParallel(dense, device_ids=[torch.cuda.current_device()])
               if world > 1 else dense)
    opt = torch.optim.AdamW(dense.parameters(), lr=1e-4)
    t, loss = run(wrapped, opt)
    res["dense_tok_s"] = round(tokens / t, 1)
    res["dense_loss"] = loss
    del dense, wrapped, opt
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    model = build()
    manager = neuzip.Manager(precision=precision)
    manager.convert(model)
    torch.cuda.empty_cache()
    # moments in bf16, as torch.optim.AdamW keeps them for bf16 parameters
    opt = CompressedAdamW(model.parameters(), lr=1e-4, state_dtype=torch.bfloat16)
    t, loss = run(model, opt)
    manager.check()
    res["neuzip_tok_s"] = round(tokens / t, 1)
    res["neuzip_loss"] = loss
    # the same with the update fused into the decode kernel (one library call per weight)
    # instead of the optimiser's three separate calls (decode, update kernel, compress)
    opt.fused_update = True
    t, _ = run(model, opt, warmup=1)
    res["neuzip_fused_update_tok_s"] = round(tokens / t, 1)
    res["neuzip_peak_bytes"] = torch.cuda.max_memory_allocated()
    res["ratio_vs_dense_tok_s"] = round(res["neuzip_tok_s"] / res["dense_tok_s"], 3)
    if world > 1:
        h = list(manager.meta_dict)[len(manager.meta_dict) // 2]
        w = manager.read(h).view(torch.int16).to(torch.int64).sum().reshape(1)
        lo, hi = w.clone(), w.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        res["replicas_identical"] = bool((lo == hi).item())
    del model, opt
    torch.cuda.empty_cache()
    return res


def tp_leg(n_layers=80, full_layers=80, shape="70b", batch=1, prompt_len=512, new_tokens=32,
           precision=3):
    """Configuration 5: tensor-parallel decode.  Every rank builds each layer whole (same
    seeds), converts it with Manager.convert(tp_rank, tp_world) -- which keeps the rank's
    rows (q, k, v, gate, up) or columns (o, down) and all-reduces after the row-parallel
    Linears -- and frees the dense layer; the dense baseline keeps the same slices
    uncompressed."""
    import torch.distributed as dist
    import neuzip
    from neuzip_b200 import layerwise, sharding
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    cfg = SHAPES[shape]
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg["vocab"], (batch, prompt_len), generator=g).cuda()
    res = {"workload": f"config 5 shape ({shape}), {n_layers} of {full_layers} layers, TP={world}, batch "
                       f"{batch}, {prompt_len}-token random prompt, {new_tokens} greedy tokens, precision "
                       f"{precision}", "tp": world, "layers": n_layers, "of_layers": full_layers}

    class ReducedLinear(torch.nn.Module):
        """Dense row-parallel Linear of the baseline: partial sums, then one all-reduce."""

        def __init__(self, lin):
            super().__init__()
            self.lin = lin

        def forward(self, x):
            y = self.lin(x)
            if world > 1:
                dist.all_reduce(y)
            return y

    def dense_shard(block):
        for name, child in list(block.named_children()):
            mode = sharding.tp_mode(name)
            if mode is None or world == 1 or not isinstance(child, torch.nn.Linear):
                continue
            w, _ = sharding.shard_linear_weight(child.weight.data, None, mode, rank, world)
            lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device="cuda", dtype=torch.bfloat16)
            lin.weight.data = w
            setattr(block, name, ReducedLinear(lin) if mode == "row" else lin)

    def build(compressed, manager=None):
        model = MiniLlama(cfg, 0, prompt_len + new_tokens + 8, batch)
        for l in range(n_layers):
            block = Block(cfg, l)
            if compressed:
                manager.convert(block, tp_rank=rank, tp_world=world)
            else:
                dense_shard(block)
            model.layers.append(block)
        model.allocate_cache(cfg["kv_heads"] // world)
        return model

    model = build(False)
    dec = Decoder(model, prompt, new_tokens)
    dec.run()
    ref, t = dec.run()
    res["dense_eager_ms_per_token"] = round(t * 1e3, 2)
    res["dense_eager_tok_s"] = round(batch / t, 2)
    del model, dec
    torch.cuda.empty_cache()
    manager = neuzip.Manager(precision=precision)
    model = build(True, manager)
    manager._be.settle_all()
    manager._be.release_scratch()
    torch.cuda.empty_cache()
    res["stored_weight_bytes_per_rank"] = manager.total_size()
    hooks = layerwise.attach(model, manager)
    dec = Decoder(model, prompt, new_tokens)
    dec.run()
    out, t = dec.run()
    manager.check()
    res["neuzip_eager_ms_per_token"] = round(t * 1e3, 2)
    res["neuzip_eager_tok_s"] = round(batch / t, 2)
    res["ratio_vs_dense_tok_s"] = round(res["neuzip_eager_tok_s"] / res["dense_eager_tok_s"], 3)
    res["tokens_identical_to_dense"] = bool(torch.equal(out, ref))       # lossy: may differ
    if world > 1:
        # the same with o_proj left out of the per-block decode: its row-parallel shard adds
        # over the ranks inside the fused linear kernel (peer stores) instead of NCCL
        for h in hooks:
            h.remove()
        for block in model.layers:
            for lin in block.modules():
                if isinstance(lin, neuzip.nn.Linear):
                    lin._p._staged, lin._p._stage_tag = None, None
        manager.fuse_tp_allreduce(None, max_rows=256)
        layerwise.attach(model, manager, exclude=lambda lin: any(lin is b.o_proj for b in model.layers))
        dec = Decoder(model, prompt, new_tokens)
        dec.run()
        out2, t = dec.run()
        manager.check()
        res["neuzip_fused_allreduce_o_proj_tok_s"] = round(batch / t, 2)
        res["fused_allreduce_tokens_equal_fraction"] = round(float((out2 == out).float().mean().item()), 4)
        manager.fuse_tp_allreduce(None, max_rows=0)
    res["peak_memory_bytes"] = torch.cuda.max_memory_allocated()
    return res


def tp_linear_leg(n_layers=0, full_layers=0, shape="70b", batch=16, precision=7, iters=30, **_):
    """The row-parallel Linears of one layer (o_proj, down_proj) as operators, `batch` input
    rows, three ways: (a) decode to bf16, library GEMM, NCCL all-reduce -- the default path;
    (b) the fused decode -> tensor-core linear, then NCCL all-reduce; (c) the fused linear whose
    epilogue stores the partial sums into every rank's memory and adds them (no collective
    call).  Device time per call (CUDA events around `iters` calls, max over ranks); every
    shard is larger than L2, so each call streams it from HBM."""
    import torch.distributed as dist
    import neuzip
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    cfg = SHAPES[shape]
    res = {"workload": f"row-parallel Linears of a {shape}-shape layer, TP={world}, {batch} input rows, "
                       f"precision {precision}", "tp": world, "rows": batch, "cases": []}
    if world < 2:
        res["skipped"] = "needs at least two ranks"
        return res
    manager = neuzip.Manager(precision=precision)
    gen = torch.Generator(device="cuda").manual_seed(3)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            y = fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return y, round(t.item(), 1)

    for name, out_f, in_f in (("o_proj", cfg["d"], cfg["d"]),
                              ("down_proj", cfg["d"], cfg["ffn"])):
        shard = in_f // world
        lin = torch.nn.Linear(shard, out_f, bias=False, device="cuda", dtype=torch.bfloat16)
        lin.weight.data.normal_(0, 0.02, generator=gen)
        layer = neuzip.nn.Linear(manager, lin, tp=("row", 0, 1, None))     # already this rank's block
        layer.reduce_output = True
        del lin
        x = torch.randn(batch, shard, device="cuda", dtype=torch.bfloat16, generator=gen)
        case = {"linear": name, "shard": [out_f, shard]}
        with torch.no_grad():
            manager.fuse_linear(0)
            manager.fuse_tp_allreduce(None, max_rows=0)
            layer.reduce_output = False
            _, case["decode_gemm_only_us"] = timed(lambda: layer(x))
            layer.reduce_output = True
            y0, case["decode_gemm_nccl_us"] = timed(lambda: layer(x))
            manager.fuse_linear(256)
            layer.reduce_output = False
            _, case["fused_linear_only_us"] = timed(lambda: layer(x))
            layer.reduce_output = True
            y1, case["fused_linear_nccl_us"] = timed(lambda: layer(x))
            manager.fuse_tp_allreduce(None, max_rows=256)
            y2, case["fused_linear_allreduce_us"] = timed(lambda: layer(x))
            manager.check()
            manager.fuse_tp_allreduce(None, max_rows=0)
            manager.fuse_linear(0)
        want = y2.float()
        case["max_abs_diff_vs_default"] = round((y0.float() - want).abs().max().item(), 5)
        case["output_abs_max"] = round(want.abs().max().item(), 3)
        res["cases"].append(case)
        del layer
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("leg", choices=["decode", "train", "tp", "tp_linear"])
    ap.add_argument("--layers", type=int, default=0, help="0 = the configuration's own count")
    ap.add_argument("--shape", default=None)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--precision", type=int, default=-1)
    ap.add_argument("--new", type=int, default=0)
    args = ap.parse_args()
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    kw = {}
    if args.batch:
        kw["batch"] = args.batch
    if args.precision >= 0:
        kw["precision"] = args.precision
    if args.new and args.leg != "train":
        kw["new_tokens"] = args.new
    shape = args.shape or {"decode": "7b", "train": "1.3b", "tp": "70b", "tp_linear": "70b"}[args.leg]
    full = SHAPES[shape]["layers"]
    fn = {"decode": decode_leg, "train": train_leg, "tp": tp_leg, "tp_linear": tp_linear_leg}[args.leg]
    res = fn(n_layers=args.layers or full, full_layers=full, shape=shape, **kw)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
