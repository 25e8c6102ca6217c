#!/usr/bin/env python
"""Tensor-parallel Llama-architecture decode with compressed weights
(the 70B inference configuration of the benchmark list: 70B, 80 layers, d_model 8192, 64 heads / 8 KV heads,
FFN 28672, vocab 32000, precision 3), dense vs. neuzip, on the ranks of one node.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        bench_llama_tp.py --config 70b --batch 1 --prompt 512 --new 32

Sharding: q/k/v/gate/up are column-parallel (each rank holds a block of output
rows), o/down are row-parallel (each rank holds a block of input columns and
compresses its own contiguous [out, in/t] copy); one NCCL all-reduce of the
[batch, d_model] activations follows o_proj and down_proj.  The codec itself
never communicates.  Weights are random (N(0, 0.02), seeded per layer, matrix
and rank): a synthetic stand-in for the Llama checkpoints.
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

CONFIGS = {
    "tiny": dict(layers=2, d=512, heads=8, kv_heads=4, ffn=1408, vocab=1024),
    "7b": dict(layers=32, d=4096, heads=32, kv_heads=32, ffn=11008, vocab=32000),
    "70b": dict(layers=80, d=8192, heads=64, kv_heads=8, ffn=28672, vocab=32000),
}


def shard_linear(out_f, in_f, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    lin = torch.nn.Linear(in_f, out_f, bias=False, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(out_f, in_f, generator=g, device="cuda") * 0.02)
                         .to(torch.bfloat16))
    return lin


class TPDecoderLayer(torch.nn.Module):
    def __init__(self, cfg, layer, rank, world):
        super().__init__()
        d, hd = cfg["d"], cfg["d"] // cfg["heads"]
        self.h, self.kvh, self.hd = cfg["heads"] // world, cfg["kv_heads"] // world, hd
        s = 100000 * layer + 1000 * rank
        self.q_proj = shard_linear(self.h * hd, d, s + 1)
        self.k_proj = shard_linear(self.kvh * hd, d, s + 2)
        self.v_proj = shard_linear(self.kvh * hd, d, s + 3)
        self.o_proj = shard_linear(d, self.h * hd, s + 4)
        self.gate_proj = shard_linear(cfg["ffn"] // world, d, s + 5)
        self.up_proj = shard_linear(cfg["ffn"] // world, d, s + 6)
        self.down_proj = shard_linear(d, cfg["ffn"] // world, s + 7)
        self.norm1 = torch.nn.RMSNorm(d, eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.norm2 = torch.nn.RMSNorm(d, eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.world = world
        self.k_cache = None
        self.v_cache = None

    def forward(self, x, cos, sin, pos):
        B, T, _ = x.shape
        h = self.norm1(x)
        q = self.q_proj(h).view(B, T, self.h, self.hd).transpose(1, 2)
        k = self.k_proj(h).view(B, T, self.kvh, self.hd).transpose(1, 2)
        v = self.v_proj(h).view(B, T, self.kvh, self.hd).transpose(1, 2)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        self.k_cache[:, :, pos:pos + T] = k
        self.v_cache[:, :, pos:pos + T] = v
        kk, vv = self.k_cache[:, :, :pos + T], self.v_cache[:, :, :pos + T]
        att = F.scaled_dot_product_attention(q, kk, vv, is_causal=(T > 1), enable_gqa=True)
        o = self.o_proj(att.transpose(1, 2).reshape(B, T, self.h * self.hd))
        if self.world > 1:
            dist.all_reduce(o)
        x = x + o
        h = self.norm2(x)
        m = self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))
        if self.world > 1:
            dist.all_reduce(m)
        return x + m


def rope(x, cos, sin):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class TPModel(torch.nn.Module):
    def __init__(self, cfg, rank, world, max_len, batch):
        super().__init__()
        self.cfg = cfg
        g = torch.Generator(device="cuda").manual_seed(7)
        self.embed = (torch.randn(cfg["vocab"], cfg["d"], generator=g, device="cuda") * 0.02
                      ).to(torch.bfloat16)
        self.lm_head = shard_linear(cfg["vocab"], cfg["d"], 8)     # replicated, never converted
        self.norm = torch.nn.RMSNorm(cfg["d"], eps=1e-5, device="cuda", dtype=torch.bfloat16)
        self.layers = torch.nn.ModuleList(
            [TPDecoderLayer(cfg, l, rank, world) for l in range(cfg["layers"])])
        hd = cfg["d"] // cfg["heads"]
        inv = 1.0 / (10000 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
        t = torch.arange(max_len, device="cuda").float()
        fr = torch.outer(t, inv)
        self.cos, self.sin = fr.cos().to(torch.bfloat16), fr.sin().to(torch.bfloat16)
        for layer in self.layers:
            layer.k_cache = torch.zeros(batch, layer.kvh, max_len, hd, device="cuda", dtype=torch.bfloat16)
            layer.v_cache = torch.zeros_like(layer.k_cache)

    @torch.no_grad()
    def forward(self, ids, pos):
        x = self.embed[ids]
        T = ids.shape[1]
        cos, sin = self.cos[pos:pos + T], self.sin[pos:pos + T]
        for layer in self.layers:
            x = layer(x, cos, sin, pos)
        return self.lm_head(self.norm(x[:, -1:]))


@torch.no_grad()
def generate(model, prompt, new_tokens):
    logits = model(prompt, 0)
    tok = logits.argmax(-1).view(-1, 1)
    out = [tok]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pos = prompt.shape[1]
    for _ in range(new_tokens - 1):
        logits = model(tok, pos)
        tok = logits.argmax(-1).view(-1, 1)
        out.append(tok)
        pos += 1
    e1.record()
    torch.cuda.synchronize()
    return torch.cat(out, 1), e0.elapsed_time(e1) * 1e-3 / max(1, new_tokens - 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="70b", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=32)
    ap.add_argument("--precision", type=int, default=3)
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--fused", action="store_true",
                    help="single-token steps multiply while decoding (batch 1 only)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import neuzip
    from neuzip_b200 import layerwise

    cfg = CONFIGS[args.config]
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg["vocab"], (args.batch, args.prompt), generator=g).cuda()
    max_len = args.prompt + args.new + 1
    res = {"mode": "tp_decode", "config": args.config, "tp": world, "batch": args.batch,
           "prompt": args.prompt, "new_tokens": args.new, "precision": args.precision,
           "data": "synthetic"}

    t0 = time.perf_counter()
    model = TPModel(cfg, rank, world, max_len, args.batch)
    torch.cuda.synchronize()
    res["build_s"] = time.perf_counter() - t0
    res["dense_weight_bytes_per_rank"] = sum(p.numel() * 2 for l in model.layers
                                             for p in l.parameters() if p.dim() == 2)
    ref_out = None
    if not args.skip_dense:
        generate(model, prompt, args.new)                      # warm-up: allocator, library heuristics
        ref_out, t_tok = generate(model, prompt, args.new)
        res["dense_ms_per_token"] = t_tok * 1e3
        res["dense_tok_s"] = args.batch / t_tok

    manager = neuzip.Manager(precision=args.precision)
    t0 = time.perf_counter()
    for layer in model.layers:
        manager.convert(layer)
    torch.cuda.synchronize()
    res["convert_s"] = time.perf_counter() - t0
    manager._be.release_scratch()
    torch.cuda.empty_cache()
    res["stored_weight_bytes_per_rank"] = manager.total_size()
    layerwise.attach(model, manager, fuse_single_token=args.fused and args.batch == 1)
    res["fused_single_token"] = bool(args.fused and args.batch == 1)
    generate(model, prompt, args.new)
    out, t_tok = generate(model, prompt, args.new)
    manager.check()
    res["neuzip_ms_per_token"] = t_tok * 1e3
    res["neuzip_tok_s"] = args.batch / t_tok
    if "dense_tok_s" in res:
        res["ratio_vs_dense_tok_s"] = res["neuzip_tok_s"] / res["dense_tok_s"]
    if ref_out is not None:
        res["tokens_identical_to_dense"] = bool(torch.equal(out, ref_out))   # lossy: may differ
    res["peak_memory_bytes"] = torch.cuda.max_memory_allocated()
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
