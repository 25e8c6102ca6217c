#!/usr/bin/env python
"""Model-level check of the codec: a random-init Llama-architecture model,
dense vs. converted with neuzip.Manager (configurations 3 and 4 of the benchmark list).

    python bench_llama.py --config 7b --prompt 128 --new 256 [--precision 7]

Builds the model with linear weights N(0, 0.02) (transformers' initialiser;
synthetic stand-in for the Llama checkpoints), times greedy decoding dense,
converts it in place, times it again per-Linear and with layer-wise batched
decode, and reports tokens/s, logits difference, token agreement and stored
bytes as one JSON line.
"""
import argparse
import json
import time

import torch

CONFIGS = {
    "tiny": dict(hidden_size=256, intermediate_size=704, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=4),
    "1.3b": dict(hidden_size=2048, intermediate_size=5504, num_hidden_layers=24,
                 num_attention_heads=16, num_key_value_heads=16),
    "7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
               num_attention_heads=32, num_key_value_heads=32),
}


def timed_generate(model, ids, new_tokens):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=new_tokens, min_new_tokens=new_tokens,
                             do_sample=False, pad_token_id=0)
    e1.record()
    torch.cuda.synchronize()
    return out, e0.elapsed_time(e1) * 1e-3, time.perf_counter() - t0


def train_mode(args):
    """Configuration 4 of the benchmark list: AdamW training with lossless compressed weights,
    per-layer decode in forward and backward, data-parallel over the ranks."""
    import os
    import torch.distributed as dist
    import transformers
    import neuzip
    from neuzip_b200.optim import CompressedAdamW

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = transformers.LlamaConfig(vocab_size=32000, max_position_embeddings=4096,
                                   rms_norm_eps=1e-5, **CONFIGS[args.config])

    def build():
        torch.manual_seed(0)
        with torch.device("cuda"):
            return transformers.LlamaForCausalLM(cfg).to(torch.bfloat16)

    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 32000, (args.batch, args.seq), generator=g).cuda()

    def run(model, opt, steps, warmup):
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

    res = {"mode": "train", "config": args.config, "batch_per_gpu": args.batch, "seq": args.seq,
           "n_gpus": world, "steps": args.steps, "data": "synthetic", "precision": args.precision}
    tokens = world * args.batch * args.seq

    if not args.skip_dense:
        dense = build()
        if world > 1:
            dense_ddp = torch.nn.parallel.DistributedDataParallel(dense, device_ids=[local])
        else:
            dense_ddp = dense
        opt = torch.optim.AdamW(dense.parameters(), lr=1e-4)
        t, loss = run(dense_ddp, opt, args.steps, 2)
        res["dense_tok_s"] = tokens / t
        res["dense_loss"] = loss
        res["dense_peak_bytes"] = torch.cuda.max_memory_allocated()
        del dense, dense_ddp, opt
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()

    model = build()
    manager = neuzip.Manager(precision=args.precision)
    manager.convert(model)
    torch.cuda.empty_cache()
    # moments in bf16, as torch.optim.AdamW keeps them for bf16 parameters
    opt = CompressedAdamW(model.parameters(), lr=1e-4, state_dtype=torch.bfloat16)
    t, loss = run(model, opt, args.steps, 2)
    manager.check()
    res["neuzip_tok_s"] = tokens / t
    res["neuzip_loss"] = loss
    res["neuzip_peak_bytes"] = torch.cuda.max_memory_allocated()
    if "dense_tok_s" in res:
        res["ratio_vs_dense_tok_s"] = res["neuzip_tok_s"] / res["dense_tok_s"]
    if world > 1:
        # replicas must hold bit-identical compressed weights after the updates
        h = list(manager.meta_dict)[len(manager.meta_dict) // 2]
        w = manager.read(h).view(torch.int16).to(torch.int64).sum().reshape(1)
        lo, hi = w.clone(), w.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        res["replicas_identical"] = bool((lo == hi).item())
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--train", action="store_true")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--config", default="7b", choices=sorted(CONFIGS))
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--precision", type=int, default=7)
    args = ap.parse_args()
    if args.train:
        return train_mode(args)

    import transformers
    import neuzip
    from neuzip_b200 import layerwise

    cfg = transformers.LlamaConfig(vocab_size=32000, max_position_embeddings=4096,
                                   rms_norm_eps=1e-5, **CONFIGS[args.config])
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16)
    model.eval()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 32000, (args.batch, args.prompt), generator=g).cuda()

    res = {"config": args.config, "precision": args.precision, "batch": args.batch,
           "prompt": args.prompt, "new_tokens": args.new, "data": "synthetic"}
    dense_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    res["dense_param_bytes"] = dense_bytes

    timed_generate(model, ids, 8)                                   # warm-up
    with torch.no_grad():
        ref_logits = model(ids).logits.float()
    ref_out, t_first, _ = timed_generate(model, ids, args.new)
    ref_out, t_gpu, _ = timed_generate(model, ids, args.new)      # second run: allocator and
    res["dense_tok_s_first_run"] = args.batch * args.new / t_first  # library heuristics are warm
    res["dense_tok_s"] = args.batch * args.new / t_gpu
    torch.cuda.reset_peak_memory_stats()

    manager = neuzip.Manager(precision=args.precision)
    t0 = time.perf_counter()
    manager.convert(model)
    torch.cuda.synchronize()
    res["convert_s"] = time.perf_counter() - t0
    manager._be.release_scratch()
    torch.cuda.empty_cache()
    stored = manager.total_size()
    converted_dense = sum(int(torch.Size(s).numel()) * 2 for s in manager.meta_dict.values())
    res["converted_tensors"] = len(manager.meta_dict)
    res["ratio_converted_weights"] = stored / converted_dense
    res["model_bytes_after"] = dense_bytes - converted_dense + stored

    timed_generate(model, ids, 8)
    with torch.no_grad():
        logits = model(ids).logits.float()
    out, t_gpu, _ = timed_generate(model, ids, args.new)
    out, t_gpu, _ = timed_generate(model, ids, args.new)
    manager.check()
    res["neuzip_tok_s"] = args.batch * args.new / t_gpu
    res["max_abs_logit_diff"] = (logits - ref_logits).abs().max().item()
    res["tokens_identical"] = bool(torch.equal(out, ref_out))

    hooks = layerwise.attach(model, manager)
    timed_generate(model, ids, 8)
    out2, t_gpu, _ = timed_generate(model, ids, args.new)
    out2, t_gpu, _ = timed_generate(model, ids, args.new)
    manager.check()
    res["neuzip_layerwise_tok_s"] = args.batch * args.new / t_gpu
    res["layerwise_tokens_identical"] = bool(torch.equal(out2, ref_out))
    res["layerwise_blocks"] = len(hooks) // 2
    res["peak_memory_bytes_compressed_run"] = torch.cuda.max_memory_allocated()
    res["ratio_vs_dense_tok_s"] = res["neuzip_layerwise_tok_s"] / res["dense_tok_s"]

    # single-token steps multiply while decoding (no bf16 write-back); the prompt keeps
    # the batched decode.  Same fp32 arithmetic, different order of the sums.
    if args.batch == 1:
        for h in hooks:
            h.remove()
        layerwise.attach(model, manager, fuse_single_token=True)
        timed_generate(model, ids, 8)
        out3, t_gpu, _ = timed_generate(model, ids, args.new)
        out3, t_gpu, _ = timed_generate(model, ids, args.new)
        manager.check()
        res["neuzip_fused_tok_s"] = args.batch * args.new / t_gpu
        res["fused_tokens_equal_fraction"] = float((out3 == ref_out).float().mean().item())
        res["fused_ratio_vs_dense_tok_s"] = res["neuzip_fused_tok_s"] / res["dense_tok_s"]
    print(json.dumps(res))


if __name__ == "__main__":
    main()
