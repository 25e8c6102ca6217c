"""GPU tests of the public Python API (Manager, nn, ops, hooks) on the CUDA
backend: what a user of the reference's package would run."""
import numpy as np
import pytest
import torch

import neuzip
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def bits_of(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)


def weights(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)


@pytest.mark.parametrize("precision", (0, 1, 3, 7))
def test_write_read_matches_oracle(precision):
    m = neuzip.Manager(precision=precision)
    w = weights((300, 517), 1)                      # not a multiple of anything
    h = m.write(w)                                   # CPU tensor is moved to the GPU
    got = m.read(h)
    m.check()
    assert got.is_cuda and got.shape == w.shape and got.dtype == torch.bfloat16
    assert not got.requires_grad
    e, f = O.split(bits_of(w), precision)
    ref = O.merge(e, f, precision, canonical_nan=True)
    assert np.array_equal(bits_of(got), ref)
    entry = m._be.entry(h)
    assert m.size(h) == entry.container.numel() + entry.fractions.numel()
    assert m.size("nope") == 0


def test_rewrite_same_handle_and_many_tensors():
    m = neuzip.Manager()
    ws = [weights((64 + 8 * i, 96), 10 + i).cuda() for i in range(5)]
    hs = [m.write(w) for w in ws]
    assert hs == [str(i) for i in range(5)]
    for h, w in zip(hs, ws):
        assert torch.equal(m.read(h), w)
    w_new = weights((7, 9), 99).cuda()
    assert m.write(w_new, hs[2]) == hs[2]
    assert torch.equal(m.read(hs[2]), w_new)
    m.check()


def test_split_is_full_precision_regardless_of_manager_precision():
    w = weights((128, 130), 3).cuda()
    for precision in (7, 1):
        e, f = neuzip.Manager(precision=precision).split(w)
        assert e.shape == w.shape and f.shape == w.shape and e.dtype == torch.uint8
        er, fr = O.split(bits_of(w), 7)
        assert np.array_equal(e.cpu().numpy().reshape(-1), er)
        assert np.array_equal(f.cpu().numpy().reshape(-1), fr)


def test_errors_follow_the_reference():
    m = neuzip.Manager()
    with pytest.raises(RuntimeError, match="Unsupported data type"):
        m.write(torch.zeros(8, 8, dtype=torch.float32))
    with pytest.raises(KeyError):
        m.read("7")
    with pytest.raises(RuntimeError, match="Data not found"):
        m._be.read("7")


def test_linear_with_and_without_bias():
    m = neuzip.Manager()
    w = weights((48, 64), 4).cuda()
    b = weights((48,), 5).cuda()
    h = m.write(w)
    x = weights((3, 5, 64), 6).cuda()
    y = m.linear(h, x)
    assert torch.allclose(y.float(), torch.matmul(x, w.t()).float(), atol=1e-3, rtol=1e-2)
    y2 = m.linear(h, x.reshape(-1, 64), b)
    ref2 = torch.nn.functional.linear(x.reshape(-1, 64), w, b)
    assert torch.allclose(y2.float(), ref2.float(), atol=1e-3, rtol=1e-2)


def test_dummy_backend_round_trip():
    m = neuzip.Manager(algorithm=neuzip.Algorithm.dummy)
    w = weights((16, 32), 7)
    h = m.write(w)
    assert torch.equal(m.read(h).cpu(), w)
    assert m.size(h) == w.numel() * 2
    x = weights((4, 32), 8).cuda()
    assert m.linear(h, x).shape == (4, 16)


def test_compressed_linear_training_step_matches_dense():
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 32, bias=True).to(torch.bfloat16)
    dense = torch.nn.Linear(64, 32, bias=True).to(torch.bfloat16)
    dense.load_state_dict(lin.state_dict())
    dense = dense.cuda()
    m = neuzip.Manager()
    model = m.convert(torch.nn.Sequential(lin)).cuda()
    x = torch.randn(10, 64, device="cuda", dtype=torch.bfloat16)

    class Sched:
        def get_last_lr(self):
            return [0.25]

    sched = Sched()
    p = model[0]._p
    p.register_post_accumulate_grad_hook(lambda q: neuzip.compressed_lomo_hook(sched, q))
    y = model(x)
    yd = dense(x)
    assert torch.equal(y, yd)                         # lossless weight, same GEMM
    y.float().pow(2).mean().backward()
    yd.float().pow(2).mean().backward()
    expect = dense.weight.data.clone()
    expect.add_(dense.weight.grad, alpha=-0.25)
    assert p._gradient is None                        # consumed by the hook
    assert torch.equal(p(), expect)                   # read -> update -> write round trip
    assert torch.allclose(model[0].bias.grad.float(), dense.bias.grad.float(), atol=1e-3)
    m.check()


def test_convert_tiny_llama_logits_and_greedy_tokens():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=352,
                                   num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=4, max_position_embeddings=128)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (1, 16), device="cuda")
    with torch.no_grad():
        ref_logits = model(ids).logits
        ref_tokens = model.generate(ids, max_new_tokens=8, do_sample=False)
    m = neuzip.Manager()
    m.convert(model)
    n_converted = sum(isinstance(mod, neuzip.nn.Linear) for mod in model.modules())
    assert n_converted == 2 * 7                      # q,k,v,o,gate,up,down per layer; lm_head kept
    assert isinstance(model.lm_head, torch.nn.Linear)
    with torch.no_grad():
        logits = model(ids).logits
        tokens = model.generate(ids, max_new_tokens=8, do_sample=False)
    m.check()
    assert (logits.float() - ref_logits.float()).abs().max().item() <= 1e-2
    assert torch.equal(tokens, ref_tokens)
    dense_bytes = sum(int(np.prod(s)) * 2 for s in m.meta_dict.values())
    assert m.total_size() < 0.75 * dense_bytes


def test_lossy_precision_error_bounds():
    w = weights((256, 256), 11).cuda()
    bounds = {0: 0.03125, 1: 0.015625, 3: 0.00390625}
    for precision, bound in bounds.items():
        m = neuzip.Manager(precision=precision)
        got = m.read(m.write(w))
        assert (got.float() - w.float()).abs().max().item() <= bound


def test_read_many_matches_read():
    m = neuzip.Manager(precision=3)
    ws = [weights(shape, 40 + i) for i, shape in enumerate([(256, 256), (704, 256), (256, 704),
                                                            (3, 5), (1024, 512)])]
    hs = [m.write(w) for w in ws]
    many = m.read_many(hs)
    for h, t in zip(hs, many):
        assert t.shape == m.meta_dict[h]
        assert torch.equal(t, m.read(h))
    m.check()


def test_layerwise_prefetch_gives_identical_outputs_and_gradients():
    transformers = pytest.importorskip("transformers")
    from neuzip_b200 import layerwise
    cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=128, intermediate_size=352,
                                   num_hidden_layers=3, num_attention_heads=4,
                                   num_key_value_heads=4, max_position_embeddings=64)
    torch.manual_seed(1)
    model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).cuda()
    m = neuzip.Manager()
    m.convert(model)
    ids = torch.randint(0, 256, (2, 12), device="cuda")
    with torch.no_grad():
        ref = model(ids).logits
    loss = model(ids, labels=ids).loss
    loss.backward()
    ref_grads = [p._gradient.clone() for p in model.parameters() if hasattr(p, "_gradient")]
    for p in model.parameters():
        if hasattr(p, "_gradient"):
            p._gradient = None
    hooks = layerwise.attach(model, m)
    assert len(hooks) == 6
    with torch.no_grad():
        got = model(ids).logits
    assert torch.equal(got, ref)
    model(ids, labels=ids).loss.backward()           # backward decodes on its own
    grads = [p._gradient for p in model.parameters() if hasattr(p, "_gradient")]
    assert len(grads) == len(ref_grads) == 21
    for a, b in zip(grads, ref_grads):
        assert torch.equal(a, b)
    for h in hooks:
        h.remove()
    m.check()


def test_compressed_adamw_matches_a_dense_restatement():
    from neuzip_b200.optim import CompressedAdamW
    torch.manual_seed(2)
    lin = torch.nn.Linear(48, 32, bias=True).to(torch.bfloat16)
    w = lin.weight.data.clone().cuda()
    m = neuzip.Manager()
    model = m.convert(torch.nn.Sequential(lin)).cuda()
    opt = CompressedAdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
    mom = torch.zeros(32, 48, device="cuda")
    var = torch.zeros(32, 48, device="cuda")
    for step in range(1, 4):
        x = torch.randn(6, 48, device="cuda", dtype=torch.bfloat16)
        y = model(x)
        gy = torch.randn_like(y)
        y.backward(gy)
        g = torch.mm(gy.t(), x).float()
        opt.step()
        opt.zero_grad()
        mom.mul_(0.9).add_(g, alpha=0.1)
        var.mul_(0.999).addcmul_(g, g, value=0.001)
        wf = w.float() * (1 - 1e-2 * 0.1)
        wf.addcdiv_(mom, (var / (1 - 0.999 ** step)).sqrt() + 1e-8, value=-1e-2 / (1 - 0.9 ** step))
        w = wf.to(torch.bfloat16)
        # fused kernel vs. this restatement: same formula, fp32 throughout; allow one bf16 ulp
        got = model[0]._p()
        assert (got.float() - w.float()).abs().max().item() <= 2.0 ** -8 * w.float().abs().max().item()
        w = got.clone()
    m.check()


def test_checkpoint_of_converted_model_round_trips_on_gpu(tmp_path):
    torch.manual_seed(5)
    def make():
        return torch.nn.Sequential(torch.nn.Linear(96, 64, bias=True), torch.nn.ReLU(),
                                   torch.nn.Linear(64, 32, bias=False)).to(torch.bfloat16)
    src = make()
    m1 = neuzip.Manager(precision=3)
    m1.convert(src)
    src.cuda()
    x = torch.randn(4, 96, device="cuda", dtype=torch.bfloat16)
    expect = src(x)
    torch.save(src.state_dict(), tmp_path / "c.pt")
    dst = make()
    m2 = neuzip.Manager(precision=3)
    m2.convert(dst)
    dst.cuda()
    dst.load_state_dict(torch.load(tmp_path / "c.pt", weights_only=False))
    assert torch.equal(dst(x), expect)
    m2.check()
    wrong = neuzip.Manager(precision=7)
    other = wrong.convert(make()).cuda()
    with pytest.raises(Exception):
        other.load_state_dict(torch.load(tmp_path / "c.pt", weights_only=False))


@pytest.mark.parametrize("precision,group", ((3, 512), (1, 64), (0, 1024), (7, 8), (3, 1)))
def test_manager_with_block_normaliser_matches_oracle(precision, group):
    m = neuzip.Manager(precision=precision, normalizer_size=group)
    w = weights((257, 300), 60 + group)
    h = m.write(w)
    got = m.read(h)
    m.check()
    scaled, norm = O.normalize_groups(bits_of(w), group)
    e, f = O.split(scaled, precision)
    ref = O.denormalize_groups(O.merge(e, f, precision, canonical_nan=True), group, norm)
    assert np.array_equal(bits_of(got), ref)
    entry = m._be.entry(h)
    assert m.size(h) == entry.container.numel() + entry.fractions.numel() + norm.size
    assert torch.equal(m.read_many([h])[0], got)
    # the normaliser tightens the lossy error
    if precision == 3:
        plain = neuzip.Manager(precision=3)
        err_plain = (plain.read(plain.write(w)).float() - w.cuda().float()).abs().mean().item()
        err_norm = (got.float() - w.cuda().float()).abs().mean().item()
        assert err_norm <= err_plain * 1.05


@pytest.mark.parametrize("precision", (7, 3))
@pytest.mark.parametrize("rows,dim", ((1000, 4096), (333, 16384), (5000, 96), (70, 20000), (32000, 512)))
def test_read_rows_and_embedding_lookup_decode_only_what_they_need(precision, rows, dim):
    """Row gather against indexing the fully decompressed table: rows that share a
    unit, rows made of whole units, and rows that straddle unit boundaries."""
    g = torch.Generator().manual_seed(rows + dim)
    table = (torch.randn(rows, dim, generator=g) * 0.02).to(torch.bfloat16).cuda()
    manager = neuzip.Manager(precision=precision)
    handle = manager.write(table)
    full = manager.read(handle)
    idx = torch.randint(0, rows, (3, 17), generator=g)
    idx[0, 0], idx[0, 1], idx[2, 16] = 0, rows - 1, rows - 1        # first, last, a repeat
    got = manager.read_rows(handle, idx.cuda())
    assert got.shape == (3, 17, dim) and got.dtype == torch.bfloat16
    assert torch.equal(got.view(torch.int16), full[idx.cuda()].view(torch.int16))
    assert manager.read_rows(handle, torch.zeros(0, dtype=torch.long)).shape == (0, dim)
    manager.check()
    emb = torch.nn.Embedding(rows, dim, padding_idx=1).to(torch.bfloat16).cuda()
    with torch.no_grad():
        emb.weight.copy_(table)
    ce = neuzip.nn.Embedding(manager, emb)
    ref = torch.nn.functional.embedding(idx.cuda(), manager.read(ce._p._handle))
    assert torch.equal(ce(idx.cuda()).view(torch.int16), ref.view(torch.int16))


def test_read_rows_reports_rows_outside_the_table():
    table = weights((4000, 512), 8).cuda()
    manager = neuzip.Manager(precision=7)
    handle = manager.write(table)
    got = manager.read_rows(handle, torch.tensor([3, 4000, 7]).cuda())
    assert torch.equal(got[0].view(torch.int16), table[3].view(torch.int16))
    assert torch.equal(got[2].view(torch.int16), table[7].view(torch.int16))
    with pytest.raises(RuntimeError):
        manager.check()


@pytest.mark.parametrize("group", (1, 4, 64, 512, 1024))
def test_read_rows_with_block_normaliser_decodes_only_the_rows(group):
    """The decoder applies the group scales itself, so a row gather on a normalised
    table needs no full read; rows, a batched read and a plain read agree with the
    oracle (decode, merge, then the scaling of cuda/kernels.cuh:208-216)."""
    g = torch.Generator().manual_seed(3)
    table = (torch.randn(600, 1024, generator=g) * 0.02).to(torch.bfloat16).cuda()
    odd = (torch.randn(3 * 8192 + 777, generator=g) * 0.02).to(torch.bfloat16).cuda()   # ragged tail
    manager = neuzip.Manager(precision=3, normalizer_size=group)
    handle, h_odd = manager.write(table), manager.write(odd)
    for t, h in ((table, handle), (odd, h_odd)):
        scaled, norm = O.normalize_groups(bits_of(t), group)
        e, f = O.split(scaled, 3)
        ref = O.denormalize_groups(O.merge(e, f, 3, canonical_nan=True), group, norm)
        assert np.array_equal(bits_of(manager.read(h)), ref)
    a, b = manager.read_many([handle, h_odd])
    assert torch.equal(a, manager.read(handle)) and torch.equal(b, manager.read(h_odd))
    idx = torch.tensor([5, 599, 0, 5]).cuda()
    assert torch.equal(manager.read_rows(handle, idx).view(torch.int16),
                       manager.read(handle)[idx].view(torch.int16))
    manager.check()


@pytest.mark.parametrize("precision", (7, 3, 1, 0))
@pytest.mark.parametrize("out_f,in_f", ((4096, 4096), (1000, 11008), (11008, 4096), (33, 768),
                                        (5, 256), (257, 28672)))
def test_fused_vector_linear_matches_decode_then_matmul(precision, out_f, in_f):
    w = weights((out_f, in_f), out_f + in_f)
    manager = neuzip.Manager(precision=precision)
    handle = manager.write(w.cuda())
    decoded = manager.read(handle).float()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 1, in_f, generator=g).to(torch.bfloat16).cuda()
    bias = (torch.randn(out_f, generator=g) * 0.1).to(torch.bfloat16).cuda()
    manager.fuse_vector_linear(True)
    for b in (None, bias):
        ref = x.float().reshape(-1) @ decoded.t()                 # fp32 products and sums
        if b is not None:
            ref = ref + b.float()
        got = manager.linear(handle, x, b)
        assert got.shape == (1, 1, out_f) and got.dtype == torch.bfloat16
        # one bf16 rounding of an fp32 sum whose order differs: half an ulp plus summation noise
        err = (got.float().reshape(-1) - ref).abs()
        tol = ref.abs() * 2.0 ** -8 + 1e-3 * decoded.abs().max() * x.float().abs().sum() / in_f ** 0.5
        assert (err <= tol).all(), float((err - tol).max())
        again = manager.linear(handle, x, b)                      # reproducible run to run
        assert torch.equal(got.view(torch.int16), again.view(torch.int16))
    # calls that do not qualify keep the decode + GEMM path, bit for bit
    x2 = torch.randn(2, in_f, generator=g).to(torch.bfloat16).cuda()
    manager.fuse_vector_linear(False)
    plain = manager.linear(handle, x2)
    manager.fuse_vector_linear(True)
    assert torch.equal(manager.linear(handle, x2).view(torch.int16), plain.view(torch.int16))
    manager.check()


def test_fused_vector_linear_with_raw_units_and_short_lanes():
    """Incompressible weights (units stored raw) and a backend with short lane streams
    (units smaller than a row)."""
    rng = np.random.default_rng(3)
    out_f, in_f = 64, 2048
    bits = rng.integers(0, 1 << 16, size=out_f * in_f, dtype=np.uint16)
    bits[(bits & 0x7F80) == 0x7F80] = 0x3C00                      # no inf / NaN
    bits[out_f * in_f // 2:] = bits_of(weights((out_f * in_f // 2,), 4))
    w = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).reshape(out_f, in_f).cuda()
    # keep magnitudes finite for the comparison
    w = torch.where(w.float().abs() < 1e4, w, torch.zeros_like(w))
    for lane_symbols in (None, 64):
        manager = neuzip.Manager(precision=7)
        if lane_symbols:
            manager._be.lane_symbols = lane_symbols
        handle = manager.write(w)
        manager.fuse_vector_linear(True)
        x = torch.randn(in_f, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
        ref = manager.read(handle).float() @ x.float()
        got = manager.linear(handle, x).float()
        assert got.shape == (out_f,)
        assert torch.allclose(got, ref, rtol=2.0 ** -7, atol=1e-2 * float(ref.abs().max()))
        manager.check()


def test_layerwise_fused_single_token_generation():
    """With fuse_single_token the one-token steps of greedy generation multiply while
    decoding; the prompt (many tokens) still takes the batched decode, bit for bit."""
    transformers = pytest.importorskip("transformers")
    from neuzip_b200 import layerwise
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=768,
                                   num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(2)
    model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    m = neuzip.Manager()
    m.convert(model)
    ids = torch.randint(0, 512, (1, 9), device="cuda")
    with torch.no_grad():
        ref_prompt = model(ids).logits
        ref_step = model(ids[:, :1]).logits                      # a one-token call, unfused
    calls = {"n": 0}
    inner = m._be._linear_vec

    def spy(name, input, shape, bias):
        out = inner(name, input, shape, bias)
        calls["n"] += out is not None
        return out

    m._be._linear_vec = spy
    hooks = layerwise.attach(model, m, fuse_single_token=True)
    with torch.no_grad():
        assert torch.equal(model(ids).logits, ref_prompt)        # 9 tokens: batched decode
        assert calls["n"] == 0
        step = model(ids[:, :1]).logits                          # 1 token: fused, 7 Linears x 2 blocks
    assert calls["n"] == 14
    assert torch.allclose(step.float(), ref_step.float(), rtol=0.05, atol=0.05)
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=6, do_sample=False)
    assert out.shape == (1, 15)
    for h in hooks:
        h.remove()
    m.check()


def test_batched_decode_can_be_captured_in_a_cuda_graph():
    """The decode entry points only enqueue work on the caller's stream (no allocation, no
    host synchronisation), so a serving loop can record them in a CUDA graph."""
    manager = neuzip.Manager(precision=7)
    shapes = [(512, 1024), (1024, 512), (256, 2048)]
    ws = [weights(s, 40 + i).cuda() for i, s in enumerate(shapes)]
    handles = [manager.write(w) for w in ws]
    be = manager._be
    outs = [torch.zeros(w.numel(), dtype=torch.bfloat16, device="cuda") for w in ws]
    batch = be.make_batch(handles, outs)
    be.run_batch(batch)                                   # warm-up outside capture
    torch.cuda.synchronize()
    for o in outs:
        o.zero_()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            be.run_batch(batch)
    torch.cuda.synchronize()
    for _ in range(3):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for o, w in zip(outs, ws):
            assert torch.equal(o.view(torch.int16), w.view(-1).view(torch.int16))
    manager.check()


def test_back_to_back_batches_with_stable_inputs_share_buffers_safely():
    """Launches that were told their inputs are stable build their tables while the previous
    kernel drains; their stores must still wait for it.  Two batches decode into the same
    buffers in turn, with a reader of those buffers between them."""
    manager = neuzip.Manager(precision=7)
    be = manager._be
    shapes = [(1024, 1024), (512, 4096), (2048, 768)]
    sets = []
    for base in (0, 10):
        ws = [weights(s, base + i).cuda() for i, s in enumerate(shapes)]
        sets.append((ws, [manager.write(w) for w in ws]))
    outs = [torch.empty(int(np.prod(s)), dtype=torch.bfloat16, device="cuda") for s in shapes]
    from neuzip_b200 import backend as B
    from neuzip_b200 import _lib
    batches = [be.make_batch(handles, outs) for _, handles in sets]
    # the first decode after the writes waits for them: the last write is the operation
    # enqueued just before it
    assert B._stable_flag(batches[1].entries, B._op_counter + 1) == 0
    expected = [[w.view(-1).float().sum() for w in ws] for ws, _ in sets]
    sums = []
    for it in range(40):
        be.run_batch(batches[it % 2])
        assert B._stable_flag(batches[0].entries + batches[1].entries, B._op_counter + 1) == \
            _lib.NZ_ITEM_INPUTS_STABLE
        sums.append([o.float().sum() for o in outs])          # a reader between the two writers
    torch.cuda.synchronize()
    for it, got in enumerate(sums):
        for g, e in zip(got, expected[it % 2]):
            assert float(g) == float(e)
    # a write in between makes the next launch conservative again
    manager.write(sets[0][0][0], sets[0][1][0])
    assert B._stable_flag([be.entry(sets[0][1][0])], B._op_counter + 1) == 0
    be.run_batch(batches[0])
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), sets[0][0][0].view(-1).view(torch.int16))
    manager.check()


def test_stable_input_promise_is_tracked_per_entry_across_managers():
    """A container written through a second Manager just before a batched decode of
    another Manager's handles must not be promised as stable, and a batch follows a
    handle that is written again (new bytes, not the ones it was built with)."""
    from neuzip_b200 import backend as B
    from neuzip_b200 import _lib
    m1, m2 = neuzip.Manager(precision=7), neuzip.Manager(precision=7)
    w1, w2 = weights((512, 1024), 1).cuda(), weights((512, 1024), 2).cuda()
    h1 = m1.write(w1)
    out = torch.empty(w1.numel(), dtype=torch.bfloat16, device="cuda")
    batch = m1._be.make_batch([h1], [out])
    for _ in range(3):
        m1._be.run_batch(batch)
    e1 = m1._be.entry(h1)
    assert B._stable_flag([e1], B._op_counter + 1) == _lib.NZ_ITEM_INPUTS_STABLE
    h2 = m2.write(w2)                              # another Manager, same stream
    e2 = m2._be.entry(h2)
    assert B._stable_flag([e2], B._op_counter + 1) == 0
    assert B._stable_flag([e1], B._op_counter + 1) == _lib.NZ_ITEM_INPUTS_STABLE
    got = m2.read_many([h2])[0]
    assert torch.equal(got.view(torch.int16), w2.view(torch.int16))
    # the same handle written again: the batch must decode the new bytes
    m1.write(w2, h1)
    m1._be.run_batch(batch)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), w2.view(-1).view(torch.int16))
    m1.check()
    m2.check()


def test_layerwise_hooks_follow_weight_updates_and_loaded_checkpoints():
    """After an optimiser step (every weight is written again) and after
    load_state_dict, a model with the layer-wise hooks attached must compute with the new
    weights, exactly like the same model without hooks."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from neuzip_b200 import layerwise
    from neuzip_b200.optim import CompressedAdamW
    torch.manual_seed(3)
    cfg = LlamaConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=64)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).cuda()
    m = neuzip.Manager(precision=7)
    m.convert(model)
    before = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in model.state_dict().items()}
    ids = torch.randint(0, 128, (2, 16), device="cuda")
    hooks = layerwise.attach(model, m)
    opt = CompressedAdamW(model.parameters(), lr=1e-2)
    loss = model(ids, labels=ids).loss
    loss.backward()
    opt.step()
    opt.zero_grad()
    with torch.no_grad():
        hooked = model(ids).logits.float()
    for h in hooks:
        h.remove()
    with torch.no_grad():
        plain = model(ids).logits.float()
    assert torch.equal(hooked, plain)
    # load the earlier checkpoint with the hooks attached
    hooks = layerwise.attach(model, m)
    with torch.no_grad():
        model(ids)
    model.load_state_dict(before)
    with torch.no_grad():
        hooked = model(ids).logits.float()
    for h in hooks:
        h.remove()
    with torch.no_grad():
        plain = model(ids).logits.float()
    assert torch.equal(hooked, plain)
    m.check()


@pytest.mark.parametrize("precision,shape,operand", ((7, (256, 2048), True), (3, (128, 4096), True),
                                                     (7, (96, 1000), False), (1, (33, 520), False)))
def test_fused_update_equals_read_adamw_write_bit_for_bit(precision, shape, operand):
    """nz_adamw_compressed_bf16 (the AdamW step inside the decode kernel, then the
    compressor) against read -> nz_adamw_bf16 -> write: same containers, fractions and
    moments, three steps in a row; stream order with a ragged last unit, and operand order."""
    from neuzip_b200 import _lib
    L = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(precision + shape[0])
    w = weights(shape, 5).cuda()
    ma, mb = neuzip.Manager(precision=precision), neuzip.Manager(precision=precision)
    ha, hb = ma.write(w, operand=operand), mb.write(w, operand=operand)
    assert (ma._be.entry(ha).operand_cols > 0) == operand
    n = w.numel()
    m1 = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    v1 = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    m2, v2 = m1.clone(), v1.clone()
    for step in range(1, 4):
        g = (torch.randn(shape, device="cuda") * 1e-2).to(torch.bfloat16).contiguous()
        # a: the single fused call
        assert ma._be.adamw_update(ha, g.view(-1), m1, v1, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, 0.5)
        # b: read, stand-alone update kernel, write
        wb = mb.read(hb).contiguous()
        _lib.check(L.nz_adamw_bf16(wb.data_ptr(), g.data_ptr(), m2.data_ptr(), v2.data_ptr(), n, 1,
                                   1e-2, 0.9, 0.999, 1e-8, 0.1, step, 0.5, st))
        mb.write(wb, hb)
        ea, eb = ma._be.entry(ha), mb._be.entry(hb)
        assert ea.operand_cols == eb.operand_cols
        assert torch.equal(m1, m2) and torch.equal(v1, v2), step
        assert torch.equal(ea.fractions, eb.fractions), step
        assert torch.equal(ea.container, eb.container), step
    assert not torch.equal(ma.read(ha), w)            # the weights did move
    ma.check()
    mb.check()


def test_converted_checkpoint_loads_into_a_meta_model_on_gpu(tmp_path):
    def make():
        return torch.nn.Sequential(torch.nn.Linear(2048, 256, bias=True), torch.nn.ReLU(),
                                   torch.nn.Linear(256, 64, bias=False)).to(torch.bfloat16)
    torch.manual_seed(8)
    src = make()
    m1 = neuzip.Manager(precision=7)
    m1.convert(src)
    src.cuda()
    x = torch.randn(4, 2048, device="cuda", dtype=torch.bfloat16)
    expect = src(x)
    assert m1._be.entry(src[0]._p._handle).operand_cols == 2048     # stored in operand order
    torch.save(src.state_dict(), tmp_path / "c.pt")
    with torch.device("meta"):
        skeleton = make()
    m2 = neuzip.Manager(precision=7)
    m2.load_converted(skeleton, torch.load(tmp_path / "c.pt", weights_only=False), device="cuda")
    assert m2._be.entry(skeleton[0]._p._handle).operand_cols == 2048
    assert torch.equal(skeleton(x), expect)
    m2.fuse_linear(64)
    fused = skeleton(x)
    assert (fused.float() - expect.float()).abs().max().item() <= 2.0 ** -6 * expect.float().abs().max().item()
    m2.check()
