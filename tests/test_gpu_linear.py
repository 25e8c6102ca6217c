"""Operand order and the fused decode -> tcgen05 GEMM (nz_linear_bf16), through the C ABI.

Integer work (operand-order containers, fractions, decoded tensors) is compared bit
for bit with the CPU oracle applied to the permuted tensor.  The GEMM is floating
point: products are exact in fp32, sums are fp32 in a different order from a library
GEMM, and the result is rounded once to bf16 -- so it is compared with an fp32
restatement (decoded weight, fp32 matmul) within 2^-7 relative (one bf16 rounding
step of the result, 2^-8, plus the same again for the restatement's own rounding)
plus an absolute term for cancellation, 2^-7 of the largest |x|.|w| row sum.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import nzabi as A

pytestmark = pytest.mark.gpu


def weights(shape, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def check_linear(y, x, w_dec, bias):
    ref = x.float() @ w_dec.float().t()
    mag = x.float().abs() @ w_dec.float().abs().t()
    if bias is not None:
        ref = ref + bias.float()
        mag = mag + bias.float().abs()
    err = (y.float() - ref).abs()
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -7 * 2.0 ** -8 * mag + 1e-30
    # the second term: fp32 accumulation error is far below it; it covers results that
    # cancel to near zero, where one bf16 step of the partial sums dominates
    bad = err > bound
    assert not bool(bad.any()), (float(err.max()), int(bad.sum()), tuple(y.shape))


@pytest.mark.parametrize("s", (7, 3, 1, 0))
@pytest.mark.parametrize("rows,cols", ((128, 1024), (8, 4096), (260, 2048), (64, 11008)))
def test_operand_order_container_equals_oracle_of_the_permuted_tensor(s, rows, cols):
    L = A.lib()
    S = int(L.nz_operand_lane_symbols(cols, s))
    assert S == O.operand_lane_symbols(cols, s)
    if S == 0:                      # no unit length near the default divides the row: pick one
        S = 128
    assert (cols // 64) % (S // 8) == 0
    w = weights((rows, cols), rows + cols + s).cuda()
    bits = A.to_bits(w)
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    stream = O.to_operand_order(bits, rows, cols)
    c_ref, f_ref = O.compress_bf16(stream, s, S)
    assert np.array_equal(cont.cpu().numpy(), c_ref)
    assert np.array_equal(frac.cpu().numpy(), f_ref)
    out, status = A.decompress_operand(cont, frac, rows, cols, s, S, mw, canon=True)
    assert status == 0
    ref = O.from_operand_order(O.decompress_bf16(c_ref, f_ref, bits.size, s, canonical_nan=True),
                               rows, cols)
    assert np.array_equal(A.to_bits(out), ref)
    if s == 7:
        assert np.array_equal(ref, bits)


def test_operand_order_with_raw_units_and_all_patterns():
    """Exponent bytes that do not compress (every pattern once) are stored raw; the
    operand-order decode must place them as well."""
    rows, cols, s = 16, 4096, 7
    S = int(A.lib().nz_operand_lane_symbols(cols, s))
    bits = np.arange(65536, dtype=np.uint16)
    rng = np.random.default_rng(3)
    rng.shuffle(bits)
    w = A.from_bits(bits)
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    hdr = O.parse_header(cont.cpu().numpy())
    assert hdr["n_raw_units"] > 0
    out, status = A.decompress_operand(cont, frac, rows, cols, s, S, mw, canon=False)
    assert status == 0
    assert np.array_equal(A.to_bits(out), bits)


def test_batched_decode_mixes_operand_order_and_stream_order_items():
    from neuzip_b200 import _lib
    L = A.lib()
    s, rows, cols = 7, 256, 2048
    S = int(L.nz_operand_lane_symbols(cols, s))
    assert S == int(L.nz_default_lane_symbols(s))
    w1, w2 = weights((rows, cols), 1).cuda(), weights((rows, cols), 2).cuda()
    c1, f1, m1 = A.compress_operand(w1, rows, cols, s, S)
    c2, f2, m2 = A.compress(w2.view(-1), s, S)
    outs = [torch.empty(rows * cols, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    items = (_lib.DecompressItem * 2)()
    for k, (c, f, mw, oc) in enumerate(((c1, f1, m1, cols), (c2, f2, m2, 0))):
        items[k].container, items[k].container_bytes = c.data_ptr(), c.numel()
        items[k].frac_in, items[k].n = f.data_ptr(), rows * cols
        items[k].max_unit_words, items[k].flags = mw, 0
        items[k].out_bf16, items[k].operand_cols = outs[k].data_ptr(), oc
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16_batch(items, 2, s, S, 1, status.data_ptr(), A.stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(outs[0].view(torch.int16), w1.view(-1).view(torch.int16))
    assert torch.equal(outs[1].view(torch.int16), w2.view(-1).view(torch.int16))


LINEAR_SHAPES = ((128, 1024), (256, 2048), (512, 4096), (136, 2048), (384, 11008))


@pytest.mark.parametrize("rows,cols", LINEAR_SHAPES)
@pytest.mark.parametrize("m", (1, 16, 100, 128))
def test_fused_linear_lossless_matches_fp32_restatement(rows, cols, m):
    s = 7
    S = int(A.lib().nz_operand_lane_symbols(cols, s))
    w = weights((rows, cols), 10 + rows).cuda()
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, cols, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    y, status = A.linear(cont, frac, rows, cols, s, S, x, None, mw)
    assert status == 0
    check_linear(y, x, w, None)


@pytest.mark.parametrize("s", (3, 1, 0))
def test_fused_linear_lossy_precisions_with_bias(s):
    rows, cols, m = 256, 4096, 48
    S = 256          # shorter than the size-optimal unit of the lossy precisions: fits next to the tiles
    w = weights((rows, cols), 77 + s).cuda()
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    w_dec, status = A.decompress_operand(cont, frac, rows, cols, s, S, mw, canon=True)
    assert status == 0
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, cols, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    bias = torch.randn(rows, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    y, status = A.linear(cont, frac, rows, cols, s, S, x, bias, mw, canon=True)
    assert status == 0
    check_linear(y, x, w_dec.view(rows, cols), bias)


@pytest.mark.parametrize("m", (256, 300, 512))
def test_fused_linear_many_tokens_take_several_passes(m):
    rows, cols, s = 256, 2048, 7
    S = int(A.lib().nz_operand_lane_symbols(cols, s))
    w = weights((rows, cols), 5).cuda()
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, cols, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    bias = torch.randn(rows, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    y, status = A.linear(cont, frac, rows, cols, s, S, x, bias, mw)
    assert status == 0
    check_linear(y, x, w, bias)


def test_fused_linear_is_reproducible_and_exact_on_integers():
    """Small integers: every product and sum is exact in fp32 and the result is exactly
    representable, so the fused kernel must reproduce the integer GEMM exactly."""
    rows, cols, s, m = 128, 2048, 7, 32
    S = int(A.lib().nz_operand_lane_symbols(cols, s))
    g = torch.Generator().manual_seed(9)
    w = torch.randint(-1, 2, (rows, cols), generator=g).to(torch.bfloat16).cuda()
    x = torch.randint(-1, 2, (m, cols), generator=g).to(torch.bfloat16).cuda()
    cont, frac, mw = A.compress_operand(w, rows, cols, s, S)
    y1, st1 = A.linear(cont, frac, rows, cols, s, S, x, None, mw)
    y2, st2 = A.linear(cont, frac, rows, cols, s, S, x, None, mw)
    assert st1 == 0 and st2 == 0
    ref = (x.double() @ w.double().t())
    assert float(ref.abs().max()) < 256          # representable in bf16 exactly
    assert torch.equal(y1.double(), ref)
    assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))


def test_fused_linear_rejects_what_it_cannot_do():
    from neuzip_b200 import _lib
    L = A.lib()
    assert L.nz_operand_lane_symbols(100, 7) == 0          # columns not a multiple of 64
    assert L.nz_operand_lane_symbols(512, 7) == 0          # rows of 8 blocks: units would be too short
    x = torch.zeros(16, 2048, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    rc = L.nz_linear_bf16(c.data_ptr(), c.numel(), c.data_ptr(), 130, 2048, 7, 256, 0, 0,
                          x.data_ptr(), 16, 0, x.data_ptr(), 0, 0, 0, A.stream())
    assert rc == _lib.NZ_E_ARG                             # rows not a multiple of 4


# ------------------------------------------------------------- through the Manager
import neuzip  # noqa: E402


def test_manager_stores_linear_weights_in_operand_order_and_reads_them_back():
    m = neuzip.Manager(precision=7)
    w = weights((256, 2048), 21).cuda()
    h = m.write(w, operand=True)
    e = m._be.entry(h)
    assert e.operand_cols == 2048 and e.lane_symbols == O.operand_lane_symbols_for(256, 2048, 7) == 128
    assert torch.equal(m.read(h).view(torch.int16), w.view(torch.int16))
    # the stored bytes are the oracle's for the permuted tensor
    stream = O.to_operand_order(A.to_bits(w), 256, 2048)
    c_ref, f_ref = O.compress_bf16(stream, 7, e.lane_symbols)
    assert np.array_equal(e.container.cpu().numpy(), c_ref)
    assert np.array_equal(e.fractions.cpu().numpy(), f_ref)
    # a shape that cannot be in operand order falls back to stream order
    h2 = m.write(weights((10, 100), 22).cuda(), operand=True)
    assert m._be.entry(h2).operand_cols == 0
    # an update under the same handle keeps the layout; so does a checkpoint round trip
    w2 = weights((256, 2048), 23).cuda()
    m.write(w2, h)
    assert m._be.entry(h).operand_cols == 2048
    blob = m.export_entry(h)
    m2 = neuzip.Manager(precision=7)
    h3 = m2.import_entry(blob)
    assert m2._be.entry(h3).operand_cols == 2048
    assert torch.equal(m2.read(h3).view(torch.int16), w2.view(torch.int16))
    # batched reads mix layouts
    a, b = m.read_many([h, h2])
    assert torch.equal(a.view(torch.int16), w2.view(torch.int16))
    rows = m.read_rows(h, torch.tensor([3, 200, 7], device="cuda"))
    assert torch.equal(rows.view(torch.int16), w2[[3, 200, 7]].view(torch.int16))
    m.check()
    m2.check()


@pytest.mark.parametrize("with_bias", (False, True))
def test_manager_linear_takes_the_fused_path_when_enabled(with_bias):
    m = neuzip.Manager(precision=7)
    w = weights((384, 2048), 31).cuda()
    h = m.write(w, operand=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 5, 2048, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(384, generator=g).to(torch.bfloat16).cuda() if with_bias else None
    plain = m.linear(h, x, bias)                       # decode, then library GEMM
    m.fuse_linear(256)
    fused = m.linear(h, x, bias)
    assert fused.shape == plain.shape == (2, 5, 384)
    check_linear(fused.reshape(10, 384), x.reshape(10, 2048), w, bias)
    assert (fused.float() - plain.float()).abs().max().item() <= 2.0 ** -6 * plain.float().abs().max().item()
    # more rows than the limit: back to decode + GEMM, bit-identical to the plain path
    m.fuse_linear(4)
    assert torch.equal(m.linear(h, x, bias), plain)
    m.check()


def test_converted_llama_with_fused_linear_matches_dense_logits_and_tokens():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=1024, intermediate_size=2048,
                                   num_hidden_layers=2, num_attention_heads=8,
                                   num_key_value_heads=8, max_position_embeddings=128)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (1, 16), device="cuda")
    with torch.no_grad():
        ref_logits = model(ids).logits
        ref_tokens = model.generate(ids, max_new_tokens=8, do_sample=False)
    m = neuzip.Manager()
    m.convert(model)
    m.fuse_linear(256)
    linears = [mod for mod in model.modules() if isinstance(mod, neuzip.nn.Linear)]
    assert len(linears) == 14
    assert all(m._be.entry(mod._p._handle).operand_cols == mod.in_features for mod in linears)
    with torch.no_grad():
        logits = model(ids).logits                     # prefill: 16 rows per Linear
        tokens = model.generate(ids, max_new_tokens=8, do_sample=False)   # then one row at a time
    m.check()
    # every Linear rounds its fp32 sums to bf16 once, like the library GEMM, but adds the column
    # segments in its own order: the logits may differ by a bf16 ulp or two of the largest one
    # (2^-8 relative each), not more
    scale = max(1.0, ref_logits.float().abs().max().item())
    assert (logits.float() - ref_logits.float()).abs().max().item() <= 2.0 ** -6 * scale
    assert torch.equal(tokens, ref_tokens)


def test_batched_decode_of_tensors_with_different_lane_symbols():
    """One launch, three tensors: operand order with units of 344 and of 256 lane
    symbols, and a stream-order tensor with 64."""
    from neuzip_b200 import _lib
    L = A.lib()
    s = 7
    specs = [((64, 11008), 344, True), ((256, 2048), 256, True), ((100, 333), 64, False)]
    ws, comps = [], []
    for k, (shape, S, operand) in enumerate(specs):
        w = weights(shape, 40 + k).cuda()
        ws.append(w)
        comps.append(A.compress_operand(w, shape[0], shape[1], s, S) if operand
                     else A.compress(w.view(-1), s, S))
    outs = [torch.empty(w.numel(), dtype=torch.bfloat16, device="cuda") for w in ws]
    items = (_lib.DecompressItem * 3)()
    for k, ((shape, S, operand), (c, f, mw)) in enumerate(zip(specs, comps)):
        items[k].container, items[k].container_bytes = c.data_ptr(), c.numel()
        items[k].frac_in, items[k].n = f.data_ptr(), ws[k].numel()
        items[k].max_unit_words, items[k].flags = mw, 0
        items[k].out_bf16 = outs[k].data_ptr()
        items[k].operand_cols = shape[1] if operand else 0
        items[k].lane_symbols = S
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16_batch(items, 3, s, 256, 1, status.data_ptr(), A.stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for w, o in zip(ws, outs):
        assert torch.equal(o.view(torch.int16), w.view(-1).view(torch.int16))
