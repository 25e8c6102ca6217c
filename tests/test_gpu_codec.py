"""GPU parity tests: every C-ABI kernel against the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import nzabi as A

pytestmark = pytest.mark.gpu

PRECISIONS = (0, 1, 3, 7)
SIZES = (1, 7, 8, 9, 63, 64, 65, 255, 256, 257, 1000, 4095, 8192, 8193, 65536, 100003, 300000)


def weights(n, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def all_patterns():
    return np.arange(65536, dtype=np.uint16)


# ---------------------------------------------------------------- split / merge
@pytest.mark.parametrize("s", PRECISIONS)
def test_split_all_patterns(s):
    bits = all_patterns()
    x = A.from_bits(bits)
    exp, frac = A.split(x, s)
    e_ref, f_ref = O.split(bits, s, literal=True)
    assert np.array_equal(exp.cpu().numpy(), e_ref)
    assert np.array_equal(frac.cpu().numpy(), f_ref)


@pytest.mark.parametrize("s", PRECISIONS)
@pytest.mark.parametrize("canon", (False, True))
def test_merge_all_patterns(s, canon):
    bits = all_patterns()
    e_ref, f_ref = O.split(bits, s)
    out = A.merge(A.dev_u8(e_ref), A.dev_u8(f_ref), bits.size, s, canon)
    ref = O.merge(e_ref, f_ref, s, canonical_nan=canon)
    assert np.array_equal(A.to_bits(out), ref)


@pytest.mark.parametrize("s", PRECISIONS)
@pytest.mark.parametrize("n", SIZES)
def test_split_merge_ragged_sizes(s, n):
    x = weights(n, 100 + n).cuda()
    bits = A.to_bits(x)
    exp, frac = A.split(x, s)
    e_ref, f_ref = O.split(bits, s)
    assert np.array_equal(exp.cpu().numpy(), e_ref)
    assert np.array_equal(frac.cpu().numpy(), f_ref)
    out = A.merge(exp, frac, n, s)
    assert np.array_equal(A.to_bits(out), O.merge(e_ref, f_ref, s))


def test_empty_inputs_are_accepted():
    L = A.lib()
    assert L.nz_split_bf16(0, 0, 7, 0, 0, A.stream()) == 0
    assert L.nz_merge_bf16(0, 0, 0, 7, 0, 0, A.stream()) == 0
    assert L.nz_decompress_bf16(0, 0, 0, 0, 7, 256, 0, 0, 0, 0, A.stream()) == 0


# ------------------------------------------------------------------- histogram
@pytest.mark.parametrize("n", (1, 15, 16, 17, 4096, 100003, 1 << 20))
def test_histogram(n):
    rng = np.random.default_rng(n)
    sym = rng.choice(np.arange(110, 126, dtype=np.uint8), size=n,
                     p=np.array([1, 1, 2, 3, 5, 8, 13, 21, 34, 55, 89, 144, 233, 120, 30, 5]) / 764)
    d = A.dev_u8(sym)
    hist = torch.full((256,), 7, dtype=torch.int32, device="cuda")
    from neuzip_b200 import _lib
    _lib.check(A.lib().nz_histogram_u8(d.data_ptr(), n, hist.data_ptr(), A.stream()))
    assert np.array_equal(hist.cpu().numpy().astype(np.uint64), O.histogram(sym))


# ------------------------------------------------------------ entropy coder
def exponent_streams():
    rng = np.random.default_rng(7)
    yield "gauss", O.split(A.to_bits(weights(70000, 3)), 7)[0]
    yield "gauss_big", O.split(A.to_bits(weights(1 << 20, 4)), 7)[0]
    yield "constant", np.full(20000, 121, np.uint8)
    yield "two_symbols", rng.choice(np.array([3, 250], np.uint8), size=33333, p=[0.9, 0.1])
    yield "uniform_incompressible", rng.integers(0, 256, size=50000, dtype=np.uint8)
    yield "all_256_skewed", np.concatenate(
        [np.arange(256, dtype=np.uint8), np.full(90000, 17, np.uint8)])
    yield "fifty_symbols", rng.choice(np.arange(60, 110, dtype=np.uint8), size=70000,
                                      p=np.r_[np.full(10, 0.08), np.full(40, 0.005)])
    yield "hundred_symbols_top_40pct", rng.choice(
        np.arange(100, 200, dtype=np.uint8), size=80000, p=np.r_[0.4, np.full(99, 0.6 / 99)])
    yield "single_element", np.array([200], np.uint8)
    yield "half_raw_half_coded", np.concatenate(
        [rng.integers(0, 256, size=32768, dtype=np.uint8), np.full(32768, 9, np.uint8)])


@pytest.mark.parametrize("S", (8, 64, 256, 384, 512, 1024))
def test_encode_matches_oracle_bytes(S):
    for name, sym in exponent_streams():
        cont, mw = A.encode(A.dev_u8(sym), S)
        ref = O.encode(sym, S)
        got = cont.cpu().numpy()
        assert got.size == ref.size, (name, S, got.size, ref.size)
        assert np.array_equal(got, ref), (name, S)
        assert mw == O.parse_header(ref)["max_coded_unit_words"]


@pytest.mark.parametrize("S", (8, 64, 256, 384, 512, 1024))
def test_decode_oracle_containers(S):
    for name, sym in exponent_streams():
        ref = O.encode(sym, S)
        hdr = O.parse_header(ref)
        for mw in (0, hdr["max_coded_unit_words"]):
            exp, status = A.decode_exponents(A.dev_u8(ref), sym.size, S, mw)
            assert status == 0, (name, S, status)
            assert np.array_equal(exp.cpu().numpy(), sym), (name, S)


@pytest.mark.parametrize("s", PRECISIONS)
@pytest.mark.parametrize("n", SIZES)
def test_compress_decompress_roundtrip(s, n):
    S = O.default_lane_symbols(s)
    x = weights(n, 500 + n).cuda()
    bits = A.to_bits(x)
    cont, frac, mw = A.compress(x, s, S)
    c_ref, f_ref = O.compress_bf16(bits, s, S)
    assert np.array_equal(cont.cpu().numpy(), c_ref)
    assert np.array_equal(frac.cpu().numpy(), f_ref)
    out, status = A.decompress(cont, frac, n, s, S, mw)
    assert status == 0
    ref = O.decompress_bf16(c_ref, f_ref, n, s)
    assert np.array_equal(A.to_bits(out), ref)
    if s == 7:
        assert np.array_equal(A.to_bits(out), bits)      # lossless = bit exact


@pytest.mark.parametrize("s", PRECISIONS)
@pytest.mark.parametrize("canon", (False, True))
def test_decompress_all_patterns_including_nan(s, canon):
    bits = np.tile(all_patterns(), 3)          # NaN / inf / denormal / -0 patterns included
    S = O.default_lane_symbols(s)
    x = A.from_bits(bits)
    cont, frac, mw = A.compress(x, s, S)
    out, status = A.decompress(cont, frac, bits.size, s, S, mw, canon)
    assert status == 0
    e_ref, f_ref = O.split(bits, s, literal=True)
    assert np.array_equal(A.to_bits(out), O.merge(e_ref, f_ref, s, canonical_nan=canon))


def test_incompressible_tensor_is_stored_raw_and_round_trips():
    rng = np.random.default_rng(11)
    bits = rng.integers(0, 65536, size=200000, dtype=np.uint16)
    bits = bits[(bits & 0x7F80) != 0x7F80]            # keep it NaN/inf free
    x = A.from_bits(bits)
    cont, frac, mw = A.compress(x, 7, 256)
    assert O.parse_header(cont.cpu().numpy())["n_raw_units"] > 0
    out, status = A.decompress(cont, frac, bits.size, 7, 256, mw)
    assert status == 0 and np.array_equal(A.to_bits(out), bits)


# ---------------------------------------------------- config 1 of the baseline
def test_config1_seed0_matrix_matches_golden():
    import json, os
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "config1.json")))
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bits = A.to_bits(w)
    assert O.crc32(bits) == int(golden["input_crc32"], 16)
    x = w.cuda().view(-1)
    for s in PRECISIONS:
        g = golden["precision"][str(s)]
        exp, frac = A.split(x, s)
        assert O.crc32(exp.cpu().numpy()) == int(g["exp_crc32"], 16)
        assert O.crc32(frac.cpu().numpy()) == int(g["frac_crc32"], 16)
        S = g["lane_symbols"]
        cont, frac2, mw = A.compress(x, s, S)
        assert cont.numel() == g["container_bytes"]
        assert O.crc32(cont.cpu().numpy()) == int(g["container_crc32"], 16)
        out, status = A.decompress(cont, frac2, x.numel(), s, S, mw, canon=True)
        assert status == 0
        assert O.crc32(A.to_bits(out)) == int(g["roundtrip_crc32"], 16)
        stored = cont.numel() + frac2.numel()
        assert stored <= 1.025 * g["ideal_bytes"], (s, stored, g["ideal_bytes"])
    # lossless: bit exact
    cont, frac, mw = A.compress(x, 7, 256)
    out, _ = A.decompress(cont, frac, x.numel(), 7, 256, mw)
    assert torch.equal(out.view(torch.int16), x.view(torch.int16))


def test_wide_alphabets_keep_frequencies_in_eleven_bits():
    rng = np.random.default_rng(11)
    for top in (0.3, 0.45, 0.47, 0.6, 0.95):
        sym = rng.choice(np.arange(256, dtype=np.uint8), size=120000,
                         p=np.r_[top, np.full(255, (1 - top) / 255)])
        cont, mw = A.encode(A.dev_u8(sym), 256)
        hdr = O.parse_header(cont.cpu().numpy())
        assert hdr["prob_bits"] == (12 if top < 0.46 else 11)
        assert int(np.frombuffer(cont.cpu().numpy()[64:576].tobytes(), np.uint16).max()) <= 2047
        exp, status = A.decode_exponents(cont, sym.size, 256, mw)
        assert status == 0 and np.array_equal(exp.cpu().numpy(), sym)
    # a container whose table holds a wider frequency is refused, not decoded wrongly
    sym = np.concatenate([np.arange(256, dtype=np.uint8), np.full(90000, 17, np.uint8)])
    forged = O.encode(sym, 256, prob_bits=12)
    assert np.array_equal(O.decode(forged, sym.size), sym)
    exp, status = A.decode_exponents(A.dev_u8(forged), sym.size, 256, 0)
    assert status & 0x1                      # NZ_STATUS_BAD_HEADER


# -------------------------------------------------------- malformed containers
def _corrupt(cont_np, where, value):
    c = cont_np.copy()
    c[where] = value
    return c


def test_malformed_containers_set_status_and_do_not_touch_guards():
    sym = O.split(A.to_bits(weights(40000, 9)), 7)[0]
    S = 256
    ref = O.encode(sym, S)
    hdr = O.parse_header(ref)
    n = sym.size
    cases = {
        "magic": (_corrupt(ref, 0, 0), 0x1),
        "n_symbols": (_corrupt(ref, 8, (ref[8] + 1) & 0xFF), 0x1),
        "freq_sum": (_corrupt(ref, 64 + 2 * 121, (ref[64 + 2 * 121] + 1) & 0xFF), 0x1),
        "offset_backwards": (_corrupt(ref, 576 + 4 + 3, 0x7F), 0x2),
        "lane_length": (_corrupt(ref, hdr["payload_offset"] + 5, 1), 0x4),
    }
    for name, (bad, bit) in cases.items():
        _, status = A.decode_exponents(A.dev_u8(bad), n, S, 0)
        assert status & bit, (name, status)
    # a flipped payload word decodes to garbage but must end in a wrong state
    bad = _corrupt(ref, hdr["payload_offset"] + 32 + 9, ref[hdr["payload_offset"] + 32 + 9] ^ 0x55)
    _, status = A.decode_exponents(A.dev_u8(bad), n, S, 0)
    assert status & 0x8
    # truncated buffer is refused on the host
    from neuzip_b200 import _lib
    L = A.lib()
    out = torch.empty(n, dtype=torch.uint8, device="cuda")
    d = A.dev_u8(ref[:512])
    assert L.nz_decode_exponents(d.data_ptr(), 512, n, S, 0, out.data_ptr(), 0, A.stream()) == _lib.NZ_E_FORMAT


def test_argument_errors():
    from neuzip_b200 import _lib
    L = A.lib()
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    e = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert L.nz_split_bf16(x.data_ptr(), 64, 5, e.data_ptr(), e.data_ptr(), 0) == _lib.NZ_E_ARG
    assert b"precision" in L.nz_last_error()
    assert L.nz_split_bf16(x.data_ptr() + 2, 8, 7, e.data_ptr(), e.data_ptr(), 0) == _lib.NZ_E_ARG
    assert L.nz_decode_exponents(e.data_ptr(), 64, 64, 12, 0, e.data_ptr(), 0, 0) == _lib.NZ_E_ARG
    assert L.nz_encode_exponents(e.data_ptr(), 64, 256, e.data_ptr(), 64, e.data_ptr(), 64, 0) == _lib.NZ_E_CAPACITY
    # gather and matrix-vector entry points: bad geometry and short scratch are refused
    w = weights(4096 * 8, 1).cuda()
    cont, frac, mw = A.compress(w, 7, 256)
    n = w.numel()
    y = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    xf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    sc = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    rows = torch.zeros(4, dtype=torch.int64, device="cuda")
    args = (cont.data_ptr(), cont.numel(), frac.data_ptr(), n, 7, 256, mw, 0)
    assert L.nz_linear_vec_bf16(*args, 100, xf.data_ptr(), None, y.data_ptr(), sc.data_ptr(),
                                sc.numel(), None, 0) == _lib.NZ_E_ARG          # rows not a multiple of 256
    assert b"multiple of 256" in L.nz_last_error()
    assert L.nz_linear_vec_bf16(*args, 4096, xf.data_ptr(), None, y.data_ptr(), sc.data_ptr(),
                                16, None, 0) == _lib.NZ_E_CAPACITY
    assert L.nz_linear_vec_scratch_bytes(n, 4096, 256) <= sc.numel()
    assert L.nz_gather_rows_bf16(*args, 1000, rows.data_ptr(), 4, y.data_ptr(), sc.data_ptr(),
                                 sc.numel(), None, 0) == _lib.NZ_E_ARG        # 1000 does not divide n
    assert L.nz_gather_rows_bf16(*args, 4096, rows.data_ptr(), 4, y.data_ptr(), sc.data_ptr(),
                                 64, None, 0) == _lib.NZ_E_CAPACITY
    assert L.nz_decompress_bf16_units(*args, None, 3, y.data_ptr(), None, 0) == _lib.NZ_E_ARG
    assert L.nz_decompress_bf16_units(*args, None, 0, y.data_ptr(), None, 0) == _lib.NZ_OK


# ------------------------------------------------------------- batched decode
@pytest.mark.parametrize("s", PRECISIONS)
def test_batched_decompress_equals_single_calls(s):
    from neuzip_b200 import _lib
    L = A.lib()
    S = O.default_lane_symbols(s)
    sizes = [1 << 20, 300, 0, 70000, 8192 * 3, 4096 * 640, 9, 1 << 16, 123457, 2 << 20, 77]
    tensors, comps, singles = [], [], []
    for i, n in enumerate(sizes):
        x = weights(max(n, 1), 900 + i)[:n].cuda().contiguous() if n else torch.empty(
            0, dtype=torch.bfloat16, device="cuda")
        tensors.append(x)
        if n:
            c, f, mw = A.compress(x, s, S)
            out, status = A.decompress(c, f, n, s, S, mw, canon=True)
            assert status == 0
        else:
            c = torch.zeros(16, dtype=torch.uint8, device="cuda")
            f = torch.zeros(16, dtype=torch.uint8, device="cuda")
            mw, out = 0, x
        comps.append((c, f, mw))
        singles.append(out)
    items = (_lib.DecompressItem * len(sizes))()
    raws, outs = [], []
    for i, n in enumerate(sizes):
        raw, out = A.guarded(2 * n, torch.bfloat16)
        raws.append(raw)
        outs.append(out)
        c, f, mw = comps[i]
        items[i].container = c.data_ptr()
        items[i].container_bytes = c.numel()
        items[i].frac_in = f.data_ptr()
        items[i].n = n
        items[i].max_unit_words = mw if i % 2 else 0
        items[i].out_bf16 = out.data_ptr() if n else 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16_batch(items, len(sizes), s, S, 1, status.data_ptr(), A.stream()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i, n in enumerate(sizes):
        assert A.guards_intact(raws[i], 2 * n)
        assert torch.equal(outs[i].view(torch.int16), singles[i].view(torch.int16)), (s, i, n)
        if s == 7 and n:
            assert torch.equal(outs[i].view(torch.int16), tensors[i].view(torch.int16))


# ------------------------------------------------------------ block normaliser
@pytest.mark.parametrize("group", (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024))
def test_normalize_and_denormalize_match_oracle(group):
    from neuzip_b200 import _lib
    L = A.lib()
    for n, seed in ((1, 1), (7, 2), (1024, 3), (1025, 4), (5000, 5), (70001, 6)):
        x = (weights(n, 700 + seed, std=0.05)).cuda()
        bits = A.to_bits(x)
        nb = int(L.nz_normalizer_bytes(n, group))
        raw_o, out = A.guarded(2 * n, torch.bfloat16)
        raw_n, norm = A.guarded(nb)
        _lib.check(L.nz_normalize_bf16(x.data_ptr(), n, group, out.data_ptr(), norm.data_ptr(), A.stream()))
        torch.cuda.synchronize()
        assert A.guards_intact(raw_o, 2 * n) and A.guards_intact(raw_n, nb)
        ref, ref_norm = O.normalize_groups(bits, group)
        assert np.array_equal(A.to_bits(out), ref), (group, n)
        assert np.array_equal(norm.cpu().numpy(), ref_norm), (group, n)
        _lib.check(L.nz_denormalize_bf16(out.data_ptr(), n, group, norm.data_ptr(), A.stream()))
        torch.cuda.synchronize()
        assert np.array_equal(A.to_bits(out), O.denormalize_groups(ref, group, ref_norm)), (group, n)
        assert A.guards_intact(raw_o, 2 * n)


def test_normalizer_on_special_values():
    from neuzip_b200 import _lib
    L = A.lib()
    bits = np.tile(all_patterns(), 2)
    x = A.from_bits(bits)
    n = bits.size
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    norm = torch.empty(int(L.nz_normalizer_bytes(n, 64)), dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_normalize_bf16(x.data_ptr(), n, 64, out.data_ptr(), norm.data_ptr(), A.stream()))
    ref, ref_norm = O.normalize_groups(bits, 64)
    assert np.array_equal(A.to_bits(out), ref) and np.array_equal(norm.cpu().numpy(), ref_norm)


# ------------------------------------------------- full-size and stress cases
def test_largest_baseline_tensor_round_trips_on_device():
    """28672 x 8192 (the largest matrix of the 70B configuration, 235 M elements):
    checked through size-independent properties on the device - lossless equality,
    lossy idempotence (compressing the decoded tensor again changes nothing) and
    the stored size against the entropy bound."""
    n = 28672 * 8192
    g = torch.Generator(device="cuda").manual_seed(70)
    x = (torch.randn(n, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    for s in (7, 3):
        S = O.default_lane_symbols(s)
        cont, frac, mw = A.compress(x, s, S)
        out, status = A.decompress(cont, frac, n, s, S, mw, canon=True)
        assert status == 0
        if s == 7:
            assert torch.equal(out.view(torch.int16), x.view(torch.int16))
        else:
            cont2, frac2, mw2 = A.compress(out, s, S)
            out2, status2 = A.decompress(cont2, frac2, n, s, S, mw2, canon=True)
            assert status2 == 0 and torch.equal(out2.view(torch.int16), out.view(torch.int16))
            assert torch.equal(frac2, frac)
        exp = ((out.view(torch.int16).to(torch.int32) >> 7) & 0xFF)
        hist = torch.bincount(exp.flatten(), minlength=256).double()
        p = hist[hist > 0] / n
        ideal = float(-(p * p.log2()).sum()) * n / 8 + frac.numel() + (n + 1023) // 1024
        assert cont.numel() + frac.numel() <= 1.025 * ideal
        del cont, frac, out


def test_concurrent_streams_do_not_interfere():
    from neuzip_b200 import _lib
    L = A.lib()
    xs = [weights(1 << 20, 800 + i).cuda() for i in range(4)]
    comps = [A.compress(x, 7, 256) for x in xs]
    outs = [torch.empty_like(x) for x in xs]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    streams = [torch.cuda.Stream() for _ in range(4)]
    torch.cuda.synchronize()
    for rep in range(5):
        for i, st in enumerate(streams):
            c, f, mw = comps[i]
            _lib.check(L.nz_decompress_bf16(c.data_ptr(), c.numel(), f.data_ptr(), xs[i].numel(), 7,
                                            256, mw, 1, outs[i].data_ptr(),
                                            status[i:].data_ptr(), st.cuda_stream))
    torch.cuda.synchronize()
    assert int(status.abs().sum().item()) == 0
    for x, o in zip(xs, outs):
        assert torch.equal(o.view(torch.int16), x.view(torch.int16))


def test_random_shapes_and_lane_lengths_property():
    rng = np.random.default_rng(123)
    for trial in range(25):
        n = int(rng.integers(1, 200000))
        s = int(rng.choice(PRECISIONS))
        S = int(rng.choice([8, 16, 64, 128, 256, 384, 512, 640, 1024]))
        std = float(rng.choice([1e-4, 0.02, 1.0, 300.0]))
        x = weights(n, 10_000 + trial, std=std).cuda()
        cont, frac, mw = A.compress(x, s, S)
        c_ref, f_ref = O.compress_bf16(A.to_bits(x), s, S)
        assert np.array_equal(cont.cpu().numpy(), c_ref), (trial, n, s, S)
        out, status = A.decompress(cont, frac, n, s, S, mw if trial % 2 else 0, canon=True)
        assert status == 0
        assert np.array_equal(A.to_bits(out), O.decompress_bf16(c_ref, f_ref, n, s, canonical_nan=True))


# ------------------------------------------------------------------ gather
@pytest.mark.parametrize("s", PRECISIONS)
def test_unit_gather_equals_slices_of_the_full_decode(s):
    rng = np.random.default_rng(21 + s)
    for S, n in ((64, 64 * 32 * 37 + 1234), (O.default_lane_symbols(s), 3_000_000 + 77)):
        U = 32 * S
        x = weights(n, 30 + s).cuda()
        cont, frac, mw = A.compress(x, s, S)
        full, status = A.decompress(cont, frac, n, s, S, mw)
        assert status == 0
        full_bits = A.to_bits(full)
        n_units = (n + U - 1) // U
        lists = [
            [0], [n_units - 1], list(range(n_units)), list(range(n_units - 1, -1, -1)),
            rng.integers(0, n_units, size=1).tolist(), rng.integers(0, n_units, size=5).tolist(),
            rng.integers(0, n_units, size=301).tolist(), [3, 3, 3, n_units - 1, n_units - 1, 0],
        ]
        for units in lists:
            out, status = A.decompress_units(cont, frac, n, s, S, units, mw)
            assert status == 0, (s, S, units[:4])
            got = A.to_bits(out).reshape(len(units), U)
            for i, u in enumerate(units):
                count = min(U, n - u * U)
                assert np.array_equal(got[i, :count], full_bits[u * U:u * U + count]), (s, S, u)
                assert (got[i, count:] == 0x1234).all()          # past the tensor: untouched


def test_unit_gather_with_raw_units_bad_numbers_and_empty_list():
    rng = np.random.default_rng(5)
    S, U = 256, 32 * 256
    # incompressible exponents in the first half: those units are stored raw
    bits = np.concatenate([rng.integers(0, 1 << 16, size=4 * U, dtype=np.uint16),
                           A.to_bits(weights(5 * U + 100, 9))])
    x = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()
    n = x.numel()
    cont, frac, mw = A.compress(x, 7, S)
    assert O.parse_header(cont.cpu().numpy())["n_raw_units"] >= 4
    units = [9, 0, 5, 3, 8, 1]
    out, status = A.decompress_units(cont, frac, n, 7, S, units, mw)
    assert status == 0
    got = A.to_bits(out).reshape(len(units), U)
    for i, u in enumerate(units):
        count = min(U, n - u * U)
        assert np.array_equal(got[i, :count], bits[u * U:u * U + count])
    # a unit number past the end: flagged, its place left alone, the others decoded
    out, status = A.decompress_units(cont, frac, n, 7, S, [2, 10, 4], mw)
    assert status == 0x20                                        # NZ_STATUS_BAD_UNIT
    got = A.to_bits(out).reshape(3, U)
    assert np.array_equal(got[0], bits[2 * U:3 * U]) and np.array_equal(got[2], bits[4 * U:5 * U])
    assert (got[1] == 0x1234).all()
    out, status = A.decompress_units(cont, frac, n, 7, S, [], mw)
    assert status == 0 and out.numel() == 0


@pytest.mark.parametrize("s", PRECISIONS)
@pytest.mark.parametrize("span", (48, 64, 120, 250))
def test_compress_wide_exponent_alphabets_match_oracle(s, span):
    """Exponents spread evenly over `span` values need 5.6 to 8 bits per symbol: lane
    streams longer than the coder's shared-memory slices (units coded a second time,
    straight into their slots), and from 8 bits on units stored raw.  Ragged size."""
    n = 3 * 8192 + 1234
    rng = np.random.default_rng(span + s)
    exp = rng.integers(2, 2 + span, size=n, dtype=np.uint16)
    rest = rng.integers(0, 256, size=n, dtype=np.uint16)
    bits = ((rest & 0x80) << 8) | (exp << 7) | (rest & 0x7F)
    x = A.from_bits(bits)
    for S in (O.default_lane_symbols(s), 64, 1024):
        cont, frac, mw = A.compress(x, s, S)
        c_ref, f_ref = O.compress_bf16(bits, s, S)
        assert np.array_equal(frac.cpu().numpy(), f_ref), (s, span, S)
        assert np.array_equal(cont.cpu().numpy(), c_ref), (s, span, S)
        out, status = A.decompress(cont, frac, n, s, S, mw, canon=True)
        assert status == 0
        assert np.array_equal(A.to_bits(out), O.decompress_bf16(c_ref, f_ref, n, s, canonical_nan=True))
