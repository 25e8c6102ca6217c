"""CPU tests of the oracle itself: the literal restatement of the reference's
split kernel against the closed form and a numpy restatement, the committed
golden values, and the NZR1 container codec."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

PRECISIONS = (0, 1, 3, 7)
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "config1.json")))


def gaussian_bits(n, seed, std=0.02):
    import torch
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    return w.view(torch.int16).numpy().view(np.uint16).copy()


@pytest.mark.parametrize("s", PRECISIONS)
def test_literal_closed_form_and_numpy_agree_on_every_pattern(s):
    bits = np.arange(65536, dtype=np.uint16)
    e1, f1 = O.split(bits, s, literal=True)
    e2, f2 = O.split(bits, s)
    e3, f3 = O.split_numpy(bits, s)
    assert np.array_equal(e1, e2) and np.array_equal(f1, f2)
    assert np.array_equal(e1, e3) and np.array_equal(f1, f3)
    m = O.merge(e1, f1, s)
    assert np.array_equal(m, O.merge_numpy(e1, f1, s))
    assert int((m == bits).sum()) == GOLDEN["precision"][str(s)]["roundtrip_identical_patterns"]


def test_lossless_merge_is_identity_except_canonical_nan():
    bits = np.arange(65536, dtype=np.uint16)
    e, f = O.split(bits, 7)
    assert np.array_equal(O.merge(e, f, 7), bits)
    canon = O.merge(e, f, 7, canonical_nan=True)
    nan = ((bits & 0x7F80) == 0x7F80) & ((bits & 0x7F) != 0)
    assert np.array_equal(canon[~nan], bits[~nan])
    assert (canon[nan] == 0x7FFF).all()


@pytest.mark.parametrize("s", (0, 1, 3))
def test_rounding_is_half_up_on_magnitude_with_carry_into_exponent(s):
    # 1.9921875 = 0x3FFF: mantissa all ones -> rounds up to 2.0 (exponent + 1, fraction 0)
    e, f = O.split(np.array([0x3FFF, 0xBFFF], np.uint16), s)
    assert list(e) == [0x80, 0x80]
    out = O.merge(e, f, s)
    assert list(out) == [0x4000, 0xC000]
    # exponent 255 that overflows wraps to 0 (uint8 store of the reference)
    e, _ = O.split(np.array([0x7FFF], np.uint16), s)
    assert e[0] == 0


def test_tail_bits_are_zero_and_sizes_follow_the_reference():
    for s in PRECISIONS:
        for n in (1, 3, 9, 1001):
            e, f = O.split(np.full(n, 0xFFFF, np.uint16), s)
            assert f.size == (n * (s + 1) + 7) // 8
            used = n * (s + 1)
            if used % 8:
                assert f[-1] & ((1 << (8 - used % 8)) - 1) == 0


def test_config1_golden_values():
    import torch
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bits = w.view(torch.int16).numpy().view(np.uint16).reshape(-1)
    assert hex(O.crc32(bits)) == GOLDEN["input_crc32"]
    assert [hex(int(v)) for v in bits[:4]] == GOLDEN["first_four"]
    for s in PRECISIONS:
        g = GOLDEN["precision"][str(s)]
        e, f = O.split(bits, s)
        assert hex(O.crc32(e)) == g["exp_crc32"]
        assert hex(O.crc32(f)) == g["frac_crc32"]
        cont, f2 = O.compress_bf16(bits, s, g["lane_symbols"])
        assert np.array_equal(f2, f)
        assert O.parse_header(cont)["prob_bits"] == g["prob_bits"]
        assert cont.size == g["container_bytes"]
        assert hex(O.crc32(cont)) == g["container_crc32"]
        rt = O.decompress_bf16(cont, f, bits.size, s, canonical_nan=True)
        assert hex(O.crc32(rt)) == g["roundtrip_crc32"]
        # stored size within 2 % of the entropy-bound size (includes ceil(N/1024) bytes
        # the reference counts for its unused normaliser buffer)
        assert cont.size + f.size <= 1.025 * g["ideal_bytes"]


# ------------------------------------------------------------------ normalise
def test_normalize_invariants():
    rng = np.random.default_rng(0)
    for trial in range(200):
        k = int(rng.integers(1, 257))
        hist = np.zeros(256, np.uint64)
        idx = rng.choice(256, size=k, replace=False)
        hist[idx] = rng.integers(1, 10 ** int(rng.integers(1, 9)), size=k).astype(np.uint64)
        pb = O.choose_prob_bits(hist)
        dominated = int(hist.max()) * 4096 >= int(hist.sum()) * 1900
        assert pb == (10 if k <= 32 else 11 if k <= 64 or dominated else 12)
        f, best = O.normalize(hist)
        assert int(f.sum()) == 1 << pb
        assert f.max() <= 2047               # what the GPU decoder's table entry can hold
        assert (f[hist > 0] >= 1).all()
        assert f.max() <= (1 << pb) - 1
        for forced in (10, 11, 12):
            if k <= (1 << forced) // 2:
                g, _ = O.normalize(hist, forced)
                assert int(g.sum()) == 1 << forced and (g[hist > 0] >= 1).all()
        if k > 1:
            assert (f[hist == 0] == 0).all()
        assert hist[best] == hist.max()


def test_normalize_single_symbol_and_empty():
    hist = np.zeros(256, np.uint64)
    hist[255] = 10
    f, _ = O.normalize(hist)
    assert f[255] == 1023 and f[0] == 1 and f.sum() == 1024
    f, _ = O.normalize(hist, 12)
    assert f[255] == 4095 and f[0] == 1 and f.sum() == 4096
    f, _ = O.normalize(np.zeros(256, np.uint64))
    assert f[0] == 1023 and f[1] == 1


# ---------------------------------------------------------------- container
def streams():
    rng = np.random.default_rng(5)
    yield "empty", np.zeros(0, np.uint8)
    yield "one", np.array([42], np.uint8)
    yield "constant", np.full(5000, 121, np.uint8)
    yield "gauss", O.split(gaussian_bits(50000, 1), 7)[0]
    yield "uniform", rng.integers(0, 256, size=30000, dtype=np.uint8)
    yield "two", rng.choice(np.array([0, 255], np.uint8), size=9999, p=[0.97, 0.03])
    yield "mixed", np.concatenate([rng.integers(0, 256, size=8192, dtype=np.uint8),
                                   np.full(8192, 7, np.uint8)])


@pytest.mark.parametrize("S", (8, 16, 256, 384, 512, 1024))
def test_container_roundtrip(S):
    for name, sym in streams():
        cont = O.encode(sym, S)
        h = O.parse_header(cont)
        assert h["n_symbols"] == sym.size and h["lane_symbols"] == S
        assert cont.size == h["total_bytes"] and cont.size % 16 == 0
        assert h["payload_offset"] % 16 == 0
        assert cont.size <= O.container_bound(sym.size, S)
        assert np.array_equal(O.decode(cont, sym.size), sym), name


def test_incompressible_units_are_stored_raw():
    rng = np.random.default_rng(1)
    sym = rng.integers(0, 256, size=1 << 16, dtype=np.uint8)
    cont = O.encode(sym, 256)
    h = O.parse_header(cont)
    assert h["n_raw_units"] == h["n_units"]
    assert cont.size <= sym.size + 576 + 4 * (h["n_units"] + 1) + 48


def test_c_decoder_matches_pure_python_decoder():
    for name, sym in streams():
        if sym.size > 20000 or sym.size == 0:
            continue
        for S in (8, 64):
            cont = O.encode(sym[:3000], S)
            assert np.array_equal(O.decode_python(cont, min(sym.size, 3000)), sym[:3000]), name


def test_compression_is_close_to_entropy():
    exp = O.split(gaussian_bits(1 << 20, 2), 7)[0]
    h = O.histogram(exp).astype(np.float64)
    p = h[h > 0] / h.sum()
    ideal = -(p * np.log2(p)).sum() * exp.size / 8
    for S, slack in ((256, 1.065), (512, 1.04), (1024, 1.03)):
        assert O.encode(exp, S).size <= slack * ideal + 1024


def test_external_frequency_table_is_honoured():
    exp = O.split(gaussian_bits(20000, 3), 7)[0]
    hist = O.histogram(exp)
    f, _ = O.normalize(hist)
    a = O.encode(exp, 256)
    b = O.encode(exp, 256, freq=f, prob_bits=O.choose_prob_bits(hist))
    assert np.array_equal(a, b)
    for pb in (9, 10, 11, 12):    # every resolution round-trips
        c = O.encode(exp, 256, prob_bits=pb)
        assert O.parse_header(c)["prob_bits"] == pb
        assert np.array_equal(O.decode(c, exp.size), exp)


def test_lossless_compress_uses_nine_bit_probabilities():
    bits = gaussian_bits(50000, 5)
    hist = O.histogram(O.split(bits, 7)[0])
    assert O.choose_prob_bits(hist) == 10 and O.choose_prob_bits(hist, 7) == 9
    assert O.choose_prob_bits(hist, 3) == 10
    for s, pb in ((7, 9), (3, 10), (1, 10), (0, 10)):
        cont, frac = O.compress_bf16(bits, s)
        assert O.parse_header(cont)["prob_bits"] == pb
        assert np.array_equal(O.decompress_bf16(cont, frac, bits.size, s),
                              O.merge(*O.split(bits, s), s))
    wide = np.arange(65536, dtype=np.uint16)          # every exponent: 12 bits at any precision
    assert O.parse_header(O.compress_bf16(wide, 7)[0])["prob_bits"] == 12


def test_corrupt_containers_are_rejected_or_decode_without_crashing():
    exp = O.split(gaussian_bits(30000, 4), 7)[0]
    cont = O.encode(exp, 256)
    h = O.parse_header(cont)
    bad = cont.copy(); bad[0] ^= 1
    assert O.decode_status(bad, exp.size) == -2
    assert O.decode_status(cont, exp.size + 1) == -3
    assert O.decode_status(cont[:-16], exp.size) == -7
    bad = cont.copy(); bad[64] ^= 1
    assert O.decode_status(bad, exp.size) == -8
    bad = cont.copy(); bad[h["payload_offset"] + 3] = 0
    assert O.decode_status(bad, exp.size) in (-11, -14)
    rng = np.random.default_rng(0)
    for _ in range(300):          # random single-byte damage never crashes the decoder
        bad = cont.copy()
        bad[int(rng.integers(0, cont.size))] ^= int(rng.integers(1, 256))
        O.decode_status(bad, exp.size)


def test_hypothesis_roundtrip():
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.binary(min_size=0, max_size=3000), st.sampled_from([8, 24, 256]))
    def run(data, S):
        sym = np.frombuffer(data, np.uint8)
        assert np.array_equal(O.decode(O.encode(sym, S), sym.size), sym)

    run()


def test_oracle_reproduces_the_reference_run_fixture():
    """tests/golden/reference_pin.json holds CRC-32s of what the reference's own
    kernel_aligned_split / kernel_aligned_merge produced on a B200 (generated by
    tests/golden/make_reference_pin.py from oracle/_ref).  The CPU oracle must give the
    same streams and the same merged tensors, NaN canonicalisation included."""
    import json
    import os
    import torch
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_pin.json")
    with open(path) as f:
        pin = json.load(f)
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    cases = {"precision": w.view(torch.int16).numpy().view(np.uint16).reshape(-1),
             "all_patterns": np.arange(65536, dtype=np.uint16)}
    assert hex(O.crc32(cases["precision"])) == pin["input_crc32"]
    for key, bits in cases.items():
        for s in (0, 1, 3, 7):
            want = pin[key][str(s)]
            e, f = O.split(bits, s)
            assert hex(O.crc32(e)) == want["exp_crc32"], (key, s)
            assert hex(O.crc32(f)) == want["frac_crc32"], (key, s)
            rt = O.merge(e, f, s, canonical_nan=True)
            assert hex(O.crc32(rt)) == want["roundtrip_crc32"], (key, s)
            if "roundtrip_identical_patterns" in want:
                assert int((rt == bits).sum()) == want["roundtrip_identical_patterns"]
