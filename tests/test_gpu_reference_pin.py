"""Pins the oracle and the product's split / merge kernels to REFERENCE-RUN outputs.

``oracle/_ref/libnz_ref_kernels.so`` holds the reference's own
``kernel_aligned_split`` / ``kernel_aligned_merge`` (cuda/kernels.cuh:53-217),
compiled from the reference tree and instantiated as its Manager instantiates
them for bf16 (cuda/high_level.cu:95-101, :194-201).  These tests run those
kernels on the GPU and require, bit for bit,

  reference kernel == CPU oracle (literal and closed form) == product kernel

on all 65 536 bf16 patterns and on the seed-0 4096 x 4096 matrix of benchmark
configuration 1, whose CRCs are also compared with the committed fixtures
(``tests/golden/config1.json``, ``tests/golden/reference_pin.json``).

Sizes are multiples of 1024 and buffers are sized as cuda/high_level.cu:81-93,
because the reference kernels do not guard their tail block.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import nzabi as A

pytestmark = pytest.mark.gpu

PRECISIONS = (0, 1, 3, 7)
HERE = os.path.dirname(os.path.abspath(__file__))


def ref():
    L = O.ref_lib()
    if L is None:
        pytest.skip("oracle/_ref/libnz_ref_kernels.so is not built (the reference tree is only "
                    "present where the project is built: make -C oracle ref)")
    return L


def ref_split(bits, s, group=0):
    L = ref()
    n = bits.size
    assert n % 1024 == 0
    x = A.from_bits(bits)
    exp = torch.full((n,), 0xEE, dtype=torch.uint8, device="cuda")
    frac = torch.full((O.frac_bytes(n, s),), 0xEE, dtype=torch.uint8, device="cuda")
    norm = torch.full(((n + (group or 1024) - 1) // (group or 1024),), 0xEE, dtype=torch.uint8,
                      device="cuda")
    rc = L.nzref_split(s, group, x.data_ptr(), exp.data_ptr(), frac.data_ptr(), norm.data_ptr(), n,
                       A.stream())
    assert rc == 0
    torch.cuda.synchronize()
    return exp.cpu().numpy(), frac.cpu().numpy(), norm.cpu().numpy()


def ref_merge(exp, frac, s, group=0, norm=None):
    L = ref()
    n = exp.size
    assert n % 1024 == 0
    d_exp, d_frac = A.dev_u8(exp), A.dev_u8(frac)
    if norm is None:
        norm = np.zeros((n + 1023) // 1024, np.uint8)
    d_norm = A.dev_u8(norm)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    rc = L.nzref_merge(s, group, out.data_ptr(), d_exp.data_ptr(), d_frac.data_ptr(),
                       d_norm.data_ptr(), n, A.stream())
    assert rc == 0
    torch.cuda.synchronize()
    return A.to_bits(out)


def config1_bits():
    torch.manual_seed(0)
    w = (torch.randn(4096, 4096, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return w.view(torch.int16).numpy().view(np.uint16).reshape(-1)


@pytest.mark.parametrize("s", PRECISIONS)
def test_split_of_all_patterns_equals_the_reference_kernel(s):
    bits = np.arange(65536, dtype=np.uint16)
    e_ref, f_ref, _ = ref_split(bits, s)
    e_lit, f_lit = O.split(bits, s, literal=True)
    e_cf, f_cf = O.split(bits, s)
    assert np.array_equal(e_ref, e_lit) and np.array_equal(f_ref, f_lit)
    assert np.array_equal(e_ref, e_cf) and np.array_equal(f_ref, f_cf)
    exp, frac = A.split(A.from_bits(bits), s)
    assert np.array_equal(exp.cpu().numpy(), e_ref)
    assert np.array_equal(frac.cpu().numpy(), f_ref)


@pytest.mark.parametrize("s", PRECISIONS)
def test_merge_of_all_patterns_equals_the_reference_kernel(s):
    """Includes what the reference does with NaN patterns (its float -> bf16 store) and
    with exponent bytes that wrapped from 255 to 0 in the lossy split."""
    bits = np.arange(65536, dtype=np.uint16)
    e_ref, f_ref, _ = ref_split(bits, s)
    got_ref = ref_merge(e_ref, f_ref, s)
    assert np.array_equal(got_ref, O.merge(e_ref, f_ref, s, canonical_nan=True))
    out = A.merge(A.dev_u8(e_ref), A.dev_u8(f_ref), bits.size, s, canon=True)
    assert np.array_equal(A.to_bits(out), got_ref)
    # the fused decode path of the product (rANS container) gives the same tensor
    S = O.default_lane_symbols(s)
    cont, frac, mw = A.compress(A.from_bits(bits), s, S)
    dec, status = A.decompress(cont, frac, bits.size, s, S, mw, canon=True)
    assert status == 0
    assert np.array_equal(A.to_bits(dec), got_ref)


def test_config1_matrix_and_its_fixtures():
    bits = config1_bits()
    with open(os.path.join(HERE, "golden", "config1.json")) as f:
        golden = json.load(f)
    pin_path = os.path.join(HERE, "golden", "reference_pin.json")
    pin = None
    if os.path.exists(pin_path):
        with open(pin_path) as f:
            pin = json.load(f)
    for s in PRECISIONS:
        e_ref, f_ref, _ = ref_split(bits, s)
        rt_ref = ref_merge(e_ref, f_ref, s)
        crcs = {"exp_crc32": hex(O.crc32(e_ref)), "frac_crc32": hex(O.crc32(f_ref)),
                "roundtrip_crc32": hex(O.crc32(rt_ref))}
        for key, value in crcs.items():
            assert golden["precision"][str(s)][key] == value, (s, key)
            if pin is not None:
                assert pin["precision"][str(s)][key] == value, (s, key)
        e, f = O.split(bits, s)
        assert np.array_equal(e, e_ref) and np.array_equal(f, f_ref)
        exp, frac = A.split(A.from_bits(bits), s)
        assert np.array_equal(exp.cpu().numpy(), e_ref)
        assert np.array_equal(frac.cpu().numpy(), f_ref)


@pytest.mark.parametrize("group", (1, 2, 4, 8, 16, 32, 1024))
@pytest.mark.parametrize("s", PRECISIONS)
def test_block_normaliser_equals_the_reference_kernel(s, group):
    """normalized=true instantiations for the group sizes whose block reduction is well
    defined in the reference (one warp at most, or the whole block)."""
    from neuzip_b200 import _lib
    g = torch.Generator().manual_seed(17 + s + group)
    w = (torch.randn(64 * 1024, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    w[5 * 1024:6 * 1024] = 0          # an all-zero group
    w[7] = 0.5
    bits = w.view(torch.int16).numpy().view(np.uint16).reshape(-1)
    n = bits.size
    e_ref, f_ref, norm_ref = ref_split(bits, s, group)
    scaled, norm = O.normalize_groups(bits, group)
    e, f = O.split(scaled, s)
    assert np.array_equal(norm, norm_ref)
    assert np.array_equal(e, e_ref) and np.array_equal(f, f_ref)
    rt_ref = ref_merge(e_ref, f_ref, s, group, norm_ref)
    rt = O.denormalize_groups(O.merge(e, f, s, canonical_nan=True), group, norm)
    assert np.array_equal(rt, rt_ref)
    # product kernels
    L = A.lib()
    x = A.from_bits(bits)
    out = torch.empty_like(x)
    d_norm = torch.empty(int(L.nz_normalizer_bytes(n, group)), dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_normalize_bf16(x.data_ptr(), n, group, out.data_ptr(), d_norm.data_ptr(), A.stream()))
    assert np.array_equal(d_norm.cpu().numpy(), norm_ref)
    exp, frac = A.split(out, s)
    assert np.array_equal(exp.cpu().numpy(), e_ref) and np.array_equal(frac.cpu().numpy(), f_ref)
    merged = A.merge(exp, frac, n, s, canon=True)
    _lib.check(L.nz_denormalize_bf16(merged.data_ptr(), n, group, d_norm.data_ptr(), A.stream()))
    assert np.array_equal(A.to_bits(merged), rt_ref)
