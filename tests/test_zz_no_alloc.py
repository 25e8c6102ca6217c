"""The allocation-free encoder entry point, nz_encode_exponents_static_scratch.

It is meant for hosts that cannot allocate device memory while compressing (a
server whose arena owns the whole GPU, a framework that bans cudaMalloc on its
hot path because it synchronises the device), so its scratch is a fixed array
inside the library.  This file is named to be collected last: if it fails, a
run that stops at the first failure has already exercised everything else.

The test calls the entry point through the C ABI twice in a row, on different
inputs of different sizes (the second call finds the first call's leftovers in
the shared array), and requires containers identical, byte for byte, to those of
nz_encode_exponents with caller-provided scratch - the same exactness every
other codec test here uses.  Inputs, outputs and the reference scratch are
allocated by the test before the calls; the entry point itself gets no scratch.
"""
import ctypes

import numpy as np
import pytest
import torch

from neuzip_b200 import _lib

pytestmark = pytest.mark.gpu


def _exponents(n, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bits = w.view(torch.int16).numpy().view(np.uint16)
    return torch.from_numpy(((bits >> 7) & 0xFF).astype(np.uint8)).cuda()


def _encode_with_caller_scratch(L, exp, S, stream):
    n = exp.numel()
    cap = int(L.nz_container_bound(n, S))
    cont = torch.zeros(cap, dtype=torch.uint8, device="cuda")
    sb = int(L.nz_encode_scratch_bytes(n, S))
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_encode_exponents(exp.data_ptr(), n, S, cont.data_ptr(), cap,
                                     scratch.data_ptr(), sb, stream))
    total = ctypes.c_uint64(0)
    _lib.check(L.nz_container_bytes(cont.data_ptr(), total, None, stream))
    return cont[: total.value].cpu().numpy()


def test_static_scratch_encoder_matches_the_allocating_one_twice_in_a_row():
    L = _lib.load()
    _lib.check(L.nz_device_check())
    stream = torch.cuda.current_stream().cuda_stream
    assert L.nz_static_scratch_bytes() == 6 << 20
    # everything the calls touch is allocated up front
    cases = [(_exponents(1_500_000, 21), 256), (_exponents(70_001, 22), 64)]
    expected = [_encode_with_caller_scratch(L, exp, S, stream) for exp, S in cases]
    outputs = []
    for exp, S in cases:
        cap = int(L.nz_container_bound(exp.numel(), S))
        outputs.append(torch.zeros(cap, dtype=torch.uint8, device="cuda"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    # free device memory as the driver reports it: unlike torch's own counter it would
    # also show a cudaMalloc made inside the library (the kernels involved ran above, so
    # their module, with its built-in array, is already resident)
    free_before, _ = torch.cuda.mem_get_info()
    for (exp, S), cont in zip(cases, outputs):          # two calls, back to back
        _lib.check(L.nz_encode_exponents_static_scratch(exp.data_ptr(), exp.numel(), S,
                                                        cont.data_ptr(), cont.numel(), stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before       # torch's allocator was not involved
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before                     # and nothing else took device memory
    for (exp, S), cont, ref in zip(cases, outputs, expected):
        total = ctypes.c_uint64(0)
        _lib.check(L.nz_container_bytes(cont.data_ptr(), total, None, stream))
        got = cont[: total.value].cpu().numpy()
        assert got.size == ref.size
        assert np.array_equal(got, ref)
    # and the containers decode back to the input
    for (exp, S), cont in zip(cases, outputs):
        n = exp.numel()
        back = torch.empty(n, dtype=torch.uint8, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(L.nz_decode_exponents(cont.data_ptr(), cont.numel(), n, S, 0, back.data_ptr(),
                                         status.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(back, exp)


def test_static_scratch_encoder_rejects_what_does_not_fit():
    L = _lib.load()
    n, S = 16 << 20, 256
    assert L.nz_encode_scratch_bytes(n, S) > L.nz_static_scratch_bytes()
    exp = torch.zeros(16, dtype=torch.uint8, device="cuda")       # never read: the call refuses first
    cont = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = L.nz_encode_exponents_static_scratch(exp.data_ptr(), n, S, cont.data_ptr(),
                                              int(L.nz_container_bound(n, S)), 0)
    assert rc == _lib.NZ_E_CAPACITY
    msg = L.nz_last_error().decode()
    assert "scratch" in msg and "nz_encode_exponents" in msg
