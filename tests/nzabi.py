"""Test helper: thin torch-tensor wrappers over the C-ABI entry points, so the
GPU parity tests call exactly what a foreign binding would call."""
import ctypes

import numpy as np
import torch

from neuzip_b200 import _lib

CANARY = 0xA5
GUARD = 256


def lib():
    return _lib.load()


def stream():
    return torch.cuda.current_stream().cuda_stream


def guarded(nbytes, dtype=torch.uint8):
    """Device buffer of nbytes with canary bands before and after it."""
    item = torch.empty(0, dtype=dtype).element_size()
    raw = torch.full((nbytes + 2 * GUARD,), CANARY, dtype=torch.uint8, device="cuda")
    view = raw[GUARD:GUARD + nbytes].view(dtype) if nbytes else raw[GUARD:GUARD].view(dtype)
    assert nbytes % item == 0
    return raw, view


def guards_intact(raw, nbytes):
    host = raw.cpu().numpy()
    return bool((host[:GUARD] == CANARY).all() and (host[GUARD + nbytes:] == CANARY).all())


def to_bits(t):
    """bf16 tensor -> numpy uint16 bit patterns."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)


def from_bits(bits, device="cuda"):
    a = np.ascontiguousarray(bits, dtype=np.uint16).view(np.int16)
    return torch.from_numpy(a.copy()).view(torch.bfloat16).to(device)


def split(x_bf16, s):
    L = lib()
    n = x_bf16.numel()
    fb = int(L.nz_frac_bytes(n, s))
    raw_e, exp = guarded(n)
    raw_f, frac = guarded(fb)
    _lib.check(L.nz_split_bf16(x_bf16.data_ptr(), n, s, exp.data_ptr(), frac.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_e, n) and guards_intact(raw_f, fb)
    return exp, frac


def merge(exp, frac, n, s, canon=False):
    L = lib()
    raw_o, out = guarded(2 * n, torch.bfloat16)
    _lib.check(L.nz_merge_bf16(exp.data_ptr(), frac.data_ptr(), n, s, int(canon), out.data_ptr(),
                               stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_o, 2 * n)
    return out


def encode(exp, S):
    """exponent bytes (cuda uint8) -> right-sized container tensor + max unit words."""
    L = lib()
    n = exp.numel()
    cap = int(L.nz_container_bound(n, S))
    raw_c, cont = guarded(cap)
    sb = int(L.nz_encode_scratch_bytes(n, S))
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_encode_exponents(exp.data_ptr(), n, S, cont.data_ptr(), cap,
                                     scratch.data_ptr(), sb, stream()))
    total, mw = ctypes.c_uint64(0), ctypes.c_uint32(0)
    _lib.check(L.nz_container_bytes(cont.data_ptr(), total, mw, stream()))
    assert guards_intact(raw_c, cap)
    return cont[: total.value].clone(), int(mw.value)


def compress(x_bf16, s, S):
    L = lib()
    n = x_bf16.numel()
    cap = int(L.nz_container_bound(n, S))
    fb = int(L.nz_frac_bytes(n, s))
    raw_c, cont = guarded(cap)
    raw_f, frac = guarded(fb)
    sb = int(L.nz_compress_scratch_bytes(n, S))
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_compress_bf16(x_bf16.data_ptr(), n, s, S, frac.data_ptr(), cont.data_ptr(), cap,
                                  scratch.data_ptr(), sb, stream()))
    total, mw = ctypes.c_uint64(0), ctypes.c_uint32(0)
    _lib.check(L.nz_container_bytes(cont.data_ptr(), total, mw, stream()))
    assert guards_intact(raw_c, cap) and guards_intact(raw_f, fb)
    return cont[: total.value].clone(), frac.clone(), int(mw.value)


def decode_exponents(cont, n, S, max_words=0):
    L = lib()
    raw_e, exp = guarded(n)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decode_exponents(cont.data_ptr(), cont.numel(), n, S, max_words,
                                     exp.data_ptr(), status.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_e, n)
    return exp, int(status.item())


def decompress(cont, frac, n, s, S, max_words=0, canon=False):
    L = lib()
    raw_o, out = guarded(2 * n, torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16(cont.data_ptr(), cont.numel(), frac.data_ptr(), n, s, S,
                                    max_words, int(canon), out.data_ptr(), status.data_ptr(),
                                    stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_o, 2 * n)
    return out, int(status.item())


def decompress_units(cont, frac, n, s, S, units, max_words=0, canon=False, fill=0x1234):
    """Gather-decode the listed units; returns (bf16 [len(units) * 32 * S], status).  The
    output starts out filled with `fill` so that untouched elements are recognisable."""
    L = lib()
    U = 32 * S
    ids = torch.as_tensor(np.asarray(units, dtype=np.int64), dtype=torch.int64).to(torch.int32).cuda()
    k = ids.numel()
    raw_o, out = guarded(2 * k * U, torch.bfloat16)
    out.view(torch.int16).fill_(fill)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16_units(cont.data_ptr(), cont.numel(), frac.data_ptr(), n, s, S,
                                          max_words, int(canon), ids.data_ptr(), k, out.data_ptr(),
                                          status.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_o, 2 * k * U)
    return out, int(status.item())


def dev_u8(a):
    """numpy uint8 -> 16-byte aligned cuda tensor."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint8).copy()).cuda()


def compress_operand(x_bf16, rows, cols, s, S):
    """[rows, cols] bf16 (cuda) -> (container, fractions, max unit words), operand order."""
    L = lib()
    n = rows * cols
    cap = int(L.nz_container_bound(n, S))
    fb = int(L.nz_frac_bytes(n, s))
    raw_c, cont = guarded(cap)
    raw_f, frac = guarded(fb)
    sb = int(L.nz_compress_operand_scratch_bytes(rows, cols, S))
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_compress_bf16_operand(x_bf16.data_ptr(), rows, cols, s, S, frac.data_ptr(),
                                          cont.data_ptr(), cap, scratch.data_ptr(), sb, stream()))
    total, mw = ctypes.c_uint64(0), ctypes.c_uint32(0)
    _lib.check(L.nz_container_bytes(cont.data_ptr(), total, mw, stream()))
    assert guards_intact(raw_c, cap) and guards_intact(raw_f, fb)
    return cont[: total.value].clone(), frac.clone(), int(mw.value)


def decompress_operand(cont, frac, rows, cols, s, S, max_words=0, canon=False):
    L = lib()
    n = rows * cols
    raw_o, out = guarded(2 * n, torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_decompress_bf16_operand(cont.data_ptr(), cont.numel(), frac.data_ptr(), rows,
                                            cols, s, S, max_words, int(canon), out.data_ptr(),
                                            status.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_o, 2 * n)
    return out, int(status.item())


def linear(cont, frac, rows, cols, s, S, x, bias=None, max_words=0, canon=False):
    """y = x W^T (+ bias) through nz_linear_bf16; x is [m, cols] bf16 (cuda).  Returns
    (y [m, rows] bf16, status)."""
    L = lib()
    m = x.shape[0]
    raw_y, y = guarded(2 * m * rows, torch.bfloat16)
    wb = int(L.nz_linear_workspace_bytes(rows, cols, S, m))
    ws = torch.empty(wb, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(L.nz_linear_bf16(cont.data_ptr(), cont.numel(), frac.data_ptr(), rows, cols, s, S,
                                max_words, int(canon), x.data_ptr(), m,
                                0 if bias is None else bias.data_ptr(), y.data_ptr(),
                                ws.data_ptr(), wb, status.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert guards_intact(raw_y, 2 * m * rows)
    return y.view(m, rows), int(status.item())
