"""numpy front-end of the CPU oracle (``nz_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the shipped package never does.  See the header of
``nz_oracle.c`` for the parity status (pinned to outputs of the reference's own
split / merge kernels run on a B200) and for the container specification.

Every function takes and returns numpy arrays; bf16 tensors travel as their
uint16 bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnz_oracle.so")

MAX_PROB_BITS = 12
HEADER_BYTES = 64
FREQ_OFFSET = 64
OFFSETS_OFFSET = 576


def build(force: bool = False) -> str:
    """Compile ``nz_oracle.c`` with the Makefile next to it (gcc only)."""
    src = os.path.join(_HERE, "nz_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libnz_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        vp, u64, u32, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
        L.nzo_split_literal.argtypes = [vp, ctypes.c_size_t, i32, vp, vp]
        L.nzo_split_literal.restype = None
        L.nzo_split.argtypes = [vp, ctypes.c_size_t, i32, vp, vp]
        L.nzo_split.restype = None
        L.nzo_merge.argtypes = [vp, vp, ctypes.c_size_t, i32, i32, vp]
        L.nzo_merge.restype = None
        L.nzo_histogram.argtypes = [vp, ctypes.c_size_t, vp]
        L.nzo_histogram.restype = None
        L.nzo_normalize.argtypes = [vp, u32, vp]
        L.nzo_choose_prob_bits.argtypes = [vp]
        L.nzo_choose_prob_bits.restype = u32
        L.nzo_choose_prob_bits_for.argtypes = [vp, ctypes.c_int]
        L.nzo_choose_prob_bits_for.restype = u32
        L.nzo_normalize.restype = u32
        L.nzo_len_quantum.argtypes = [u32]
        L.nzo_len_quantum.restype = u32
        L.nzo_container_bound.argtypes = [u64, u32]
        L.nzo_container_bound.restype = u64
        L.nzo_encode.argtypes = [vp, u64, u32, vp, u32, vp, u64]
        L.nzo_encode.restype = u64
        L.nzo_decode.argtypes = [vp, u64, vp, u64]
        L.nzo_decode.restype = i32
        L.nzo_compress_bf16.argtypes = [vp, u64, i32, u32, vp, vp, vp, u64]
        L.nzo_compress_bf16.restype = u64
        L.nzo_decompress_bf16.argtypes = [vp, u64, vp, u64, i32, i32, vp, vp]
        L.nzo_decompress_bf16.restype = i32
        L.nzo_normalize_groups.argtypes = [vp, u64, u32, vp, vp]
        L.nzo_normalize_groups.restype = None
        L.nzo_denormalize_groups.argtypes = [vp, u64, u32, vp]
        L.nzo_denormalize_groups.restype = None
        L.nzo_crc32.argtypes = [vp, u64]
        L.nzo_crc32.restype = u32
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def frac_bytes(n: int, s: int) -> int:
    """Size of the packed sign+mantissa stream (cuda/high_level.cu:81-83)."""
    return (n * (s + 1) + 7) // 8


def default_lane_symbols(s: int) -> int:
    """Symbols per lane stream written by default: the shorter the lane stream the more
    parallel the decode, the longer the smaller the container; lossy modes store fewer
    bytes in total, so the coarsest get the longer streams (the GPU library's
    nz_default_lane_symbols must agree)."""
    return {7: 256, 3: 256, 1: 384, 0: 512}[s]


def split(bits: np.ndarray, s: int, literal: bool = False) -> Tuple[np.ndarray, np.ndarray]:
    bits = np.ascontiguousarray(bits.reshape(-1), dtype=np.uint16)
    n = bits.size
    exp = np.empty(n, np.uint8)
    frac = np.empty(frac_bytes(n, s), np.uint8)
    fn = lib().nzo_split_literal if literal else lib().nzo_split
    fn(_p(bits), n, s, _p(exp), _p(frac))
    return exp, frac


def merge(exp: np.ndarray, frac: np.ndarray, s: int, canonical_nan: bool = False) -> np.ndarray:
    exp = np.ascontiguousarray(exp.reshape(-1), dtype=np.uint8)
    frac = np.ascontiguousarray(frac.reshape(-1), dtype=np.uint8)
    n = exp.size
    assert frac.size >= frac_bytes(n, s)
    out = np.empty(n, np.uint16)
    lib().nzo_merge(_p(exp), _p(frac), n, s, int(canonical_nan), _p(out))
    return out


def histogram(sym: np.ndarray) -> np.ndarray:
    sym = np.ascontiguousarray(sym.reshape(-1), dtype=np.uint8)
    h = np.zeros(256, np.uint64)
    lib().nzo_histogram(_p(sym), sym.size, _p(h))
    return h


def choose_prob_bits(hist: np.ndarray, precision: Optional[int] = None) -> int:
    """Resolution for an exponent histogram; with `precision`, the choice of the
    whole-tensor compressor (9 bits instead of 10 at precision 7)."""
    hist = np.ascontiguousarray(hist, dtype=np.uint64)
    if precision is None:
        return int(lib().nzo_choose_prob_bits(_p(hist)))
    return int(lib().nzo_choose_prob_bits_for(_p(hist), int(precision)))


def normalize(hist: np.ndarray, prob_bits: Optional[int] = None) -> Tuple[np.ndarray, int]:
    hist = np.ascontiguousarray(hist, dtype=np.uint64)
    if prob_bits is None:
        prob_bits = choose_prob_bits(hist)
    f = np.zeros(256, np.uint16)
    best = lib().nzo_normalize(_p(hist), prob_bits, _p(f))
    return f, int(best)


def container_bound(n: int, lane_symbols: int) -> int:
    return int(lib().nzo_container_bound(n, lane_symbols))


def encode(sym: np.ndarray, lane_symbols: int, freq: Optional[np.ndarray] = None,
           prob_bits: int = 0) -> np.ndarray:
    sym = np.ascontiguousarray(sym.reshape(-1), dtype=np.uint8)
    cap = container_bound(sym.size, lane_symbols)
    out = np.zeros(cap, np.uint8)
    fp = None
    if freq is not None:
        freq = np.ascontiguousarray(freq, dtype=np.uint16)
        fp = _p(freq)
    got = lib().nzo_encode(_p(sym), sym.size, lane_symbols, fp, prob_bits, _p(out), cap)
    if got == 0:
        raise ValueError("oracle encode failed (bad lane_symbols or capacity)")
    return out[:got].copy()


def decode(container: np.ndarray, n: int) -> np.ndarray:
    container = np.ascontiguousarray(container, dtype=np.uint8)
    out = np.empty(n, np.uint8)
    rc = lib().nzo_decode(_p(container), container.size, _p(out), n)
    if rc != 0:
        raise ValueError(f"oracle decode failed with code {rc}")
    return out


def decode_status(container: np.ndarray, n: int) -> int:
    container = np.ascontiguousarray(container, dtype=np.uint8)
    out = np.empty(max(n, 1), np.uint8)
    return int(lib().nzo_decode(_p(container), container.size, _p(out), n))


def compress_bf16(bits: np.ndarray, s: int, lane_symbols: Optional[int] = None):
    """split + encode; returns (container, packed fractions)."""
    bits = np.ascontiguousarray(bits.reshape(-1), dtype=np.uint16)
    S = lane_symbols or default_lane_symbols(s)
    n = bits.size
    cap = container_bound(n, S)
    cont = np.zeros(cap, np.uint8)
    frac = np.empty(frac_bytes(n, s), np.uint8)
    scratch = np.empty(max(n, 1), np.uint8)
    got = lib().nzo_compress_bf16(_p(bits), n, s, S, _p(scratch), _p(frac), _p(cont), cap)
    if got == 0:
        raise ValueError("oracle compress failed")
    return cont[:got].copy(), frac


def decompress_bf16(cont: np.ndarray, frac: np.ndarray, n: int, s: int,
                    canonical_nan: bool = False, scratch: Optional[np.ndarray] = None,
                    out: Optional[np.ndarray] = None) -> np.ndarray:
    cont = np.ascontiguousarray(cont, dtype=np.uint8)
    frac = np.ascontiguousarray(frac, dtype=np.uint8)
    if scratch is None:
        scratch = np.empty(max(n, 1), np.uint8)
    if out is None:
        out = np.empty(n, np.uint16)
    rc = lib().nzo_decompress_bf16(_p(cont), cont.size, _p(frac), n, s, int(canonical_nan),
                                   _p(scratch), _p(out))
    if rc != 0:
        raise ValueError(f"oracle decompress failed with code {rc}")
    return out


def normalize_groups(bits: np.ndarray, group: int) -> Tuple[np.ndarray, np.ndarray]:
    """Block normaliser before the split: returns (scaled bf16 bits, normaliser bytes)."""
    bits = np.ascontiguousarray(bits.reshape(-1), dtype=np.uint16)
    out = np.empty_like(bits)
    norm = np.empty((bits.size + group - 1) // group, np.uint8)
    lib().nzo_normalize_groups(_p(bits), bits.size, group, _p(out), _p(norm))
    return out, norm


def denormalize_groups(bits: np.ndarray, group: int, normalizers: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(bits.reshape(-1), dtype=np.uint16).copy()
    normalizers = np.ascontiguousarray(normalizers, dtype=np.uint8)
    lib().nzo_denormalize_groups(_p(out), out.size, group, _p(normalizers))
    return out


def crc32(a: np.ndarray) -> int:
    a = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
    return int(lib().nzo_crc32(_p(a), a.size))


def parse_header(container: np.ndarray) -> dict:
    c = np.ascontiguousarray(container, dtype=np.uint8)
    h32 = c[:64].view(np.uint32)
    h64 = c[:64].view(np.uint64)
    return dict(magic=int(h32[0]), version=int(h32[1]), n_symbols=int(h64[1]),
                lane_symbols=int(h32[4]), len_quantum=int(h32[5]), n_units=int(h32[6]),
                prob_bits=int(h32[7]), payload_offset=int(h64[4]), payload_words=int(h64[5]),
                total_bytes=int(h64[6]), n_raw_units=int(h32[14]),
                max_coded_unit_words=int(h32[15]))


# --------------------------------------------------------------------------
# Independent pure-numpy restatements, used to cross-check the C code on small
# inputs (a second implementation of the same specification).

def split_numpy(bits: np.ndarray, s: int) -> Tuple[np.ndarray, np.ndarray]:
    """Closed form of cuda/kernels.cuh:120-155 with numpy integer ops."""
    v = bits.reshape(-1).astype(np.uint32)
    n = v.size
    sign = v >> 15
    mag = v & 0x7FFF
    rnd = ((mag >> (6 - s)) & 1) if s < 7 else np.zeros_like(mag)
    keep = ((mag >> (7 - s)) + rnd) & ((1 << (8 + s)) - 1)
    field = (sign << s) | (keep & ((1 << s) - 1))
    exp = (keep >> s).astype(np.uint8)
    per = 8 // (s + 1)
    pad = (-n) % per
    f = np.concatenate([field, np.zeros(pad, np.uint32)]).reshape(-1, per)
    shifts = np.array([7 - s - j * (s + 1) for j in range(per)], np.uint32)
    frac = np.bitwise_or.reduce(f << shifts, axis=1).astype(np.uint8)
    return exp, frac


def merge_numpy(exp: np.ndarray, frac: np.ndarray, s: int) -> np.ndarray:
    """cuda/kernels.cuh:197-216 without the NaN canonicalisation."""
    n = exp.size
    idx = np.arange(n, dtype=np.uint64)
    bit = idx * (s + 1)
    shift = (7 - s - (bit & 7)).astype(np.uint32)
    repr_ = frac.astype(np.uint32)[(bit >> 3).astype(np.int64)] >> shift
    fraction = (repr_ & ((1 << s) - 1)) << (7 - s)
    sign = (repr_ >> s) & 1
    return ((sign << 15) | (exp.astype(np.uint32) << 7) | fraction).astype(np.uint16)


def decode_python(container: np.ndarray, n: int) -> np.ndarray:
    """Pure-Python decoder of the NZR1 container (small inputs only)."""
    c = np.ascontiguousarray(container, dtype=np.uint8)
    h = parse_header(c)
    S, lenq, pb = h["lane_symbols"], h["len_quantum"], h["prob_bits"]
    U = 32 * S
    n_units = h["n_units"]
    freq = c[FREQ_OFFSET:FREQ_OFFSET + 512].view(np.uint16).astype(np.int64)
    cum = np.concatenate([[0], np.cumsum(freq)])
    slot_sym = np.repeat(np.arange(256), freq)
    offs = c[OFFSETS_OFFSET:OFFSETS_OFFSET + 4 * (n_units + 1)].view(np.uint32)
    pay = c[h["payload_offset"]:h["payload_offset"] + 2 * h["payload_words"]].view(np.uint16)
    out = np.zeros(n, np.uint8)
    for u in range(n_units):
        w0 = int(offs[u] & 0x7FFFFFFF)
        first = u * U
        count = min(U, n - first)
        if offs[u] >> 31:
            out[first:first + count] = pay[w0:w0 + (count + 1) // 2].view(np.uint8)[:count]
            continue
        lens = pay[w0:w0 + 16].view(np.uint8).astype(np.int64) * lenq
        p = w0 + 16
        for j in range(32):
            ws = pay[p:p + lens[j]]
            x = int(ws[0]) | (int(ws[1]) << 16)
            q = 2
            for i in range(S):
                slot = x & ((1 << pb) - 1)
                sy = int(slot_sym[slot])
                x = int(freq[sy]) * (x >> pb) + slot - int(cum[sy])
                if x < (1 << 16):
                    x = (x << 16) | int(ws[q])
                    q += 1
                e = first + (i >> 3) * 256 + j * 8 + (i & 7)
                if e < n:
                    out[e] = sy
            assert x == 1 << 16
            p += int(lens[j])
    return out


# --------------------------------------------------------------------------
# The reference's own split / merge kernels (GPU), compiled from the reference
# tree by `make -C oracle ref` into oracle/_ref/libnz_ref_kernels.so.  The tree is
# only present where the project is built; the library travels with the built
# files.  Used by the GPU parity tests to pin this oracle and the product's
# kernels to reference-run outputs.

_REF_SO = os.path.join(_HERE, "_ref", "libnz_ref_kernels.so")
REFERENCE_DIR = os.environ.get("NZ_REFERENCE_DIR", "/root/reference")
REF_GROUPS = (0, 1, 2, 4, 8, 16, 32, 1024)   # 0 = normalized=false; see ref_kernels.cu
_ref_lib = None


def build_ref() -> Optional[str]:
    """Compile the reference kernels when the reference tree is present; returns the
    library path, or None when neither the tree nor a built library exists."""
    kernels = os.path.join(REFERENCE_DIR, "cuda", "kernels.cuh")
    if os.path.exists(kernels):
        harness = os.path.join(_HERE, "ref_kernels.cu")
        stale = (not os.path.exists(_REF_SO)
                 or os.path.getmtime(_REF_SO) < max(os.path.getmtime(harness),
                                                    os.path.getmtime(kernels)))
        if stale:
            subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE_DIR={REFERENCE_DIR}"],
                           check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _REF_SO if os.path.exists(_REF_SO) else None


def ref_lib() -> Optional[ctypes.CDLL]:
    """The reference-kernel library (needs `import torch` first: it links libc10),
    or None when it has not been built."""
    global _ref_lib
    if _ref_lib is None and os.path.exists(_REF_SO):
        import torch  # noqa: F401  (loads libc10 / libtorch the harness links against)
        L = ctypes.CDLL(_REF_SO)
        vp = ctypes.c_void_p
        for fn in (L.nzref_split, L.nzref_merge):
            fn.argtypes = [ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, ctypes.c_size_t, vp]
            fn.restype = ctypes.c_int
        _ref_lib = L
    return _ref_lib


# --------------------------------------------------------------------------
# Operand order: a [rows, cols] matrix whose stream blocks of 256 elements are
# 4-row x 64-column patches (stream element ((g*cols/64 + kb)*4 + r)*64 + c is matrix
# element (4g + r, 64kb + c)).  The codec is applied to the permuted tensor.

def to_operand_order(bits: np.ndarray, rows: int, cols: int) -> np.ndarray:
    assert rows % 4 == 0 and cols % 64 == 0 and bits.size == rows * cols
    return np.ascontiguousarray(
        bits.reshape(rows // 4, 4, cols // 64, 64).transpose(0, 2, 1, 3)).reshape(-1)


def operand_lane_symbols_for(rows: int, cols: int, s: int) -> int:
    """The unit length the GPU library picks when the row count is known
    (nz_operand_lane_symbols_for): fewest decode steps in sequence for one work item per
    128-row tile and unit-long column segment, 148 at a time; the longer unit on a tie."""
    if rows == 0:
        return operand_lane_symbols(cols, s)
    if cols <= 0 or cols % 64 or rows % 4:
        return 0
    spr, tiles = cols // 64, (rows + 127) // 128
    best, best_cost = 0, 0
    for beta in range(16, min(48, spr) + 1):
        if spr % beta:
            continue
        cost = -(-(tiles * (spr // beta)) // 148) * (beta + 6)
        if not best or cost <= best_cost:
            best, best_cost = beta, cost
    return best * 8 if best else operand_lane_symbols(cols, s)


def from_operand_order(stream: np.ndarray, rows: int, cols: int) -> np.ndarray:
    assert rows % 4 == 0 and cols % 64 == 0 and stream.size == rows * cols
    return np.ascontiguousarray(
        stream.reshape(rows // 4, cols // 64, 4, 64).transpose(0, 2, 1, 3)).reshape(-1)


def operand_lane_symbols(cols: int, s: int) -> int:
    """The unit length (in lane symbols) for a matrix of `cols` columns in operand
    order: lane_symbols / 8 is the divisor of cols / 64 closest in ratio to the default,
    within a factor of two of it and between 16 and 128; 0 when there is none."""
    if cols <= 0 or cols % 64:
        return 0
    spr, want = cols // 64, default_lane_symbols(s) // 8
    best, best_cost = 0, 0.0
    for beta in range(16, min(128, spr) + 1):
        if spr % beta:
            continue
        ratio = beta / want if beta > want else want / beta
        if ratio > 2.0:
            continue
        if not best or ratio < best_cost:
            best, best_cost = beta, ratio
    return best * 8
