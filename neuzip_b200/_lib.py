"""ctypes loader of ``libneuzip_b200.so`` (the C-ABI library declared in
``include/neuzip_b200.h``).

There is no CPU fallback: if the shared library is missing or the current
device is not a B200-class GPU, the calls raise.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_SO_PATH = os.path.join(_PKG_DIR, "libneuzip_b200.so")
_CSRC = os.path.join(_PKG_DIR, "csrc")

NZ_OK = 0
NZ_ITEM_INPUTS_STABLE = 0x1
NZ_E_ARG, NZ_E_CUDA, NZ_E_CAPACITY, NZ_E_FORMAT, NZ_E_DEVICE = -1, -2, -3, -4, -5
STATUS_BITS = {
    0x1: "bad header",
    0x2: "bad unit offsets",
    0x4: "bad lane lengths",
    0x8: "bad final state",
    0x10: "bulk-copy wait timed out",
    0x20: "gather list names a unit that does not exist",
}

# name -> (restype, argtypes); mirrors include/neuzip_b200.h one to one
_vp, _u64, _u32, _int = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
SIGNATURES = {
    "nz_version": (_int, []),
    "nz_last_error": (ctypes.c_char_p, []),
    "nz_device_check": (_int, []),
    "nz_frac_bytes": (_u64, [_u64, _int]),
    "nz_default_lane_symbols": (_u32, [_int]),
    "nz_container_bound": (_u64, [_u64, _u32]),
    "nz_encode_scratch_bytes": (_u64, [_u64, _u32]),
    "nz_compress_scratch_bytes": (_u64, [_u64, _u32]),
    "nz_split_bf16": (_int, [_vp, _u64, _int, _vp, _vp, _vp]),
    "nz_merge_bf16": (_int, [_vp, _vp, _u64, _int, _int, _vp, _vp]),
    "nz_normalizer_bytes": (_u64, [_u64, _u32]),
    "nz_normalize_bf16": (_int, [_vp, _u64, _u32, _vp, _vp, _vp]),
    "nz_denormalize_bf16": (_int, [_vp, _u64, _u32, _vp, _vp]),
    "nz_histogram_u8": (_int, [_vp, _u64, _vp, _vp]),
    "nz_encode_exponents": (_int, [_vp, _u64, _u32, _vp, _u64, _vp, _u64, _vp]),
    "nz_static_scratch_bytes": (_u64, []),
    "nz_encode_exponents_static_scratch": (_int, [_vp, _u64, _u32, _vp, _u64, _vp]),
    "nz_container_bytes": (_int, [_vp, ctypes.POINTER(_u64), ctypes.POINTER(_u32), _vp]),
    "nz_container_header_async": (_int, [_vp, _vp, _vp]),
    "nz_parse_header": (_int, [_vp, ctypes.POINTER(_u64), ctypes.POINTER(_u32)]),
    "nz_decode_exponents": (_int, [_vp, _u64, _u64, _u32, _u32, _vp, _vp, _vp]),
    "nz_compress_bf16": (_int, [_vp, _u64, _int, _u32, _vp, _vp, _u64, _vp, _u64, _vp]),
    "nz_decompress_bf16": (_int, [_vp, _u64, _vp, _u64, _int, _u32, _u32, _int, _vp, _vp, _vp]),
}



class DecompressItem(ctypes.Structure):
    """struct nz_decompress_item"""
    _fields_ = [("container", _vp), ("container_bytes", _u64), ("frac_in", _vp), ("n", _u64),
                ("max_unit_words", _u32), ("flags", _u32), ("out_bf16", _vp),
                ("operand_cols", _u64), ("lane_symbols", _u32), ("normalizer_group", _u32),
                ("normalizers", _vp)]


_f32 = ctypes.c_float
SIGNATURES["nz_adamw_bf16"] = (_int, [_vp, _vp, _vp, _vp, _u64, _int, _f32, _f32, _f32, _f32, _f32,
                                       _u32, _f32, _vp])
SIGNATURES["nz_decompress_bf16_units"] = (
    _int, [_vp, _u64, _vp, _u64, _int, _u32, _u32, _int, _vp, _u32, _vp, _vp, _vp])
SIGNATURES["nz_gather_scratch_bytes"] = (_u64, [_u32, _u64, _u32])
SIGNATURES["nz_gather_rows_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _int, _u32, _u32, _int, _u64, _vp, _u32, _vp, _vp, _u64, _vp, _vp])
SIGNATURES["nz_gather_rows_normalized_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _int, _u32, _u32, _int, _u64, _vp, _u32, _vp, _u32, _vp, _vp, _u64, _vp,
           _vp])
SIGNATURES["nz_linear_vec_scratch_bytes"] = (_u64, [_u64, _u64, _u32])
SIGNATURES["nz_linear_vec_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _int, _u32, _u32, _int, _u64, _vp, _vp, _vp, _vp, _u64, _vp, _vp])
SIGNATURES["nz_decompress_bf16_batch"] = (
    _int, [ctypes.POINTER(DecompressItem), _u32, _int, _u32, _int, _vp, _vp])

SIGNATURES["nz_operand_lane_symbols"] = (_u32, [_u64, _int])
SIGNATURES["nz_operand_lane_symbols_for"] = (_u32, [_u64, _u64, _int])
SIGNATURES["nz_compress_operand_scratch_bytes"] = (_u64, [_u64, _u64, _u32])
SIGNATURES["nz_compress_bf16_operand"] = (
    _int, [_vp, _u64, _u64, _int, _u32, _vp, _vp, _u64, _vp, _u64, _vp])
SIGNATURES["nz_decompress_bf16_operand"] = (
    _int, [_vp, _u64, _vp, _u64, _u64, _int, _u32, _u32, _int, _vp, _vp, _vp])
SIGNATURES["nz_linear_workspace_bytes"] = (_u64, [_u64, _u64, _u32, _u64])
SIGNATURES["nz_linear_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _u64, _int, _u32, _u32, _int, _vp, _u64, _vp, _vp, _vp, _u64, _vp,
           _vp])

SIGNATURES["nz_adamw_compressed_scratch_bytes"] = (_u64, [_u64, _u32])
SIGNATURES["nz_adamw_compressed_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _u64, _int, _u32, _u32, _int, _vp, _vp, _vp, _f32, _f32, _f32, _f32,
           _f32, _u32, _f32, _vp, _vp, _u64, _vp, _u64, _vp, _vp])



class PeerGroup(ctypes.Structure):
    """struct nz_peer_group"""
    _fields_ = [("world", _u32), ("rank", _u32), ("workspace", _vp * 8), ("arrivals", _vp * 8),
                ("workspace_bytes", _u64)]


SIGNATURES["nz_linear_allreduce_workspace_bytes"] = (_u64, [_u64, _u64, _u32, _u64, _u32])
SIGNATURES["nz_linear_allreduce_bf16"] = (
    _int, [_vp, _u64, _vp, _u64, _u64, _int, _u32, _u32, _int, _vp, _u64, _vp, _vp,
           ctypes.POINTER(PeerGroup), _u32, ctypes.POINTER(_u32), _vp, _vp])
SIGNATURES["nz_peer_alloc"] = (_int, [_u64, ctypes.POINTER(_vp), _vp])
SIGNATURES["nz_peer_open"] = (_int, [_vp, ctypes.POINTER(_vp)])
SIGNATURES["nz_peer_close"] = (_int, [_vp])
SIGNATURES["nz_peer_free"] = (_int, [_vp])

_lock = threading.Lock()
_lib = None


def build(verbose: bool = False) -> str:
    """Compile the CUDA sources for sm_100a with the Makefile in ``csrc``."""
    proc = subprocess.run(["make", "-C", _CSRC, "-j4"], stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        print(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("building libneuzip_b200.so failed")
    return _SO_PATH


def library_path() -> str:
    return _SO_PATH


def load() -> ctypes.CDLL:
    """Load the library (once) and attach the prototypes."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_SO_PATH):
                raise ImportError(
                    f"{_SO_PATH} is not built; run `python -c 'import __graft_entry__ as g; "
                    "g.build()'` or `make -C neuzip_b200/csrc`. There is no CPU fallback.")
            lib = ctypes.CDLL(_SO_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


class NeuzipError(RuntimeError):
    pass


def check(rc: int) -> None:
    """Turn a status code of the library into a Python exception."""
    if rc == NZ_OK:
        return
    msg = load().nz_last_error().decode("utf-8", "replace")
    if rc == NZ_E_ARG:
        raise ValueError(msg)
    raise NeuzipError(f"neuzip_b200 error {rc}: {msg}")


def describe_status(word: int) -> str:
    return ", ".join(txt for bit, txt in STATUS_BITS.items() if word & bit) or "ok"
