"""The C-ABI library loads without a GPU and exports exactly the symbols that
include/neuzip_b200.h declares; the size helpers agree with the oracle."""
import ctypes
import os
import re

import pytest

from neuzip_b200 import _lib
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "neuzip_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nz_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.library_path())
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_text():
    L = _lib.load()
    assert L.nz_version() >= 100
    assert isinstance(L.nz_last_error(), bytes)


@pytest.mark.parametrize("s", (0, 1, 3, 7))
def test_size_helpers_match_oracle(s):
    L = _lib.load()
    for n in (0, 1, 7, 8, 1000, 4096 * 4096, 4096 * 11008):
        assert L.nz_frac_bytes(n, s) == O.frac_bytes(n, s)
        S = L.nz_default_lane_symbols(s)
        assert S == O.default_lane_symbols(s)
        assert L.nz_container_bound(n, S) == O.container_bound(n, S)
        assert L.nz_encode_scratch_bytes(n, S) > 0
        # the whole-tensor compressor keeps no exponent stream: unit slots and tables only
        assert 0 < L.nz_compress_scratch_bytes(n, S) <= L.nz_encode_scratch_bytes(n, S) + 32 * (n // (32 * S) + 1)
    assert L.nz_frac_bytes(10, 5) == 0
    assert L.nz_default_lane_symbols(2) == 0
    assert L.nz_container_bound(10, 12) == 0


@pytest.mark.parametrize("s", (0, 1, 3, 7))
def test_operand_unit_length_rule_matches_the_oracle(s):
    """The unit length of operand-order matrices is part of the stored format's geometry: the
    library's choice (a host function) and the oracle's restatement must agree, with and without
    a known row count; spot values for the Llama shapes at precision 7."""
    L = _lib.load()
    for rows in (0, 4, 128, 2048, 4096, 5504, 8192, 11008, 28672, 32000):
        for cols in (64, 100, 512, 1024, 2048, 4096, 5504, 6144, 8192, 11008, 14336, 28672):
            assert L.nz_operand_lane_symbols_for(rows, cols, s) == O.operand_lane_symbols_for(rows, cols, s)
            assert L.nz_operand_lane_symbols(cols, s) == O.operand_lane_symbols(cols, s)
    if s == 7:
        want = {(4096, 4096): 128, (11008, 4096): 128, (4096, 11008): 344, (8192, 8192): 256,
                (8192, 28672): 224, (2048, 2048): 128, (2048, 5504): 344}
        for (rows, cols), S in want.items():
            assert L.nz_operand_lane_symbols_for(rows, cols, s) == S, (rows, cols)
    assert L.nz_operand_lane_symbols_for(6, 4096, s) == 0          # rows not a multiple of 4


def test_argument_validation_needs_no_gpu():
    L = _lib.load()
    assert L.nz_split_bf16(0, 16, 4, 0, 0, 0) == _lib.NZ_E_ARG
    assert b"precision" in L.nz_last_error()
    assert L.nz_decompress_bf16(0, 0, 0, 16, 7, 100, 0, 0, 0, 0, 0) == _lib.NZ_E_ARG
    with pytest.raises(ValueError):
        _lib.check(L.nz_compress_bf16(0, 16, 9, 256, 0, 0, 0, 0, 0, 0))


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "neuzip_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(base, f)).read()
                assert "oracle" not in src.replace("oracle/nz_oracle.c", "").replace(
                    "CPU oracle", "").replace("the oracle's", "").replace("nz_oracle", ""), f
