"""One compress + decompress of a single synthetic bf16 matrix through the
C-ABI library: the small, self-checking case to put under a profiler.

    python -m neuzip_b200.profile_case --precision 7 --rows 4096 --cols 11008

Every kernel of the codec launches at least once (split, histogram, table
normalisation, rANS encode, offset scan, compaction, fused decode+merge, and the
stand-alone merge).  Exits non-zero if the lossless round trip is not bit exact
or the decode status word is set.
"""
from __future__ import annotations

import argparse
import ctypes
import sys

import torch

from . import _lib


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--precision", type=int, default=7, choices=(0, 1, 3, 7))
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=11008)
    ap.add_argument("--lane-symbols", type=int, default=0)
    ap.add_argument("--repeat", type=int, default=3, help="decode launches")
    ap.add_argument("--seed", type=int, default=1)
    args = ap.parse_args(argv)

    L = _lib.load()
    _lib.check(L.nz_device_check())
    s = args.precision
    S = args.lane_symbols or int(L.nz_default_lane_symbols(s))
    n = args.rows * args.cols
    gen = torch.Generator(device="cuda").manual_seed(args.seed)
    x = (torch.randn(n, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream

    cap = int(L.nz_container_bound(n, S))
    cont = torch.empty(cap, dtype=torch.uint8, device="cuda")
    frac = torch.empty(int(L.nz_frac_bytes(n, s)), dtype=torch.uint8, device="cuda")
    sb = int(L.nz_compress_scratch_bytes(n, S))
    scratch = torch.empty(sb, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_compress_bf16(x.data_ptr(), n, s, S, frac.data_ptr(), cont.data_ptr(), cap,
                                  scratch.data_ptr(), sb, st))
    total, mw = ctypes.c_uint64(0), ctypes.c_uint32(0)
    _lib.check(L.nz_container_bytes(cont.data_ptr(), total, mw, st))

    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(args.repeat):
        _lib.check(L.nz_decompress_bf16(cont.data_ptr(), total.value, frac.data_ptr(), n, s, S,
                                        mw.value, 1, out.data_ptr(), status.data_ptr(), st))
    # stand-alone split / merge (the exponent stream through global memory)
    exp = torch.empty(n, dtype=torch.uint8, device="cuda")
    _lib.check(L.nz_split_bf16(x.data_ptr(), n, s, exp.data_ptr(), frac.data_ptr(), st))
    out2 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    _lib.check(L.nz_merge_bf16(exp.data_ptr(), frac.data_ptr(), n, s, 1, out2.data_ptr(), st))
    torch.cuda.synchronize()

    ok = int(status.item()) == 0 and torch.equal(out.view(torch.int16), out2.view(torch.int16))
    if s == 7:
        ok = ok and torch.equal(out.view(torch.int16), x.view(torch.int16))
    stored = total.value + frac.numel()
    print(f"precision={s} lane_symbols={S} elements={n} container={total.value} fractions={frac.numel()} "
          f"ratio={stored / (2 * n):.5f} algorithmic_bytes={2 * n + stored} ok={ok}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
