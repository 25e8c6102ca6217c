"""Generates tests/golden/config2_layer0.json from the CPU oracle.

Run from the repository root:  python tests/golden/make_config2_layer0.py

Layer set 0 of configuration 2 of the benchmark list: matrix j of layer l is
(torch.randn(shape, generator=CPU generator seeded 1000 + 7 l + j) * 0.02).to(bfloat16)
with shapes 4 x 4096x4096, 2 x 11008x4096, 1 x 4096x11008.  For each of the seven
matrices the file records CRC-32s of the input bits and, at precision 7 with the
default unit length, of the oracle's container and fraction stream, plus the stored
size.  bench.py compresses the same matrices on the GPU and compares (zlib.crc32 is
the same polynomial), so the benchmark's workload is pinned to the oracle without
the benchmark's product path touching it.
"""
import json
import os
import sys
import zlib

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

SHAPES = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]


def main():
    out = {"layer": 0, "precision": 7, "lane_symbols": O.default_lane_symbols(7), "matrices": []}
    for j, shape in enumerate(SHAPES):
        g = torch.Generator().manual_seed(1000 + j)
        w = (torch.randn(shape, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        bits = w.view(torch.int16).numpy().view(np.uint16).reshape(-1)
        cont, frac = O.compress_bf16(bits, 7)
        assert zlib.crc32(bits.tobytes()) == O.crc32(bits)
        out["matrices"].append({
            "shape": list(shape), "seed": 1000 + j,
            "input_crc32": hex(zlib.crc32(bits.tobytes())),
            "container_crc32": hex(zlib.crc32(cont.tobytes())),
            "frac_crc32": hex(zlib.crc32(frac.tobytes())),
            "container_bytes": int(cont.size), "frac_bytes": int(frac.size)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config2_layer0.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", path)


if __name__ == "__main__":
    main()
