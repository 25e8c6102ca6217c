"""Generates tests/golden/reference_pin.json from a run of the REFERENCE's own
split / merge kernels on a GPU (oracle/_ref/libnz_ref_kernels.so, built from the
reference tree by `make -C oracle ref`).

Run on a B200 from the repository root:
    python tests/golden/make_reference_pin.py [output.json]

Input: configuration 1 of the benchmark list (torch.manual_seed(0) on the CPU
generator, (randn(4096, 4096) * 0.02).to(bfloat16)) and all 65 536 bf16 patterns.
For every precision the file records CRC-32s of the reference kernels' exponent
stream, packed fractions and merged round trip.  Nothing in it comes from this
project's oracle or kernels; tests/test_gpu_reference_pin.py and
tests/test_oracle.py compare against it.
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402  (CRC-32 helper and library loader only)
from tests import test_gpu_reference_pin as T  # noqa: E402


def main():
    assert O.ref_lib() is not None, "build oracle/_ref first: make -C oracle ref"
    out = {"source": "kernel_aligned_split / kernel_aligned_merge of the reference, run on "
                     + torch.cuda.get_device_name(0),
           "precision": {}, "all_patterns": {}}
    bits = T.config1_bits()
    out["input_crc32"] = hex(O.crc32(bits))
    allp = np.arange(65536, dtype=np.uint16)
    for s in (0, 1, 3, 7):
        e, f, _ = T.ref_split(bits, s)
        rt = T.ref_merge(e, f, s)
        out["precision"][str(s)] = {"exp_crc32": hex(O.crc32(e)), "frac_crc32": hex(O.crc32(f)),
                                    "roundtrip_crc32": hex(O.crc32(rt))}
        e, f, _ = T.ref_split(allp, s)
        rt = T.ref_merge(e, f, s)
        out["all_patterns"][str(s)] = {
            "exp_crc32": hex(O.crc32(e)), "frac_crc32": hex(O.crc32(f)),
            "roundtrip_crc32": hex(O.crc32(rt)),
            "roundtrip_identical_patterns": int((rt == allp).sum())}
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(
        os.path.dirname(os.path.abspath(__file__)), "reference_pin.json")
    with open(path, "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)
    print("wrote", path)


if __name__ == "__main__":
    main()
