#!/usr/bin/env python
"""Writes tests/golden/ref_kernels.npz: outputs of the reference's own attention kernels (flash_attention,
attn_decode_gqa, attention_combine of kernels/40_attention.metal, run by the SIMT emulator behind
oracle/_ref/libplan_ref.so) on the seeded cases of tests/test_ref_kernels.py. The inputs are regenerated
from their seeds by the tests; only the fp16 outputs are stored. Run where the reference tree is present:
    python tests/golden/make_ref_kernel_golden.py"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref  # noqa: E402
from tests.test_ref_kernels import CASES, make_case, ref_forward  # noqa: E402


def main():
    assert ref.load() is not None, "build oracle/_ref first (make -C oracle ref)"
    out = {}
    for name in sorted(CASES):
        w, split, groups = make_case(name)
        O, (tiles, jobs, n_parts), _ = ref_forward(w, split, groups)
        out[name + "_O"] = O
        out[name + "_plan"] = np.array([len(tiles), len(jobs), n_parts], dtype=np.int32)
    path = os.path.join(ROOT, "tests", "golden", "ref_kernels.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
