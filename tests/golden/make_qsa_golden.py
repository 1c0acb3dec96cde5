#!/usr/bin/env python
"""Writes tests/golden/qsa.npz: what the reference's own sparse-attention pipeline (qsa_plan, plan_tiles, qsa_select,
qsa_tiles, flash_attention_qsa, attention_combine - compiled from the reference tree into oracle/_ref/libplan_ref.so, the
kernels run by the SIMT emulator) produces on the seeded cases of tests/test_qsa.py. Inputs are regenerated from their
seeds by the tests. Run where the reference tree is present:  python tests/golden/make_qsa_golden.py"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests.test_qsa import reference_pipeline  # noqa: E402


def main():
    out = {}
    for name in ("mixed", "decode"):
        r = reference_pipeline(name)
        out[name + "_counts"] = np.array(r["plan"]["counts"], dtype=np.int32)
        out[name + "_rinfo"] = r["plan"]["rinfo"]
        out[name + "_sel"], out[name + "_tcount"] = r["sel"], r["tcount"]
        tl = r["tlist"].copy()
        for i, n in enumerate(r["tcount"]):
            tl[i, n:] = 0
        out[name + "_tlist"], out[name + "_O"] = tl, r["O"]
    path = os.path.join(ROOT, "tests", "golden", "qsa.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
