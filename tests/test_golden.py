"""Golden fixtures (tests/golden/*.npz, written by tests/golden/make_golden.py from the float64
oracle). On CPU: the oracle and the input generator still reproduce them bit for bit. On the
GPU: the CUDA path meets the stated tolerance against the committed numbers."""
import os

import numpy as np
import pytest

from espetero_b200 import workloads as wl
from tests import util
from tests.golden.make_golden import CASES, build

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_fixture(name):
    want = np.load(os.path.join(GOLDEN, name + ".npz"))
    got = build(name)
    assert np.array_equal(got["input_digest"], want["input_digest"]), "the workload generator changed"
    assert np.array_equal(got["rows"], want["rows"])
    assert np.array_equal(got["O"], want["O"]) and np.array_equal(got["lse"], want["lse"])


TILE_ROWS = {"verify_tree16": 16, "prefill_causal": 128}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_path_meets_fixture(name):
    from espetero_b200 import host
    want = np.load(os.path.join(GOLDEN, name + ".npz"))
    w = CASES[name]()
    O, lse, parts, plan, kernel = host.run_pass(w, tile_rows=TILE_ROWS.get(name, 8))
    rows = want["rows"]
    util.check_output(O, want["O"], w, rows=rows, ref_abs=want["Oabs"].astype(np.float64), what=f"{name}/{kernel}")
    fin = np.isfinite(want["lse"])
    assert np.abs(lse[rows][fin] - want["lse"][fin]).max() < 2e-3
