"""Golden fixtures (tests/golden/*.npz, written by tests/golden/make_golden.py from the float64
oracle). On CPU: the oracle and the input generator still reproduce them bit for bit. On the
GPU: the CUDA path meets the stated tolerance against the committed numbers."""
import os

import numpy as np
import pytest

from espetero_b200 import workloads as wl
from tests import util
from tests.golden.make_golden import CASES, build, build_prep, prep_case

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


def test_prep_oracle_reproduces_fixture():
    want = np.load(os.path.join(GOLDEN, "attn_prep_gated256.npz"))
    got = build_prep()
    assert np.array_equal(got["input_digest"], want["input_digest"]), "the input generator changed"
    for k in ("Q", "K", "V"):
        assert np.array_equal(got[k], want[k]), k


@pytest.mark.gpu
def test_cuda_prep_meets_fixture():
    import torch
    from espetero_b200 import capi, host
    want = np.load(os.path.join(GOLDEN, "attn_prep_gated256.npz"))
    c = prep_case()
    op = host.AttnOp(c["H"], c["Hkv"], c["HD"], 16, wl.BF16, wl.BF16, 1.0)
    try:
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(op.device)
        o = c["pp"]
        pp = capi.PrepParams(o.H, o.Hkv, o.ld, o.q_off, o.q_stride, o.k_off, o.v_off, o.q_ld, o.kv_ld, o.rot_half, o.eps, o.qscale, o.bt, 0, 0)
        Q = torch.zeros((c["rows"], pp.q_ld), dtype=torch.int16, device=op.device)
        Kb = torch.zeros((c["rows"], pp.kv_ld), dtype=torch.int16, device=op.device)
        Vb = torch.zeros_like(Kb)
        op.attn_prep(t(c["X"]), t(c["qn_w"]), t(c["kn_w"]), t(c["pos"]), t(c["inv_freq"]), t(c["sel"]), Q, Kb, Vb, pp)
        torch.cuda.synchronize()
        for got_t, ref in ((Q, want["Q"]), (Kb, want["K"]), (Vb, want["V"])):
            got = wl.from_bits16(got_t.cpu().numpy().view(np.uint16), wl.BF16).astype(np.float64)
            # one rounding to bf16 (half an ulp = 2^-9 relative) plus fp32 arithmetic on the head's scale
            assert (np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-5 * np.abs(ref).max()).all()
    finally:
        op.close()
