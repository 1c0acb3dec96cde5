"""Generates the golden fixtures of tests/golden/ from the float64 oracle.

The reference holds no golden vectors for its attention path (its kernels run only on Metal),
so these fixtures pin the ORACLE, not the reference: a change to oracle/ or to the workload
generator that alters any number shows up as a diff against the committed .npz. They also give
the GPU tests a second, file-based expectation that does not depend on the oracle library being
built on the GPU box.

    python tests/golden/make_golden.py          # rewrites tests/golden/*.npz
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from espetero_b200 import workloads as wl  # noqa: E402

# name -> workload builder; small enough that a fixture is a few tens of KB
CASES = {
    "decode_f16_c1like": lambda: wl.make_pass("g_c1", 0xA1, [(1024, 1)], 8, 2, 128, 16, wl.F16),
    "decode_bf16_batch": lambda: wl.make_pass("g_c2", 0xA2, [(512, 1), (777, 1), (33, 1), (0, 1)], 16, 2, 128, 16, wl.BF16),
    "decode_fp8_hd256": lambda: wl.make_pass("g_c5", 0xA5, [(2048, 1)], 8, 2, 256, 16, wl.BF16, wl.E4M3),
    "verify_tree16": lambda: wl.make_pass("g_c4", 0xA4, [(256, 16), (100, 16)], 16, 2, 128, 16, wl.BF16, mask="tree"),
    "prefill_causal": lambda: wl.make_pass("g_c3", 0xA3, [(0, 150), (0, 129)], 8, 2, 128, 16, wl.BF16),
    "forest_gate_f16": lambda: wl.make_pass("g_forest", 0xA6, [(40, 20), (0, 9)], 8, 2, 128, 16, wl.F16, mask="forest", gate=True),
    "window_ring_bidi": lambda: wl.make_window_pass("g_win", 0xA7, [(300, 24), (90, 10)], 8, 2, 256, 16, wl.BF16, 128, ring=24,
                                                    images={0: (4, 15)}, scale=1.0 / 16),
}


def prep_case():
    """Inputs of the attn_prep fixture: the gate-interleaved 256-dim layout of kernels/40_attention.metal:23-102."""
    rng = np.random.default_rng(0xA8)
    H, Hkv, HD, rot_half, rows = 4, 2, 256, 32, 6
    k_off = 2 * H * HD
    v_off = k_off + Hkv * HD
    ld = v_off + Hkv * HD
    X = rng.standard_normal((rows, ld)).astype(np.float32)
    qn, kn = rng.uniform(0.5, 1.5, HD).astype(np.float32), rng.uniform(0.5, 1.5, HD).astype(np.float32)
    inv_freq = (1e6 ** (-np.arange(rot_half) / rot_half)).astype(np.float32)
    sel = (np.arange(rot_half) * 3 // rot_half).astype(np.int32)
    pos = rng.integers(0, 100000, size=(rows, 4)).astype(np.int32)
    pp = oracle.PrepParams(H, Hkv, ld, 0, 2 * HD, k_off, v_off, H * HD, Hkv * HD, rot_half, 1e-6, 1.0, 16, 0, 0)
    return dict(H=H, Hkv=Hkv, HD=HD, rows=rows, X=X, qn_w=qn, kn_w=kn, inv_freq=inv_freq, sel=sel, pos=pos, pp=pp)


def build_prep():
    c = prep_case()
    Q, K, V = oracle.attn_prep_f64(c["X"], c["qn_w"], c["kn_w"], c["pos"], c["inv_freq"], c["sel"], c["rows"], c["HD"], c["pp"])
    digest = np.array([float(np.abs(c["X"]).sum()), float(c["pos"].sum())])
    return dict(Q=Q, K=K, V=V, input_digest=digest)


def build(name):
    w = CASES[name]()
    O, lse, Oabs = oracle.attention_f64(w, with_abs=True, threads=1)
    sel = np.random.default_rng(1).choice(w.n_rows, size=min(w.n_rows, 8), replace=False)
    sel.sort()
    # checksum of the generated inputs, so that a change of the generator is told apart from a change of the oracle
    digest = np.array([int(w.Q.astype(np.uint64).sum()), int(w.kv.astype(np.uint64).sum()), int(w.blocks.astype(np.int64).sum())],
                      dtype=np.uint64)
    return dict(rows=sel.astype(np.int32), O=O[sel].astype(np.float64), lse=lse[sel].astype(np.float64), Oabs=Oabs[sel].astype(np.float32),
                input_digest=digest)


if __name__ == "__main__":
    for name in CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **build(name))
        print("wrote", name)
    np.savez_compressed(os.path.join(HERE, "attn_prep_gated256.npz"), **build_prep())
    print("wrote attn_prep_gated256")
