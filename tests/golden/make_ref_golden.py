#!/usr/bin/env python
"""Writes tests/golden/ref_vectors.npz: input / output vectors produced by the reference's OWN code
(oracle/_ref/libplan_ref.so, built from the reference tree by `make -C oracle ref`), so that machines that
never see the reference tree still check the product against it (tests/test_ref_golden.py).
Run on a machine where the reference tree is present:  python tests/golden/make_ref_golden.py"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from espetero_b200 import workloads as wl  # noqa: E402
from oracle import ref  # noqa: E402
import oracle  # noqa: E402
from tests.test_planner import _trees  # noqa: E402


def main():
    assert ref.load() is not None, "build oracle/_ref first (make -C oracle ref)"
    rng = np.random.default_rng(0x5EF)
    out = {}
    # ---- plan_tiles / g4_plan_tiles
    n_plan = 40
    for i in range(n_plan):
        n = int(rng.integers(1, 12))
        trees = _trees([(int(rng.choice([0, 63, 64, 65, 512, 4096, 40000, int(rng.integers(0, 70000))])), int(rng.choice([1, 1, 7, 8, 9, 16, 100])))
                        for _ in range(n)])
        prm = np.array([int(rng.choice([1, 2, 4, 8])), int(rng.choice([0, 128, 512])), int(rng.choice([256, 64, 1024])), int(rng.choice([32, 128]))], dtype=np.int32)
        t, j, npart = ref.plan_tiles(trees, int(prm[0]), int(prm[1]), int(prm[2]), int(prm[3]))
        out[f"plan{i}_trees"], out[f"plan{i}_prm"], out[f"plan{i}_tiles"], out[f"plan{i}_jobs"] = trees, prm, t, j
        out[f"plan{i}_nparts"] = np.int32(npart)
    n_g4 = 30
    for i in range(n_g4):
        pm = [(int(rng.integers(0, 5000)), int(rng.integers(1, 40))) for _ in range(int(rng.integers(1, 6)))]
        trees = _trees(pm)
        pos = np.zeros((sum(m for _, m in pm), 4), dtype=np.int32)
        for tr in trees:
            b0, P, M = int(tr["base"]), int(tr["P"]), int(tr["M"])
            pos[b0:b0 + M, 0] = P + np.sort(rng.integers(0, M, size=M))
        prm = np.array([int(rng.choice([1, 2, 8, 32])), int(rng.choice([0, 256, 512])), int(rng.choice([8, 16])), int(rng.choice([0, 17, 512, 100000]))], dtype=np.int32)
        t, j, npart, rows = ref.g4_plan_tiles(trees, int(prm[0]), int(prm[1]), int(prm[2]), int(prm[3]), pos)
        out[f"g4_{i}_trees"], out[f"g4_{i}_pos"], out[f"g4_{i}_prm"], out[f"g4_{i}_tiles"], out[f"g4_{i}_jobs"] = trees, pos, prm, t, j
        out[f"g4_{i}_np_rows"] = np.array([npart, rows], dtype=np.int32)
    # ---- target_blocks
    n_tb = 60
    tb_in, tb_out = [], []
    for i in range(n_tb):
        bt, n = int(rng.choice([16, 64])), 40
        pool = ref.Pool(n, bt)
        P = int(rng.integers(0, 6 * bt))
        parent = [pool.alloc() for _ in range((P + bt - 1) // bt)]
        shared = [int(rng.random() < 0.3) for _ in parent]
        for blk, s in zip(parent, shared):
            if s:
                pool.retain(blk)
        w0 = int(rng.integers(max(0, P - 1), P + 1)) if P else 0
        end = w0 + int(rng.integers(1, 3 * bt))
        in_place = int(rng.integers(0, 2))
        nb = pool.new_blocks(parent, P, w0, end, in_place)
        blocks, cow = pool.target_blocks(parent, P, w0, end, in_place)
        tb_in.append(np.array([bt, n, P, w0, end, in_place] + shared + [-1] * (8 - len(shared)), dtype=np.int32))
        tb_out.append(np.array([nb, len(blocks)] + blocks + [-1] * (16 - len(blocks)) + [len(cow)] + [x for pr in cow for x in pr] + [-1] * (8 - 2 * len(cow))
                               + pool.refs(), dtype=np.int32))
        pool.close()
    out["tb_in"], out["tb_out"] = np.stack(tb_in), np.stack(tb_out)
    # ---- leaf hosting + row records
    n_tr = 40
    for i in range(n_tr):
        Tr = int(rng.integers(1, 6))
        root = rng.integers(0, 50, Tr).astype(np.int32)
        leaves = []
        for _ in range(int(rng.integers(0, 7))):
            if leaves and rng.random() < 0.5:
                src = leaves[int(rng.integers(0, len(leaves)))]
                leaf = src[:int(rng.integers(1, len(src) + 1))] + [int(x) for x in rng.integers(0, 4, int(rng.integers(0, 3)))]
            else:
                leaf = [int(x) for x in rng.integers(0, 4, int(rng.integers(1, 5)))]
            leaves.append(leaf)
        base, pnext, sr = int(rng.integers(0, 100)), int(rng.integers(0, 1000)), int(rng.integers(0, 2))
        r = ref.tree_rows(root, leaves, None, False, bool(sr), base, pnext)
        offs = np.zeros(len(leaves) + 1, dtype=np.int32)
        offs[1:] = np.cumsum([len(x) for x in leaves])
        out[f"tr{i}_root"], out[f"tr{i}_offs"] = root, offs
        out[f"tr{i}_toks"] = np.array([t for x in leaves for t in x], dtype=np.int32)
        out[f"tr{i}_prm"] = np.array([base, pnext, sr], dtype=np.int32)
        out[f"tr{i}_host"], out[f"tr{i}_off"], out[f"tr{i}_tok"], out[f"tr{i}_pos"], out[f"tr{i}_desc"] = r["host"], r["off"], r["tok"], r["pos"], r["desc"]
        out[f"tr{i}_readout"], out[f"tr{i}_next"] = r["readout"], np.int32(r["next_root"])
    # ---- attention_combine of the reference (HD 256, fp16 out, gated): one case
    H, Hkv, HD, G = 2, 1, 256, 2
    jobs = np.array([(0, 3, 0, 9), (8, 8, 9, 2)], dtype=wl.COMBINE_DT)
    parts = rng.standard_normal(11 * Hkv * 8 * G * (HD + 2)).astype(np.float32)
    rec = parts.reshape(-1, HD + 2)
    rec[:, HD], rec[:, HD + 1] = rng.uniform(-5, 5, len(rec)), rng.uniform(0.5, 40, len(rec))
    rec[5, HD], rec[5, HD + 1], rec[5, :HD] = -np.inf, 0.0, 0.0
    X = rng.standard_normal((16, 2 * H * HD)).astype(np.float32)
    p = oracle.Params(H, Hkv, H * HD, Hkv * HD, 2 * H * HD, 16, 0)
    O = np.zeros((16, H * HD), dtype=np.uint16)
    ref.load().ref_attention_combine(C.c_void_p(parts.ctypes.data), C.c_void_p(X.ctypes.data), C.c_void_p(O.ctypes.data), C.byref(p),
                                     C.c_void_p(jobs.ctypes.data), len(jobs))
    out["cmb_parts"], out["cmb_X"], out["cmb_jobs"], out["cmb_O"] = parts.astype(np.float16).astype(np.float32), X.astype(np.float16).astype(np.float32), jobs, None
    # (inputs are stored rounded to fp16 to keep the file small; recompute O from the stored inputs)
    parts, X = out["cmb_parts"], out["cmb_X"]
    rec = parts.reshape(-1, HD + 2)
    rec[5, HD] = -np.inf
    O[:] = 0
    ref.load().ref_attention_combine(C.c_void_p(parts.ctypes.data), C.c_void_p(X.ctypes.data), C.c_void_p(O.ctypes.data), C.byref(p),
                                     C.c_void_p(jobs.ctypes.data), len(jobs))
    out["cmb_parts"], out["cmb_X"], out["cmb_O"] = parts.astype(np.float16), X.astype(np.float16), O
    # ---- E4M3: the grid ds4_round_e4m3 lands on, for a seeded sample
    xs = np.concatenate([rng.standard_normal(2000) * rng.choice([1e-3, 0.05, 1.0, 30.0, 400.0], 2000),
                         np.array([0.0, 448.0, 449.0, 1e9, -1e9, 2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10, 0.0146484375])]).astype(np.float32)
    out["e4m3_x"], out["e4m3_q"] = xs, np.array([ref.round_e4m3(float(x)) for x in xs], dtype=np.float32)
    out["counts"] = np.array([n_plan, n_g4, n_tb, n_tr], dtype=np.int32)
    path = os.path.join(ROOT, "tests", "golden", "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
