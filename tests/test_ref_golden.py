"""The product's host functions and the oracle's restatements against vectors produced by the reference's
own code (tests/golden/ref_vectors.npz, written by tests/golden/make_ref_golden.py from
oracle/_ref/libplan_ref.so): plan_tiles, g4_plan_tiles with its window branch, target_blocks /
target_new_blocks, leaf hosting and row records, attention_combine, the E4M3 grid. Runs everywhere: no
reference tree and no GPU needed. The GPU test at the end runs the CUDA combine kernel on the same case."""
import ctypes as C
import os

import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from tests.test_forest_host import Pool, _tree_rows

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_vectors.npz"))
N_PLAN, N_G4, N_TB, N_TR = (int(x) for x in G["counts"])


def test_planners_reproduce_the_reference_vectors(oracle_lib):
    for i in range(N_PLAN):
        trees, (Hkv, split, groups, min_chunk) = G[f"plan{i}_trees"], (int(x) for x in G[f"plan{i}_prm"])
        got = host.plan_tiles(trees, Hkv, capi.ESP_PLAN_REFERENCE, split, min_chunk, groups, 8)
        assert got.n_parts == int(G[f"plan{i}_nparts"]) and got.tiles.tobytes() == G[f"plan{i}_tiles"].tobytes(), i
        assert got.jobs.tobytes() == G[f"plan{i}_jobs"].tobytes(), i
        t, j, n = oracle_lib.plan_tiles(trees, Hkv, split, groups, min_chunk, 8)
        assert t.tobytes() == G[f"plan{i}_tiles"].tobytes() and j.tobytes() == G[f"plan{i}_jobs"].tobytes(), i
    for i in range(N_G4):
        trees, pos, (groups, split, rows, window) = G[f"g4_{i}_trees"], G[f"g4_{i}_pos"], (int(x) for x in G[f"g4_{i}_prm"])
        got = host.plan_window(trees, groups, split, rows, window, pos)
        assert [got.n_parts, got.tile_rows] == list(G[f"g4_{i}_np_rows"]), i
        assert got.tiles.tobytes() == G[f"g4_{i}_tiles"].tobytes() and got.jobs.tobytes() == G[f"g4_{i}_jobs"].tobytes(), i


def test_target_blocks_reproduce_the_reference_vectors():
    for i in range(N_TB):
        row, want = [int(x) for x in G["tb_in"][i]], [int(x) for x in G["tb_out"][i]]
        bt, n, P, w0, end, in_place = row[:6]
        a = Pool(n, bt)
        parent = [a.alloc() for _ in range((P + bt - 1) // bt)]
        for blk, s in zip(parent, row[6:]):
            if s == 1:
                a.retain(blk)
        assert a.new_blocks(parent, P, w0, end, in_place) == want[0], i
        blocks, cow = a.target_blocks(parent, P, w0, end, in_place)
        assert blocks == want[2:2 + want[1]], i
        nc = want[18]
        assert [x for pr in cow for x in pr] == want[19:19 + 2 * nc] and len(cow) == nc, i
        assert a.refs() == want[27:27 + n], i
        a.close()


def test_tree_rows_reproduce_the_reference_vectors():
    for i in range(N_TR):
        offs, toks = G[f"tr{i}_offs"], G[f"tr{i}_toks"]
        leaves = [[int(t) for t in toks[offs[k]:offs[k + 1]]] for k in range(len(offs) - 1)]
        base, pnext, sr = (int(x) for x in G[f"tr{i}_prm"])
        got = _tree_rows([int(t) for t in G[f"tr{i}_root"]], leaves, base, pnext, None, False, bool(sr))
        assert got["host"] == list(G[f"tr{i}_host"]) and got["off"] == list(G[f"tr{i}_off"]) and got["tok"] == list(G[f"tr{i}_tok"]), i
        assert got["pos"] == G[f"tr{i}_pos"].tolist() and got["desc"] == G[f"tr{i}_desc"].tolist() and got["next_root"] == int(G[f"tr{i}_next"]), i
        want_read = list(G[f"tr{i}_readout"])
        assert got["readouts"][:len(want_read)] == want_read, i


def test_e4m3_grid_reproduces_the_reference_vectors(oracle_lib):
    lib = oracle_lib.load()
    xs, q = G["e4m3_x"], G["e4m3_q"]
    assert np.array_equal(wl.e4m3_decode(wl.e4m3_encode(xs)), q)
    assert all(lib.orc_round_e4m3(float(x)) == float(v) for x, v in zip(xs, q))


def _combine_case():
    H, Hkv, HD = 2, 1, 256
    parts, X = G["cmb_parts"].astype(np.float32), G["cmb_X"].astype(np.float32)
    w = wl.make_pass("cmb", 1, [(0, 16)], H, Hkv, HD, 16, wl.F16, gate=True)
    w.X = X
    return w, parts, G["cmb_jobs"], G["cmb_O"]


def test_combine_restatement_reproduces_the_reference_kernel(oracle_lib):
    w, parts, jobs, want = _combine_case()
    got = np.zeros_like(want)
    lse = np.zeros((16, w.H), dtype=np.float32)
    oracle_lib.combine_f32(w, parts, jobs, got, lse, 8)
    live = np.r_[0:3, 8:16]
    a, b = wl.f16_bits_to_f32(got[live]), wl.f16_bits_to_f32(want[live])
    assert (got[live] != want[live]).mean() < 1e-3 and np.abs(a - b).max() <= 2.0 ** -10 * max(1.0, np.abs(b).max())


@pytest.mark.gpu
def test_cuda_combine_matches_the_reference_kernel():
    """esp_attn_combine_parts on the records of the stored case against what the reference's own
    attention_combine kernel produced from them: fp16 outputs within one unit in the last place."""
    import torch
    w, parts, jobs, want = _combine_case()
    op = host.AttnOp.for_workload(w, 8)
    try:
        dp = op.upload(w)
        parts_d = torch.from_numpy(parts).cuda()
        jobs_d = host._dev(jobs, op.device)
        op.combine(dp, parts_d, jobs_d, len(jobs))
        op.check_status()
        torch.cuda.synchronize()
        got = dp.O.cpu().numpy().view(np.uint16)
    finally:
        op.close()
    live = np.r_[0:3, 8:16]
    a, b = wl.f16_bits_to_f32(got[live]), wl.f16_bits_to_f32(want[live])
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(b), 2.0 ** -14))) - 10)
    assert (np.abs(a - b) <= ulp).all() and (got[live] != want[live]).mean() < 0.02
