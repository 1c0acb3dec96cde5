"""Qwen sparse attention (kernels/45_qsa.metal:281-690; host src/model/impl/forest.h:1462-1676): a row at sequence
index s with nb = (s + 1) / 4 > 512 complete blocks attends the 512 blocks its indexer scores highest plus its tail.
The library takes the scores and provides the rest. Checked here:
  CPU  - esp_qsa_plan and esp_attn_plan_qsa against the reference's own qsa_plan / plan_tiles (oracle/_ref), bit for bit;
       - the reference's qsa_select / qsa_tiles / flash_attention_qsa (SIMT emulator) against a direct float64 softmax
         over the keys each row selects (what tools/qsa_check.mm does for a few rows on a GPU);
       - the stored vectors (tests/golden/qsa.npz) still are what that pipeline produces.
  GPU  - esp_qsa_select and esp_qsa_tiles bit for bit, and esp_attn_forward over the lists within 2e-3, against the
         stored outputs of the reference pipeline (and against the float64 softmax)."""
import ctypes as C
import os

import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from oracle import ref

HAVE_REF = ref.load() is not None
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qsa.npz")
TOPK, LMAX = 512, 4112


def build_case(name):
    """A pass mixing a sparse decode row, a verify tree whose rows are all sparse, a tree that crosses the threshold
    inside an 8-row group, and a short dense tree; 256-dim fp16 heads with the gate (the reference kernel's shape)."""
    if name == "mixed":
        trees, H, Hkv, seed = [(2300, 1), (2200, 12), (2042, 14), (300, 3)], 2, 1, 9100
    else:  # "decode": single rows only, G = 4
        trees, H, Hkv, seed = [(2500, 1), (2051, 1), (2050, 1), (40, 1)], 8, 2, 9101
    mask = "forest" if name == "mixed" else "causal"
    w = wl.make_pass("qsa_" + name, seed, trees, H, Hkv, 256, 16, wl.F16, gate=True, scale=1.0 / 16.0, mask=mask)
    return w


def scores_for(w, plan, seed):
    """Indexer scores >= 0 with many ties (multiples of 1/8) and garbage past each row's nb."""
    rng = np.random.default_rng(seed)
    n, nbmax = plan["counts"][1], max(plan["counts"][2], 1)
    sc = (rng.integers(0, 64, size=(n, nbmax)) / 8.0).astype(np.float32)
    sc[rng.random(sc.shape) < 0.3] += np.float32(rng.random()) * 3
    return sc


def product_qsa_plan(trees, desc, sparse=True):
    lib = capi.load()
    trees = np.ascontiguousarray(trees)
    counts = (C.c_int32 * 6)()
    d = None if desc is None else np.ascontiguousarray(desc, dtype=np.int32)
    dp = None if d is None else C.c_void_p(d.ctypes.data)
    capi.check(lib.esp_qsa_plan(C.c_void_p(trees.ctypes.data), len(trees), dp, int(sparse), None, 0, None, 0, None, 0, None, 0, counts))
    M, n_sparse, nbmax, nbb, ncb, n_tiles = list(counts)
    groups = int(sum((int(t["M"]) + 7) // 8 for t in trees))
    rinfo, srows = np.zeros((M, 4), dtype=np.int32), np.zeros(max(1, n_sparse), dtype=np.int32)
    qtiles, qt_of = np.zeros((max(1, n_tiles), 4), dtype=np.int32), np.zeros(max(1, groups), dtype=np.int32)
    capi.check(lib.esp_qsa_plan(C.c_void_p(trees.ctypes.data), len(trees), dp, int(sparse), C.c_void_p(rinfo.ctypes.data), M, C.c_void_p(srows.ctypes.data),
                                len(srows), C.c_void_p(qtiles.ctypes.data), len(qtiles), C.c_void_p(qt_of.ctypes.data), len(qt_of), counts))
    return dict(rinfo=rinfo, srows=srows[:n_sparse], qtiles=qtiles[:n_tiles], qt_of=qt_of[:groups], counts=list(counts))


def product_plan_tiles(trees, Hkv, qt, split=512, groups=256, min_chunk=32):
    lib = capi.load()
    trees = np.ascontiguousarray(trees, dtype=wl.TREE_DT)
    qt = np.ascontiguousarray(qt, dtype=np.int32)
    opts = capi.PlanOpts(capi.ESP_PLAN_REFERENCE, split, min_chunk, groups, 8, 64)
    nt, nj, npart = C.c_int32(), C.c_int32(), C.c_int32()
    tp = trees.ctypes.data_as(C.POINTER(capi.Tree))
    capi.check(lib.esp_attn_plan_qsa(tp, len(trees), Hkv, C.byref(opts), C.c_void_p(qt.ctypes.data), None, 0, None, 0, C.byref(nt), C.byref(nj), C.byref(npart)))
    tiles, jobs = np.zeros(max(1, nt.value), dtype=wl.TILE_DT), np.zeros(max(1, nj.value), dtype=wl.COMBINE_DT)
    capi.check(lib.esp_attn_plan_qsa(tp, len(trees), Hkv, C.byref(opts), C.c_void_p(qt.ctypes.data), tiles.ctypes.data_as(C.POINTER(capi.Tile)), len(tiles),
                                     jobs.ctypes.data_as(C.POINTER(capi.Combine)), len(jobs), C.byref(nt), C.byref(nj), C.byref(npart)))
    return host.Plan(tiles[:nt.value], jobs[:nj.value], npart.value, 8)


def selected_keys_f64(w, rinfo, sel, scores_unused=None):
    """Direct float64 softmax over the keys every row attends under the selection: the dense rule for rows with nb <= 512;
    else the selected blocks' tokens and the tail, among the cached keys and the row's visible batch keys."""
    from oracle import attention_f64  # noqa: F401  (the dense oracle is not used: the key sets differ)
    G, HD = w.G, w.HD
    Q = wl.f16_bits_to_f32(w.Q).astype(np.float64).reshape(w.n_rows, w.H, HD)
    Kb = wl.f16_bits_to_f32(w.Kb).astype(np.float64).reshape(w.n_rows, w.Hkv, HD)
    Vb = wl.f16_bits_to_f32(w.Vb).astype(np.float64).reshape(w.n_rows, w.Hkv, HD)
    pool = wl.f16_bits_to_f32(w.kv).astype(np.float64).reshape(w.n_blocks, 2, w.bt, w.Hkv, HD)
    out = np.zeros((w.n_rows, w.H, HD))
    for ti, t in enumerate(w.trees):
        base, P, table, M = (int(t[k]) for k in ("base", "P", "table", "M"))
        for rr in range(M):
            r = base + rr
            s, nb, srow, _ = (int(x) for x in rinfo[r])
            d = [int(x) for x in w.desc[r]]
            keys = []                                        # (K row, V row) per kv head come from here
            for j in range(P):                               # cached key j has sequence index j
                if srow < 0 or j >= 4 * nb or (int(sel[srow, (j >> 2) >> 5]) >> ((j >> 2) & 31)) & 1:
                    b = int(w.blocks[table + j // w.bt])
                    keys.append((pool[b, 0, j % w.bt], pool[b, 1, j % w.bt]))
            for j in range(M):                               # batch key j of the tree
                if not (j < d[2] or d[0] <= j <= rr):
                    continue
                sj = P + (j if j < d[2] else d[2] + (j - d[0]))
                if srow < 0 or sj >= 4 * nb or (int(sel[srow, (sj >> 2) >> 5]) >> ((sj >> 2) & 31)) & 1:
                    keys.append((Kb[base + j], Vb[base + j]))
            K = np.stack([k for k, _ in keys])               # [n, Hkv, HD]
            V = np.stack([v for _, v in keys])
            for h in range(w.H):
                sc = (K[:, h // G] @ Q[r, h]) * w.scale
                p = np.exp(sc - sc.max())
                o = (p / p.sum()) @ V[:, h // G]
                gate = w.X[r, h * 2 * HD + HD:h * 2 * HD + 2 * HD].astype(np.float64)
                out[r, h] = o / (1.0 + np.exp(-gate))
    return out.reshape(w.n_rows, -1)


def reference_pipeline(name):
    """plan, scores, selection, lists and attention as the reference runs them (its own code throughout)."""
    w = build_case(name)
    plan = ref.qsa_plan(w.trees, w.desc)
    scores = scores_for(w, plan, 77)
    nbmax = max(plan["counts"][2], 1)
    tiles, jobs, n_parts = ref.plan_tiles(w.trees, w.Hkv, 512, 256, 32, qt=plan["qt_of"])
    sel = ref.qsa_select(scores, plan["srows"], plan["rinfo"], nbmax)
    tlist, tcount = ref.qsa_tiles(sel, w.trees, plan["rinfo"], plan["qtiles"], nbmax)
    O, parts = ref.attention_qsa(w, tiles, n_parts, tlist, tcount, plan["rinfo"], sel, nbmax)
    if len(jobs):
        import oracle
        p = oracle.Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
        X = np.ascontiguousarray(w.X, dtype=np.float32)
        ref.load().ref_attention_combine(C.c_void_p(parts.ctypes.data), C.c_void_p(X.ctypes.data), C.c_void_p(O.ctypes.data), C.byref(p),
                                         C.c_void_p(np.ascontiguousarray(jobs).ctypes.data), len(jobs))
    return dict(w=w, plan=plan, scores=scores, nbmax=nbmax, tiles=tiles, jobs=jobs, n_parts=n_parts, sel=sel, tlist=tlist, tcount=tcount, O=O)


needs_ref = pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref/libplan_ref.so was not built (no reference tree on this machine)")


@needs_ref
def test_qsa_plan_and_planner_branch_bit_for_bit():
    rng = np.random.default_rng(9200)
    for case in range(120):
        n = int(rng.integers(1, 6))
        pm = [(int(rng.choice([0, 100, 2040, 2047, 2051, 2100, 4000, int(rng.integers(0, 6000))])), int(rng.choice([1, 1, 3, 8, 9, 16, 20]))) for _ in range(n)]
        w = wl.make_pass("qp", 1, [(0, m) for _, m in pm], 2, 1, 128, 16, wl.BF16, mask="forest" if case % 2 else "causal")
        trees = w.trees.copy()
        tab = 0
        for i, (P, _) in enumerate(pm):
            trees[i]["P"], trees[i]["table"] = P, tab
            tab += (P + 15) // 16
        desc = w.desc if case % 3 else None
        sparse = case % 7 != 0
        want, got = ref.qsa_plan(trees, desc, sparse), product_qsa_plan(trees, desc, sparse)
        assert got["counts"] == want["counts"], case
        for k in ("rinfo", "srows", "qtiles", "qt_of"):
            assert np.array_equal(got[k], want[k]), (case, k)
        Hkv, split, groups = int(rng.choice([1, 2, 4])), int(rng.choice([0, 128, 512])), int(rng.choice([256, 64, 1024]))
        t, j, npart = ref.plan_tiles(trees, Hkv, split, groups, 32, qt=want["qt_of"])
        p = product_plan_tiles(trees, Hkv, got["qt_of"], split, groups)
        assert p.n_parts == npart and p.tiles.tobytes() == t.tobytes() and p.jobs.tobytes() == j.tobytes(), case


@needs_ref
@pytest.mark.parametrize("name", ["mixed", "decode"])
def test_reference_pipeline_matches_a_direct_float64_softmax(name):
    r = reference_pipeline(name)
    w, plan, sel = r["w"], r["plan"], r["sel"]
    assert plan["counts"][1] > 0 and (np.asarray(r["tiles"]["pad0"]) != 0).any()
    # every sparse row selects exactly 512 blocks among its nb
    for i, row in enumerate(plan["srows"]):
        nb = int(plan["rinfo"][row, 1])
        bits = np.unpackbits(sel[i].view(np.uint8), bitorder="little")
        assert bits[:nb].sum() == TOPK and bits[nb:].sum() == 0
        sc = r["scores"][i, :nb]
        thr = np.sort(sc)[-TOPK]
        assert (sc[bits[:nb] == 1] >= thr).all() and (sc[bits[:nb] == 0] <= thr).all()
        tied = np.flatnonzero(sc == thr)
        taken = tied[bits[tied] == 1]
        assert np.array_equal(taken, tied[:len(taken)])      # ties go to the lowest blocks
    want = selected_keys_f64(w, plan["rinfo"], sel)
    got = wl.f16_bits_to_f32(r["O"]).astype(np.float64)
    assert np.abs(got - want).max() < 1.5e-3
    # and the selection matters: the dense result differs
    import oracle
    dense, _ = oracle.attention_f64(w)
    assert np.abs(dense - want).max() > 1e-2


@needs_ref
def test_stored_vectors_are_what_the_reference_pipeline_produces():
    g = np.load(GOLDEN)
    for name in ("mixed", "decode"):
        r = reference_pipeline(name)
        assert np.array_equal(r["sel"], g[name + "_sel"]) and np.array_equal(r["tcount"], g[name + "_tcount"])
        for i, n in enumerate(r["tcount"]):
            assert np.array_equal(r["tlist"][i, :n], g[name + "_tlist"][i, :n])
        assert np.array_equal(r["O"], g[name + "_O"])


def _golden_case(name):
    """The case and the reference pipeline's stored outputs; the plan comes from the product's own host functions."""
    g = np.load(GOLDEN)
    w = build_case(name)
    plan = product_qsa_plan(w.trees, w.desc)
    assert plan["counts"] == [int(x) for x in g[name + "_counts"]] and np.array_equal(plan["rinfo"], g[name + "_rinfo"])
    scores = scores_for(w, plan, 77)
    return g, w, plan, scores, max(plan["counts"][2], 1)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "decode"])
def test_cuda_selection_lists_and_attention_match_the_reference(name):
    import torch
    lib = capi.load()
    g, w, plan, scores, nbmax = _golden_case(name)
    nbw = (nbmax + 31) // 32
    dev = torch.device("cuda", 0)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    d_scores, d_srows = torch.from_numpy(scores).to(dev), torch.from_numpy(plan["srows"]).to(dev)
    d_rinfo, d_qtiles = torch.from_numpy(plan["rinfo"]).to(dev), torch.from_numpy(plan["qtiles"]).to(dev)
    n_sparse, n_qt = len(plan["srows"]), len(plan["qtiles"])
    d_sel = torch.full((n_sparse, nbw), -1, dtype=torch.int32, device=dev)
    d_tlist = torch.zeros((n_qt, LMAX), dtype=torch.int32, device=dev)
    d_tcount = torch.zeros(n_qt, dtype=torch.int32, device=dev)
    op = host.AttnOp.for_workload(w, 8)
    try:
        ptiles = product_plan_tiles(w.trees, w.Hkv, plan["qt_of"])
        dp = op.upload(w, ptiles)
        capi.check(lib.esp_qsa_select(s, C.c_void_p(d_scores.data_ptr()), C.c_void_p(d_srows.data_ptr()), C.c_void_p(d_rinfo.data_ptr()),
                                      C.c_void_p(d_sel.data_ptr()), n_sparse, nbmax, nbw))
        capi.check(lib.esp_qsa_tiles(s, C.c_void_p(d_sel.data_ptr()), C.c_void_p(dp.trees.data_ptr()), C.c_void_p(d_rinfo.data_ptr()),
                                     C.c_void_p(d_qtiles.data_ptr()), n_qt, C.c_void_p(d_tlist.data_ptr()), C.c_void_p(d_tcount.data_ptr()), nbmax, nbw))
        torch.cuda.synchronize()
        sel = d_sel.cpu().numpy().view(np.uint32)
        tcount, tlist = d_tcount.cpu().numpy().view(np.uint32), d_tlist.cpu().numpy().view(np.uint32)
        assert np.array_equal(sel, g[name + "_sel"]) and np.array_equal(tcount, g[name + "_tcount"])
        for i, n in enumerate(tcount):
            assert np.array_equal(tlist[i, :n], g[name + "_tlist"][i, :n])
        a = op.make_args(dp)
        a.qsa_tlist, a.qsa_tcount, a.qsa_rinfo, a.qsa_sel = d_tlist.data_ptr(), d_tcount.data_ptr(), d_rinfo.data_ptr(), d_sel.data_ptr()
        a.qsa_nbw, a.qsa_n_lists = nbw, n_qt
        op.forward(dp, a)
        op.check_status()
        torch.cuda.synchronize()
        assert op.last_kernel == "flash_general"
        got = wl.f16_bits_to_f32(dp.O.cpu().numpy().view(np.uint16)).astype(np.float64)
        want = wl.f16_bits_to_f32(g[name + "_O"]).astype(np.float64)
        half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 2.0 ** -14))) - 11)
        assert (np.abs(got - want) <= 2e-3 + half_ulp).all(), f"max abs err {np.abs(got - want).max():.3e}"
        f64 = selected_keys_f64(w, plan["rinfo"], sel)
        assert np.abs(got - f64).max() < 2e-3
        # without the lists the same plan is refused (its sparse tiles name entries, not keys), nothing is launched
        b = op.make_args(dp)
        with pytest.raises(capi.EspError):
            op.forward(dp, b)
    finally:
        op.close()
