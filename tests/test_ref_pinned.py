"""Pins against the reference's OWN code. oracle/_ref/libplan_ref.so holds plan_tiles, g4_plan_tiles, the
KV pool with target_blocks / target_new_blocks, kv_row_table, run_forest's leaf hosting, row records and
block tables, the E4M3 codec and the three per-thread kernels (attention_combine, kv_save, kv_copy_blocks),
cut out of the reference tree and compiled as they stand (oracle/extract_ref.py, oracle/ref_glue.cpp). The
product's host functions (through the C ABI) and the oracle's restatements must agree with it bit for bit
on random and edge inputs. No GPU needed. Skipped only where the library was never built (a machine that
has never seen the reference tree); tests/golden/ref_vectors.npz carries vectors it produced for those."""
import ctypes as C

import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from espetero_b200.workloads import KVSAVE_DT, TREE_DT
from oracle import ref
from tests.test_forest_host import Pool, _tree_rows
from tests.test_planner import _trees

pytestmark = pytest.mark.skipif(ref.load() is None, reason="oracle/_ref/libplan_ref.so was not built (no reference tree on this machine)")


def _random_trees(rng):
    n = int(rng.integers(1, 40))
    return _trees([(int(rng.choice([0, 1, 31, 63, 64, 65, 100, 511, 512, 513, 4096, 40000, int(rng.integers(0, 70000))])),
                    int(rng.choice([1, 1, 1, 2, 7, 8, 9, 16, 17, 100]))) for _ in range(n)])


def test_plan_tiles_bit_for_bit(oracle_lib):
    rng = np.random.default_rng(111)
    for case in range(300):
        trees = _random_trees(rng)
        Hkv, split = int(rng.choice([1, 2, 4, 8])), int(rng.choice([0, 128, 512, 1024]))
        min_chunk, groups = int(rng.choice([32, 32, 128, 512])), int(rng.choice([256, 64, 1024]))
        want_t, want_j, want_n = ref.plan_tiles(trees, Hkv, split, groups, min_chunk)
        got = host.plan_tiles(trees, Hkv, capi.ESP_PLAN_REFERENCE, split, min_chunk, groups, 8)
        assert got.n_parts == want_n and got.tiles.tobytes() == want_t.tobytes() and got.jobs.tobytes() == want_j.tobytes(), case
        t2, j2, n2 = oracle_lib.plan_tiles(trees, Hkv, split, groups, min_chunk, 8)
        assert n2 == want_n and t2.tobytes() == want_t.tobytes() and j2.tobytes() == want_j.tobytes(), case
    # the configurations' own plans
    for pm, Hkv in (([(1024, 1)], 2), ([(131072, 1)], 8), ([(0, 8192)] * 4, 8), ([(4096, 16)] * 16, 4)):
        trees = _trees(pm)
        want_t, want_j, want_n = ref.plan_tiles(trees, Hkv)
        got = host.plan_tiles(trees, Hkv)
        assert got.n_parts == want_n and got.tiles.tobytes() == want_t.tobytes() and got.jobs.tobytes() == want_j.tobytes()


def test_g4_plan_tiles_bit_for_bit(oracle_lib):
    rng = np.random.default_rng(112)
    for case in range(200):
        n = int(rng.integers(1, 20))
        trees = _trees([(int(rng.integers(0, 50000)), int(rng.choice([1, 1, 8, 24, 100]))) for _ in range(n)])
        groups, split, rows = int(rng.choice([1, 2, 4, 8, 16])), int(rng.choice([0, 512])), int(rng.choice([8, 16]))
        want_t, want_j, want_n, want_rows = ref.g4_plan_tiles(trees, groups, split, rows)
        got = host.plan_tiles(trees, groups, capi.ESP_PLAN_G4, split, 32, 256, rows)
        assert got.n_parts == want_n and got.tiles.tobytes() == want_t.tobytes() and got.jobs.tobytes() == want_j.tobytes(), case
        t2, j2, n2, r2 = oracle_lib.g4_plan_tiles(trees, groups, split, rows)
        assert (n2, r2) == (want_n, want_rows) and t2.tobytes() == want_t.tobytes() and j2.tobytes() == want_j.tobytes(), case
    # with the sliding-window branch
    rng = np.random.default_rng(113)
    for case in range(100):
        n_trees = int(rng.integers(1, 6))
        pm = [(int(rng.integers(0, 5000)), int(rng.integers(1, 40))) for _ in range(n_trees)]
        trees = _trees(pm)
        n_rows = sum(m for _, m in pm)
        pos = np.zeros((n_rows, 4), dtype=np.int32)
        for t in trees:
            b0, P, M = int(t["base"]), int(t["P"]), int(t["M"])
            pos[b0:b0 + M, 0] = P + np.sort(rng.integers(0, M, size=M))
        window, groups = int(rng.choice([0, 1, 17, 512, 1024, 100000])), int(rng.choice([1, 2, 8, 32]))
        split, rows = int(rng.choice([0, 256, 512])), int(rng.choice([8, 16]))
        want_t, want_j, want_n, want_rows = ref.g4_plan_tiles(trees, groups, split, rows, window, pos)
        got = host.plan_window(trees, groups, split, rows, window, pos)
        assert (got.n_parts, got.tile_rows) == (want_n, want_rows), case
        assert got.tiles.tobytes() == want_t.tobytes() and got.jobs.tobytes() == want_j.tobytes(), case
        t2, j2, n2, r2 = oracle_lib.g4_plan_tiles(trees, groups, split, rows, window, pos)
        assert (n2, r2) == (want_n, want_rows) and t2.tobytes() == want_t.tobytes() and j2.tobytes() == want_j.tobytes(), case


def test_kv_pool_and_target_blocks_bit_for_bit():
    a, b = Pool(4, 16), ref.Pool(4, 16)
    assert [a.alloc() for _ in range(4)] == [b.alloc() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(capi.EspError) as e1:
        a.alloc()
    with pytest.raises(RuntimeError) as e2:
        b.alloc()
    assert str(e2.value) in str(e1.value) and "KV cache full" in str(e2.value)   # the reference's message, word for word
    a.release(2), b.release(2), a.release(0), b.release(0)
    assert (a.alloc(), a.alloc()) == (b.alloc(), b.alloc())                # the same LIFO order
    a.close(), b.close()
    rng = np.random.default_rng(121)
    for case in range(400):
        bt, n = int(rng.choice([16, 64])), 40
        a, b = Pool(n, bt), ref.Pool(n, bt)
        P = int(rng.integers(0, 6 * bt))
        parent = [a.alloc() for _ in range((P + bt - 1) // bt)]
        assert parent == [b.alloc() for _ in parent]
        for blk in parent:
            if rng.random() < 0.3:
                a.retain(blk), b.retain(blk)
        w0 = int(rng.integers(max(0, P - 1), P + 1)) if P else 0
        end = w0 + int(rng.integers(1, 3 * bt))
        in_place = bool(rng.integers(0, 2))
        assert a.new_blocks(parent, P, w0, end, in_place) == b.new_blocks(parent, P, w0, end, in_place), case
        got, want = a.target_blocks(parent, P, w0, end, in_place), b.target_blocks(parent, P, w0, end, in_place)
        assert got == want and a.refs() == b.refs() and a.free() == b.free(), case
        a.close(), b.close()


def test_row_table_and_block_tables_bit_for_bit():
    lib = capi.load()
    rng = np.random.default_rng(131)
    for case in range(200):
        rows = int(rng.integers(1, 30))
        ents = []
        for r in range(rows):
            for _ in range(int(rng.integers(0, 3))):
                ents.append((r, int(rng.integers(0, 100)), int(rng.integers(0, 16)), 0))
        order = rng.permutation(len(ents))
        ents = np.array([ents[i] for i in order], dtype=KVSAVE_DT) if ents else np.zeros(0, dtype=KVSAVE_DT)
        table = np.zeros(rows * 4, dtype=np.int32)
        capi.check(lib.esp_kv_row_table(ents.ctypes.data if len(ents) else None, len(ents), rows, table.ctypes.data))
        assert table.tobytes() == ref.kv_row_table(ents, rows).tobytes(), case
    # run_forest's table building for a few targets: the product's pieces composed the same way
    for case in range(150):
        bt, n = int(rng.choice([16, 64])), 64
        a, b = Pool(n, bt), ref.Pool(n, bt)
        n_trees = int(rng.integers(1, 5))
        parents, P, base, save_len, same = [], [], [], [], []
        row = 0
        for _ in range(n_trees):
            p = int(rng.integers(0, 4 * bt))
            blocks = [a.alloc() for _ in range((p + bt - 1) // bt)]
            assert blocks == [b.alloc() for _ in blocks]
            parents.append(blocks), P.append(p), base.append(row), same.append(int(rng.integers(0, 2)))
            save_len.append(int(rng.integers(1, 2 * bt)))
            row += save_len[-1]
        table, lists, cow, saves = ref.block_tables(b, parents, P, base, save_len, same)
        got_table, got_cow, got_saves = [], [], []
        for i in range(n_trees):
            got_table += parents[i][:(P[i] + bt - 1) // bt]
            out, cw = a.target_blocks(parents[i], P[i], P[i], P[i] + save_len[i], bool(same[i]))
            assert out == lists[i], case
            got_cow += cw
            ent = np.zeros(save_len[i], dtype=KVSAVE_DT)
            ob = np.asarray(out, dtype=np.int32)
            capi.check(lib.esp_kv_save_entries(ob.ctypes.data, len(ob), bt, P[i], base[i], save_len[i], ent.ctypes.data))
            got_saves.append(ent)
        assert got_table == table and got_cow == cow, case
        assert np.concatenate(got_saves).tobytes() == saves.tobytes(), case
        assert a.refs() == b.refs()
        a.close(), b.close()


def test_tree_rows_bit_for_bit():
    rng = np.random.default_rng(141)
    for case in range(300):
        Tr = int(rng.integers(1, 6))
        root = [int(x) for x in rng.integers(0, 50, Tr)]
        leaves = []
        for _ in range(int(rng.integers(0, 7))):
            if leaves and rng.random() < 0.5:
                src = leaves[int(rng.integers(0, len(leaves)))]
                leaf = src[:int(rng.integers(1, len(src) + 1))] + [int(x) for x in rng.integers(0, 4, int(rng.integers(0, 3)))]
            else:
                leaf = [int(x) for x in rng.integers(0, 4, int(rng.integers(1, 5)))]
            leaves.append(leaf)
        root_pos = [[int(x) for x in rng.integers(0, 30, 3)] for _ in range(Tr)] if rng.random() < 0.3 else None
        base, pnext, sr = int(rng.integers(0, 100)), int(rng.integers(0, 1000)), bool(rng.integers(0, 2))
        noncausal = not leaves and bool(rng.integers(0, 2))
        got = _tree_rows(root, leaves, base, pnext, root_pos, noncausal, sr)
        want = ref.tree_rows(root, leaves, None if root_pos is None else np.asarray(root_pos).reshape(-1), noncausal, sr, base, pnext)
        assert got["host"] == list(want["host"]) and got["off"] == list(want["off"]) and got["M"] == want["n_rows"], case
        assert got["tok"] == list(want["tok"]) and got["pos"] == want["pos"].tolist() and got["desc"] == want["desc"].tolist(), case
        assert got["next_root"] == want["next_root"], case
        assert got["readouts"][:len(want["readout"])] == list(want["readout"]), case


def test_e4m3_codec_bit_for_bit(oracle_lib):
    lib = oracle_lib.load()
    # every code decodes as the reference's ds4_e4m3x2 says (value * 2^-8 there)
    codes = np.arange(256, dtype=np.uint8)
    dec = wl.e4m3_decode(codes)
    for c in range(256):
        if (c & 0x7F) == 0x7F:
            continue                                       # the NaN codes: the reference's bit trick maps them to a number
        lo, hi = ref.e4m3x2(c | (c << 8))
        assert lo == hi == float(dec[c]) * 2.0 ** -8 == lib.orc_e4m3_decode(c) * 2.0 ** -8, c
    # rounding to the grid: the oracle's and numpy's encoders land where ds4_round_e4m3 does
    rng = np.random.default_rng(151)
    xs = np.concatenate([rng.standard_normal(20000) * rng.choice([1e-3, 0.05, 1.0, 30.0, 400.0], 20000),
                         dec[np.isfinite(dec)], (dec[:-1] + dec[1:])[np.isfinite(dec[:-1] + dec[1:])] / 2,
                         np.array([0.0, -0.0, 448.0, -448.0, 449.0, 1e9, -1e9, 2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10])]).astype(np.float32)
    enc = wl.e4m3_encode(xs)
    back = wl.e4m3_decode(enc)
    for x, q, e in zip(xs, back, enc):
        want = ref.round_e4m3(float(x))
        assert float(q) == want and lib.orc_round_e4m3(float(x)) == want and lib.orc_e4m3_encode(float(x)) == int(e), float(x)


def test_combine_and_kv_kernels_against_the_reference_kernels(oracle_lib):
    """attention_combine, kv_save and kv_copy_blocks of kernels/40_attention.metal run thread by thread on the
    CPU (they use no threadgroup cooperation); the oracle's restatements must give the same bits - for the
    combine, up to the last bit of the fp32 weights (libm exp on both sides, same order)."""
    lib, rl = oracle_lib.load(), ref.load()
    rng = np.random.default_rng(161)
    H, Hkv, HD, G = 16, 2, 256, 8
    for case in range(20):
        n_jobs = int(rng.integers(1, 4))
        jobs, part = [], 0
        for j in range(n_jobs):
            rows, nparts = int(rng.integers(1, 9)), int(rng.choice([1, 2, 7, 8, 9, 20]))
            jobs.append((8 * j, rows, part, nparts))
            part += nparts
        jobs = np.array(jobs, dtype=wl.COMBINE_DT)
        n_rows = 8 * n_jobs
        parts = rng.standard_normal(part * Hkv * 8 * G * (HD + 2)).astype(np.float32)
        rec = parts.reshape(-1, HD + 2)
        rec[:, HD] = rng.uniform(-5, 5, len(rec))
        rec[:, HD + 1] = rng.uniform(0.5, 40, len(rec))
        empty = rng.random(len(rec)) < 0.1
        rec[empty, HD], rec[empty, HD + 1], rec[empty, :HD] = -np.inf, 0.0, 0.0
        X = rng.standard_normal((n_rows, 2 * H * HD)).astype(np.float32)
        p = oracle_lib.Params(H, Hkv, H * HD, Hkv * HD, 2 * H * HD, 16, 0)
        want = np.zeros((n_rows, H * HD), dtype=np.uint16)
        rl.ref_attention_combine(C.c_void_p(parts.ctypes.data), C.c_void_p(X.ctypes.data), C.c_void_p(want.ctypes.data), C.byref(p),
                                 C.c_void_p(jobs.ctypes.data), n_jobs)
        w = wl.make_pass("cmb", 1, [(0, n_rows)], H, Hkv, HD, 16, wl.F16, gate=True)
        w.X = X
        got = np.zeros_like(want)
        lse = np.zeros((n_rows, H), dtype=np.float32)
        oracle_lib.combine_f32(w, parts, jobs, got, lse, 8)
        live = np.zeros(n_rows, dtype=bool)
        for j in jobs:
            live[int(j["r0"]):int(j["r0"]) + int(j["rows"])] = True
        a, b = wl.f16_bits_to_f32(got[live]), wl.f16_bits_to_f32(want[live])
        assert np.array_equal(got[live], want[live]) or np.abs(a - b).max() <= 2.0 ** -10 * np.abs(b).max(), case
        assert (np.abs(a - b) > 0).mean() < 1e-3, case
    # kv_save / kv_copy_blocks: pure copies
    w = wl.make_pass("kvs", 2, [(40, 12)], 8, 2, 256, 16, wl.F16)
    p = oracle_lib.Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, 0)
    ents = np.array([(r, int(rng.integers(0, w.n_blocks)), int(rng.integers(0, 16)), 0) for r in range(12)], dtype=KVSAVE_DT)
    want, got = w.kv.copy(), w.kv.copy()
    rl.ref_kv_save(C.c_void_p(w.Kb.ctypes.data), C.c_void_p(w.Vb.ctypes.data), C.c_void_p(want.ctypes.data), C.c_void_p(ents.ctypes.data), len(ents), C.byref(p))
    oracle_lib.kv_save(w, got, ents)
    assert np.array_equal(got, want) and not np.array_equal(got, w.kv)
    region = w.n_blocks * 2 * w.bt * w.kv_ld
    pool3 = np.concatenate([w.kv, w.kv[::-1].copy(), w.kv]).copy()
    want, got = pool3.copy(), pool3.copy()
    pairs = np.array([[0, 3], [2, 1]], dtype=np.int32)
    rl.ref_kv_copy_blocks(C.c_void_p(want.ctypes.data), C.c_void_p(pairs.ctypes.data), 2, C.byref(p), region, 3)
    oracle_lib.kv_copy_blocks(w, got, pairs, region, 3)
    assert np.array_equal(got, want) and not np.array_equal(got, pool3)
