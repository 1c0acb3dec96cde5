"""The integer planner: the product's esp_attn_plan (host code of the C-ABI library) must
match the oracle's restatement of plan_tiles (src/model/impl/forest.h:1378-1433) and
g4_plan_tiles (src/model/impl/gemma.h:77-116) bit for bit, and hand-derived cases."""
import numpy as np
import pytest

from espetero_b200 import capi, host
from espetero_b200.workloads import TREE_DT


def _trees(pm):
    t = np.zeros(len(pm), dtype=TREE_DT)
    base = tab = 0
    for i, (P, M) in enumerate(pm):
        t[i] = (base, P, tab, M)
        base += M
        tab += (P + 15) // 16
    return t


def test_reference_mode_matches_oracle(oracle_lib):
    rng = np.random.default_rng(11)
    for case in range(300):
        n = int(rng.integers(1, 40))
        pm = [(int(rng.choice([0, 1, 31, 63, 64, 65, 100, 511, 512, 513, 4096, 40000, int(rng.integers(0, 70000))])),
               int(rng.choice([1, 1, 1, 2, 7, 8, 9, 16, 17, 100]))) for _ in range(n)]
        trees = _trees(pm)
        Hkv = int(rng.choice([1, 2, 4, 8]))
        split = int(rng.choice([0, 128, 512, 1024]))
        min_chunk = int(rng.choice([32, 32, 128, 512]))
        groups = int(rng.choice([256, 64, 1024]))
        got = host.plan_tiles(trees, Hkv, capi.ESP_PLAN_REFERENCE, split, min_chunk, groups, 8)
        tiles, jobs, nparts = oracle_lib.plan_tiles(trees, Hkv, split, groups, min_chunk, 8)
        assert got.n_parts == nparts, case
        assert np.array_equal(got.tiles, tiles), case
        assert np.array_equal(got.jobs, jobs), case


def test_g4_mode_matches_oracle(oracle_lib):
    rng = np.random.default_rng(12)
    for case in range(200):
        n = int(rng.integers(1, 20))
        pm = [(int(rng.integers(0, 50000)), int(rng.choice([1, 1, 8, 24, 100]))) for _ in range(n)]
        trees = _trees(pm)
        groups = int(rng.choice([1, 2, 4, 8, 16]))
        split = int(rng.choice([0, 512]))
        rows = int(rng.choice([8, 16]))
        got = host.plan_tiles(trees, groups, capi.ESP_PLAN_G4, split, 32, 256, rows)
        tiles, jobs, nparts, plan_rows = oracle_lib.g4_plan_tiles(trees, groups, split, rows)
        assert got.n_parts == nparts
        assert np.array_equal(got.tiles, tiles)
        assert np.array_equal(got.jobs, jobs)


def test_hand_derived_cases():
    # One decode row at a 1024-token context, Hkv 2: budget = 256 / (2 * 1) = 128; chunk =
    # max(32, min(512, ceil(1024/128) rounded up to 32)) = 32; 32 parts of 32 keys.
    p = host.plan_tiles(_trees([(1024, 1)]), 2)
    assert len(p.tiles) == 32 and p.n_parts == 32 and len(p.jobs) == 1
    assert [int(t["k0"]) for t in p.tiles] == list(range(0, 1024, 32))
    assert all(int(t["k1"]) - int(t["k0"]) == 32 for t in p.tiles)
    assert [int(t["last"]) for t in p.tiles] == [0] * 31 + [1]
    assert [int(t["part"]) for t in p.tiles] == list(range(32))
    assert tuple(p.jobs[0]) == (0, 1, 0, 32)
    # 131072 keys, Hkv 8: budget 32; chunk = min(512, 4096) = 512 -> ceil(P / 512) = 256 capped by budget 32:
    # 32 parts of 4096 keys.
    p = host.plan_tiles(_trees([(131072, 1)]), 8)
    assert len(p.tiles) == 32 and all(int(t["k1"]) - int(t["k0"]) == 4096 for t in p.tiles)
    # Short context: below 64 keys nothing is split.
    p = host.plan_tiles(_trees([(63, 1)]), 2)
    assert len(p.tiles) == 1 and int(p.tiles[0]["part"]) == -1 and int(p.tiles[0]["last"]) == 1 and len(p.jobs) == 0
    # Prefill: many tiles -> budget 1 -> unsplit 8-row tiles, the last one short.
    p = host.plan_tiles(_trees([(0, 8192)]), 8)
    assert len(p.tiles) == 1024 and p.n_parts == 0
    p = host.plan_tiles(_trees([(100, 20)]), 4)
    assert [int(t["r0"]) for t in p.tiles if t["k0"] == 0] == [0, 8, 16]
    # split = 0 never splits
    p = host.plan_tiles(_trees([(5000, 1)]), 2, split=0)
    assert len(p.tiles) == 1 and p.n_parts == 0
    # 64 parts at most
    p = host.plan_tiles(_trees([(64 * 32 * 4, 1)]), 1, split=32)
    assert len(p.tiles) <= 64


@pytest.mark.parametrize("groups", [148, 296, 592])
def test_b200_mode_properties(groups):
    rng = np.random.default_rng(13)
    for case in range(100):
        n = int(rng.integers(1, 40))
        pm = [(int(rng.integers(0, 40000)), int(rng.choice([1, 1, 1, 16]))) for _ in range(n)]
        trees = _trees(pm)
        Hkv = int(rng.choice([2, 4, 8]))
        TR = int(rng.choice([8, 16]))
        p = host.plan_tiles(trees, Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, groups, TR)
        # every row group's cached range is covered exactly once, in order, on 32-key boundaries
        seen = {}
        for t in p.tiles:
            key = (int(t["tree"]), int(t["r0"]))
            seen.setdefault(key, []).append(t)
        for (ti, r0), ts in seen.items():
            P = int(trees[ti]["P"])
            assert int(ts[0]["k0"]) == 0 and int(ts[-1]["k1"]) == P
            for a, b in zip(ts, ts[1:]):
                assert int(a["k1"]) == int(b["k0"]) and int(a["k1"]) % 32 == 0
            assert [int(t["last"]) for t in ts] == [0] * (len(ts) - 1) + [1]
            if len(ts) == 1:
                assert int(ts[0]["part"]) == -1
            else:
                assert len(ts) <= 64
        assert len(seen) == sum((int(t["M"]) + TR - 1) // TR for t in trees)
        # records are numbered consecutively and each job covers its group's records
        parts = sorted(int(t["part"]) for t in p.tiles if t["part"] >= 0)
        assert parts == list(range(p.n_parts))
        assert sum(int(j["nparts"]) for j in p.jobs) == p.n_parts


def test_b200_mode_balances_c2_like_batch():
    rng = np.random.default_rng(14)
    lens = rng.integers(512, 32769, size=32)
    trees = _trees([(int(p), 1) for p in lens])
    p = host.plan_tiles(trees, 4, capi.ESP_PLAN_B200, 1 << 20, 32, 4 * 296, 8)
    sizes = np.array([int(t["k1"]) - int(t["k0"]) for t in p.tiles])
    assert 250 <= len(p.tiles) <= 400
    assert sizes.max() <= 2 * np.median(sizes)


def test_plan_errors():
    lib = capi.load()
    import ctypes as C
    nt, nj, np_ = C.c_int32(), C.c_int32(), C.c_int32()
    trees = _trees([(1024, 1)])
    opts = capi.PlanOpts(7, 512, 32, 256, 8, 64)
    rc = lib.esp_attn_plan(trees.ctypes.data_as(C.POINTER(capi.Tree)), 1, 2, C.byref(opts), None, 0, None, 0, C.byref(nt), C.byref(nj), C.byref(np_))
    assert rc == capi.ESP_ERR_INVALID and b"mode" in lib.esp_attn_last_error()
    opts = capi.PlanOpts(0, 512, 32, 256, 8, 64)
    tiles = (capi.Tile * 4)()
    rc = lib.esp_attn_plan(trees.ctypes.data_as(C.POINTER(capi.Tree)), 1, 2, C.byref(opts), tiles, 4, None, 0, C.byref(nt), C.byref(nj), C.byref(np_))
    assert rc == capi.ESP_ERR_CAPACITY and nt.value == 32


def test_window_planner_matches_restatement(oracle_lib):
    """esp_attn_plan_window against the restatement of g4_plan_tiles with its window branch
    (src/model/impl/gemma.h:77-116): same tiles (k0 at the first visible key, first batch key in pad0),
    jobs and tile height, bit for bit, for split and unsplit budgets."""
    from espetero_b200 import host
    rng = np.random.default_rng(9)
    for case in range(40):
        n_trees = int(rng.integers(1, 6))
        trees = np.zeros(n_trees, dtype=TREE_DT)
        base = tab = 0
        for i in range(n_trees):
            P, M = int(rng.integers(0, 5000)), int(rng.integers(1, 40))
            trees[i] = (base, P, tab, M)
            base += M
            tab += (P + 15) // 16
        pos = np.zeros((base, 4), dtype=np.int32)
        for t in trees:
            b0, P, M = int(t["base"]), int(t["P"]), int(t["M"])
            pos[b0:b0 + M, 0] = P + np.sort(rng.integers(0, M, size=M))     # tree rows: repeated depths
        window = int(rng.choice([0, 1, 17, 512, 1024, 100000]))
        groups = int(rng.choice([1, 2, 8, 32]))
        split = int(rng.choice([0, 256, 512]))
        rows = int(rng.choice([8, 16]))
        plan = host.plan_window(trees, groups, split, rows, window, pos)
        tiles, jobs, n_parts, plan_rows = oracle_lib.g4_plan_tiles(trees, groups, split, rows, window, pos)
        assert plan.tile_rows == plan_rows and plan.n_parts == n_parts
        assert plan.tiles.tobytes() == tiles.tobytes(), case
        assert plan.jobs.tobytes() == jobs.tobytes(), case
