"""Host-side pieces of bench.py that need no GPU: the workloads the flags select, their plans and the algorithmic
work the roofline figures are computed from (hand-counted on small cases)."""
import numpy as np

import bench
from espetero_b200 import workloads as wl


def test_flops_of_a_causal_prefill_and_of_its_windowed_variant():
    w = bench.build_workload("c3", 0, small=True)
    M = int(w.trees[0]["M"])
    assert bench.attention_flops(w) == 4.0 * (M * (M + 1) // 2) * w.H * w.HD
    ww = bench.build_workload("c3", 0, small=True, window=512)
    assert ww.name == "c3_causal_prefill_window" and ww.extra["window"]["window"] == 512
    pairs = sum(min(r + 1, 512) for r in range(M))
    assert bench.attention_flops(ww) == 4.0 * pairs * ww.H * ww.HD


def test_flops_of_a_tree_verify_count_ancestor_masks():
    w = bench.build_workload("c4", 0, small=True)
    vis = 0
    for t in w.trees:
        b, M, P = int(t["base"]), int(t["M"]), int(t["P"])
        vis += M * P + sum(bin(int(w.anc_mask[b + r])).count("1") for r in range(M))
    assert bench.attention_flops(w) == 4.0 * vis * w.H * w.HD


def test_window_workload_is_planned_with_tcgen05_sized_tiles():
    ww = bench.build_workload("c3", 0, small=True, window=512)
    plan = bench.bench_plan("c3", ww)
    assert plan.tile_rows == 128 and plan.n_parts == 0
    M = int(ww.trees[0]["M"])
    assert len(plan.tiles) == M // 128
    for i, t in enumerate(plan.tiles):      # no cached keys: the window shows in the first batch key to scan
        assert int(t["k0"]) == 0 and int(t["k1"]) == 0 and int(t["last"]) == 1
        assert int(t["pad0"]) == max(0, 128 * i - 512 + 1)


def test_the_fp8_variant_of_the_verify_workload():
    w = bench.build_workload("c4", 0, small=True, kv="e4m3")
    assert w.name == "c4_tree_verify_e4m3" and w.kv_dtype == wl.E4M3 and w.kv_elem_bytes == 1
    w16 = bench.build_workload("c4", 0, small=True)
    pages = sum((int(t["P"]) + w.bt - 1) // w.bt for t in w.trees)
    assert w16.name == "c4_tree_verify" and w.kv_bytes_read() == w16.kv_bytes_read() // 2 + pages * 2 * w.Hkv * 4   # codes + scales
    assert np.array_equal(w.trees[["P", "M"]], w16.trees[["P", "M"]])


def test_hd_flag_builds_the_256_dim_passes():
    """--hd 256: c3 / c4 with the reference kernels' own head dim; c3 keeps its flops (half the heads), c4 doubles its key bytes."""
    a, b = bench.build_workload("c3", 0, True), bench.build_workload("c3", 0, True, hd=256)
    assert (b.HD, b.H, b.Hkv) == (256, 32, 4) and b.name.endswith("_hd256")
    assert bench.attention_flops(a) == bench.attention_flops(b)
    a, b = bench.build_workload("c4", 0, True), bench.build_workload("c4", 0, True, hd=256)
    assert (b.HD, b.H, b.Hkv) == (256, 32, 4) and b.name == "c4_tree_verify_hd256"
    assert 2 * a.kv_bytes_read() == b.kv_bytes_read()


def test_decode_batch_variants():
    """--hd / --kv on the batched decode: the same sequences, another head dim or an E4M3 pool; bytes follow."""
    a = bench.build_workload("c2", 0, True)
    b = bench.build_workload("c2", 0, True, hd=512)
    c = bench.build_workload("c2", 0, True, kv="e4m3", hd=256)
    assert b.name == "c2_batched_decode_hd512" and c.name == "c2_batched_decode_hd256_e4m3"
    assert [int(t["P"]) for t in a.trees] == [int(t["P"]) for t in b.trees] == [int(t["P"]) for t in c.trees]
    assert b.kv_bytes_read() == 4 * a.kv_bytes_read()
    assert c.kv_dtype == wl.E4M3 and a.kv_bytes_read() <= c.kv_bytes_read() < 1.1 * a.kv_bytes_read()   # half the bytes per element, twice the dims, + scales
