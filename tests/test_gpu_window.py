"""Sliding-window layers of the generic attention kernel (kernels/80_gemma.metal:123-142, :250, :284-285;
planner src/model/impl/gemma.h:77-116) through the C ABI against the float64 oracle: window masks on cached
and batch keys, ring addressing of the cached keys, bidirectional image rows, and single-row (decode)
passes whose window lives in the plan (tiles start at the first visible key, at any alignment)."""
import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


def _run(w, plan, options=None):
    op = host.AttnOp.for_workload(w, plan.tile_rows)
    try:
        for k, v in (options or {}).items():
            op.set_option(k, v)
        dp = op.upload(w, plan)
        op.forward(dp)
        op.check_status()
        torch.cuda.synchronize()
        return dp.O.cpu().numpy().view(np.uint16), dp.lse.cpu().numpy(), op.last_kernel
    finally:
        op.close()


def _check(oracle_lib, w, plan, expect_kernel, options=None):
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    O, lse, kernel = _run(w, plan, options)
    assert kernel == expect_kernel
    util.check_output(O, ref, w, ref_abs=ref_abs, what=w.name)
    fin = np.isfinite(lse_ref)
    assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3
    return O


@pytest.mark.parametrize("HD", [128, 256])
@pytest.mark.parametrize("window", [64, 1000])
def test_window_masks_multi_row(oracle_lib, HD, window):
    """Chunked prefill / verify rows behind a cached prefix: the window cuts into the prefix for the late
    rows and into the batch keys for the early ones."""
    w = wl.make_window_pass("win", 21, [(700, 40), (30, 90), (0, 17)], 8, 2, HD, 16, wl.BF16, window, scale=HD ** -0.5)
    win = w.extra["window"]
    plan = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=8, window=window, pos=win["pos"])
    assert any(int(t["k0"]) % 16 for t in plan.tiles) or window >= 1000
    # (the harness mirrors the positions on the host, so the 8-row plan is planned again for the tcgen05 kernels -
    # test_reference_shaped_window_plans_reach_the_tensor_cores; option replan = 0 keeps the plan as given)
    _check(oracle_lib, w, plan, "flash_umma_duo" if HD == 128 else "flash_umma_pair")
    _check(oracle_lib, w, plan, "flash_general", options={"replan": 0})
    # the mask alone (no help from the plan): full-range tiles give the same answer
    full = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=8, window=0, pos=None)
    _check(oracle_lib, w, full, "flash_general", options={"replan": 0})


def test_window_changes_the_result(oracle_lib):
    """The same inputs with and without the window differ (the test above would pass on a kernel that
    ignores the window only if the oracle did too)."""
    w = wl.make_window_pass("win2", 22, [(600, 24)], 8, 2, 128, 16, wl.BF16, 50, scale=128 ** -0.5)
    plan = host.plan_window(w.trees, groups=w.Hkv, split=0, rows=8, window=0, pos=None)
    O_win = _check(oracle_lib, w, plan, "flash_general")
    w.extra.pop("window")
    O_all = _check(oracle_lib, w, plan, "flash_general", options={"replan": 0})  # an ordinary layer now: keep it on the same kernel
    assert not np.array_equal(O_win, O_all)


def test_ring_addressing_and_bidi_images(oracle_lib):
    """Cached keys in per-sequence rings (no page table) and image rows that see their whole image."""
    bt, ring = 16, 12
    w = wl.make_window_pass("ring", 23, [(150, 30), (100, 12)], 8, 2, 256, bt, wl.F16, 96, ring=ring, images={0: (5, 21)},
                            scale=256 ** -0.5)
    w.blocks[:] = -1                                   # the page table must not be read
    win = w.extra["window"]
    assert win["bidi"] == 1 and win["ring"] == ring
    plan = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=8, window=96, pos=win["pos"])
    _check(oracle_lib, w, plan, "flash_umma_pair")                            # planned again with 128-row tiles (positions mirrored)
    _check(oracle_lib, w, plan, "flash_general", options={"replan": 0})     # as given


@pytest.mark.parametrize("kvdt", [None, wl.E4M3], ids=["bf16", "fp8"])
@pytest.mark.parametrize("ring", [0, 80])
def test_window_decode_plan_starts_at_any_key(oracle_lib, kvdt, ring):
    """Single-row trees: the decode kernel applies no window mask, the plan starts each tile at the
    row's first visible key - here at every alignment modulo 16 - and splits the rest."""
    Ps = [1000 + i for i in range(17)] + [30, 1023, 1024, 1025, 5]
    window = 777
    bt = 16
    if ring:                                            # a ring must hold the window
        assert ring * bt >= window + bt
    w = wl.make_window_pass("windec", 24, [(P, 1) for P in Ps], 32, 4, 128, bt, wl.BF16, window, ring=ring, scale=128 ** -0.5,
                            kv_dtype=kvdt)
    win = w.extra["window"]
    plan = host.plan_window(w.trees, groups=w.Hkv, split=256, rows=8, window=window, pos=win["pos"])
    starts = {int(t["k0"]) % 16 for t in plan.tiles}
    assert len(starts) >= 12
    assert plan.n_parts > 0
    _check(oracle_lib, w, plan, "decode_gqa")


def test_window_needs_positions():
    w = wl.make_window_pass("winv", 25, [(100, 4)], 8, 2, 128, 16, wl.BF16, 32)
    plan = host.plan_window(w.trees, groups=w.Hkv, split=0, rows=8, window=32, pos=w.extra["window"]["pos"])
    op = host.AttnOp.for_workload(w, plan.tile_rows)
    try:
        dp = op.upload(w, plan)
        a = op.make_args(dp)
        a.pos = None
        with pytest.raises(capi.EspError) as e:
            op.forward(dp, a)
        assert e.value.code == capi.ESP_ERR_INVALID
    finally:
        op.close()


@pytest.mark.parametrize("HD", [128, 256])
@pytest.mark.parametrize("case", ["prefill", "chunked", "chunked_f16", "ring", "positions_with_gaps", "images", "rows64"])
def test_window_layers_on_the_tensor_cores(oracle_lib, case, HD):
    """Sliding-window passes planned with tcgen05-sized tiles (esp_attn_plan_window, rows = 128: the generic planner
    gives its caller's tile height to passes of 256 row groups x kv heads or more) run on flash_umma_duo (128-dim heads)
    or flash_umma_pair (256-dim heads, the sliding layers of kernels/80_gemma.metal): window edge
    inside cached blocks (tiles start at unaligned keys), inside batch blocks (per-key positions), ring addressing,
    batch blocks below the window skipped, image rows that see their whole image. Against the float64 oracle and against the general kernel on an 8-row plan."""
    rows = 128
    if case == "prefill":
        w = wl.make_window_pass("winp", 31, [(0, 1500), (0, 700)], 8, 2, HD, 16, wl.BF16, 300, scale=HD ** -0.5)
    elif case == "chunked":
        w = wl.make_window_pass("winc", 32, [(1234, 600), (77, 900)], 8, 2, HD, 16, wl.BF16, 517, scale=HD ** -0.5)
    elif case == "chunked_f16":
        w = wl.make_window_pass("wing", 33, [(2000, 1100)], 16, 4, HD, 16, wl.F16, 1024, scale=HD ** -0.5)
    elif case == "rows64":
        # 64-row tiles: a query tile is 64 rows x 2 heads, a CTA covers 4 heads of the kv group
        w = wl.make_window_pass("win64", 37, [(500, 2100)], 8, 2, HD, 16, wl.BF16, 700, scale=HD ** -0.5)
        rows = 64
    elif case == "images":
        # rows 100..419 and 600..700 are images: their rows see the whole image (blocks beyond the diagonal)
        w = wl.make_window_pass("wini", 36, [(200, 900), (0, 300)], 8, 2, HD, 16, wl.BF16, 4096, images={0: (100, 420), 1: (130, 290)},
                                scale=HD ** -0.5)
    elif case == "ring":
        w = wl.make_window_pass("winr", 34, [(640, 1300)], 8, 2, HD, 16, wl.BF16, 256, ring=48, scale=HD ** -0.5)
        w.blocks[:] = -1                               # the page table must not be read
    else:
        # positions that are not the row index plus P (the later rows sit 100 positions earlier than their index says):
        # the window mask of a batch block comes from the keys' own positions. (Positions may lag behind P + j, never
        # run ahead of it: the planner's first batch key, gemma.h:89-94, assumes no key is later than that.)
        w = wl.make_window_pass("winj", 35, [(300, 1400)], 8, 2, HD, 16, wl.BF16, 350, scale=HD ** -0.5)
        pos = w.extra["window"]["pos"]
        pos[700:, 0:3] -= 100
    win = w.extra["window"]
    plan = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=rows, window=win["window"], pos=win["pos"])
    assert plan.tile_rows == rows
    if case not in ("positions_with_gaps", "images"):
        assert any(int(t["k0"]) % 16 for t in plan.tiles) or any(int(t["pad0"]) > 0 for t in plan.tiles)
    O = _check(oracle_lib, w, plan, "flash_umma_duo" if HD == 128 else "flash_umma_pair")
    small = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=8, window=win["window"], pos=win["pos"])
    O8 = _check(oracle_lib, w, small, "flash_general", options={"replan": 0})
    a, b = wl.from_bits16(O, w.q_dtype), wl.from_bits16(O8, w.q_dtype)
    assert (np.abs(a - b) <= 2 * util.TOL_16 + 2.0 ** -7 * np.abs(b)).all()   # two roundings to the output type: one ulp


@pytest.mark.parametrize("HD", [128, 256])
def test_window_prefill_from_position_zero_ignores_the_pool_type(oracle_lib, HD):
    """A sliding-window prefill with no cached keys over an E4M3 pool never reads the pool: tcgen05 kernel, no scratch."""
    w = wl.make_window_pass("winfp8", 51, [(0, 1500), (0, 400)], 8, 2, HD, 16, wl.BF16, 300, scale=HD ** -0.5, kv_dtype=wl.E4M3)
    win = w.extra["window"]
    plan = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=128, window=win["window"], pos=win["pos"])
    _check(oracle_lib, w, plan, "flash_umma_duo" if HD == 128 else "flash_umma_pair")


@pytest.mark.parametrize("HD", [128, 256])
@pytest.mark.parametrize("case", ["prefill", "chunked_ring"])
def test_reference_shaped_window_plans_reach_the_tensor_cores(oracle_lib, case, HD):
    """A drop-in caller plans a sliding-window layer the reference's way (g4_plan_tiles, gemma.h:77-116: 8-row tiles) on
    a context with tile_rows 8. With the host mirror of the positions (pos_host) the library plans the pass again with
    128-row tiles and runs the tcgen05 kernel; without it the pass runs on the general kernel as given. Same results."""
    if case == "prefill":
        w = wl.make_window_pass("win8", 41, [(0, 1500), (0, 900)], 8, 2, HD, 16, wl.BF16, 300, scale=HD ** -0.5)
    else:
        w = wl.make_window_pass("win8r", 42, [(640, 1300)], 8, 2, HD, 16, wl.BF16, 256, ring=48, scale=HD ** -0.5)
        w.blocks[:] = -1
    win = w.extra["window"]
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    plan = host.plan_window(w.trees, groups=w.Hkv, split=512, rows=8, window=win["window"], pos=win["pos"])
    assert plan.tile_rows == 8
    op = host.AttnOp.for_workload(w, 8)
    try:
        dp = op.upload(w, plan)
        tiles_before = dp.tiles.clone()
        for _ in range(6):                                   # several passes reuse the staging slots
            op.forward(dp)
        op.check_status()
        assert op.last_kernel == ("flash_umma_duo" if HD == 128 else "flash_umma_pair"), "a reference-shaped window plan fell onto the CUDA-core kernel"
        assert torch.equal(dp.tiles, tiles_before)           # the caller's plan is read, never written
        O = dp.O.cpu().numpy().view(np.uint16).copy()
        util.check_output(O, ref, w, ref_abs=ref_abs, what=case)
        a = op.make_args(dp)
        a.pos_host = None                                     # no mirror: as given, on the general kernel
        dp.O.zero_()
        op.forward(dp, a)
        op.check_status()
        assert op.last_kernel == "flash_general"
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what=case + "/general")
    finally:
        op.close()
