"""Parity of the tcgen05 kernels (flash_umma: one CTA per SM, 128-key blocks, deep rings;
flash_umma_pair: two CTAs per SM, 64-key blocks; flash_umma_duo: one CTA per SM with two query
tiles against 128-key blocks, where two tiles' heads share a kv head; all with TMEM
accumulators) with the float64 oracle, through the C ABI; every case runs on each: tree verify (16-row tiles x 8 heads), causal prefill
(128-row tiles), forest masks, chunked prefill over a cached prefix, split-K records + combine,
and integer-exact mask probes."""
import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu

KERNELS = {1: "flash_umma", 2: "flash_umma_pair"}


def _duo_or_pair(w, tile_rows):
    """What option umma_kernel = 3 runs: flash_umma_duo when the 2 * (128 / tile_rows) heads of a CTA fit one kv head."""
    G, hpc2 = w.H // w.Hkv, 2 * (128 // tile_rows)
    return "flash_umma_duo" if w.HD == 128 and hpc2 <= G and G % hpc2 == 0 else "flash_umma_pair"


def _check(oracle_lib, w, tile_rows, mode=capi.ESP_PLAN_REFERENCE, groups=256, split=512, with_abs=True):
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    plan = None
    for opt, name in list(KERNELS.items()) + [(3, _duo_or_pair(w, tile_rows))]:
        O, lse, parts, plan, kernel = host.run_pass(w, mode=mode, tile_rows=tile_rows, split=split, groups=groups,
                                                    options={"umma_kernel": opt})
        assert kernel == name
        util.check_output(O, ref, w, ref_abs=ref_abs if with_abs else None, what=f"{w.name}/{name}")
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3
    return plan


def test_verify_tile_16x8(oracle_lib):
    w = wl.config_c4(n_seqs=3, prefix=1024)
    plan = _check(oracle_lib, w, 16, with_abs=False)
    assert plan.n_parts > 0  # few tiles: the prefix is split and combined


def test_verify_b200_plan_unsplit_and_split(oracle_lib):
    w = wl.config_c4(n_seqs=2, prefix=2000)  # prefix not a multiple of 64: tail block
    _check(oracle_lib, w, 16, mode=capi.ESP_PLAN_B200, groups=8, split=1 << 20, with_abs=False)     # unsplit
    _check(oracle_lib, w, 16, mode=capi.ESP_PLAN_B200, groups=592, split=1 << 20, with_abs=False)   # split


@pytest.mark.parametrize("rows", [128, 300, 5])
def test_causal_prefill(oracle_lib, rows):
    w = wl.config_c3(n_seqs=2, rows=rows)
    _check(oracle_lib, w, 128)


def test_prefill_f16_and_gate(oracle_lib):
    w = wl.make_pass("prefill_f16", 71, [(0, 200), (0, 129)], 8, 2, 128, 16, wl.F16, gate=True)
    _check(oracle_lib, w, 128)


def test_chunked_prefill_over_cached_prefix(oracle_lib):
    w = wl.make_pass("chunked", 72, [(300, 150), (1000, 64), (37, 1)], 8, 4, 128, 16, wl.BF16)
    _check(oracle_lib, w, 128)


@pytest.mark.parametrize("mask", ["forest", "tree"])
@pytest.mark.parametrize("tr,H,Hkv", [(128, 8, 2), (16, 16, 2), (32, 8, 2), (64, 4, 2)])
def test_masks_and_tile_shapes(oracle_lib, mask, tr, H, Hkv):
    w = wl.make_pass("masks", 73 + tr, [(40, 20), (0, 9), (100, 16), (33, 1), (200, 50)], H, Hkv, 128, 16, wl.BF16, mask=mask)
    _check(oracle_lib, w, tr)


def test_records_match_f64_without_rounding(oracle_lib):
    w = wl.config_c4(n_seqs=2, prefix=512)
    ref, lse_ref = oracle_lib.attention_f64(w)
    for opt, name in KERNELS.items():
        O, lse, parts, plan, kernel = host.run_pass(w, tile_rows=16, force_parts=True, options={"umma_kernel": opt})
        assert kernel == name
        O64, lse64 = util.records_to_output(parts, w, plan.tiles, plan.jobs, 16)
        assert np.abs(O64 - ref).max() <= util.TOL_16
        assert np.abs(lse64 - lse_ref).max() < 1e-3


@pytest.mark.parametrize("umma_kernel", [1, 2], ids=["stream", "pair"])
def test_tree_mask_probe_is_exact_on_tensor_cores(umma_kernel):
    """Q = 0 and one-hot V rows: the fp32 record of node n must hold exactly its ancestor set and
    exact integer sums of the prefix codes (P = 1.0 exactly in bf16, fp32 accumulation in TMEM)."""
    P, M, H, Hkv, HD, bt = 200, 16, 16, 2, 128, 16
    w = wl.make_pass("umma_probe", 74, [(P, M), (0, M)], H, Hkv, HD, bt, wl.BF16, mask="tree")
    w.Q[:] = 0
    pool = np.full((w.n_blocks, 2, bt, Hkv, HD), 3.0, dtype=np.float32)  # poison
    for j in range(P):
        b = int(w.blocks[j // bt])
        pool[b, 1, j % bt] = 0
        for kvh in range(Hkv):
            pool[b, 1, j % bt, kvh, 64:68] = [j % 16, (j // 16) % 16, kvh + 1, 1]
    w.kv = wl.f32_to_bf16_bits(pool.reshape(-1))
    vb = np.zeros((w.n_rows, Hkv, HD), dtype=np.float32)
    for r in range(w.n_rows):
        vb[r, :, r % M] = 1.0
    w.Vb = wl.f32_to_bf16_bits(vb.reshape(w.n_rows, -1))
    O, lse, parts, plan, kernel = host.run_pass(w, tile_rows=16, force_parts=True, split=0, options={"umma_kernel": umma_kernel})
    assert kernel == KERNELS[umma_kernel]
    G = w.G
    rec = parts[: plan.n_parts * Hkv * 16 * G * (HD + 2)].reshape(plan.n_parts, Hkv, 16, G, HD + 2)
    for t in plan.tiles:
        ti, part = int(t["tree"]), int(t["part"])
        par = w.extra["parents"][ti]
        Pt = int(w.trees[ti]["P"])
        for node in range(M):
            anc, k = set(), node
            while k >= 0:
                anc.add(k)
                k = par[k]
            r = rec[part, :, node]
            assert np.all(r[..., HD] == 0.0)
            assert np.all(r[..., HD + 1] == Pt + len(anc))
            want = np.array([1.0 if n in anc else 0.0 for n in range(M)], dtype=np.float32)
            assert np.all(r[..., :M] == want)
            if Pt:
                js = np.arange(Pt)
                for kvh in range(Hkv):
                    assert np.all(r[kvh, :, 64] == (js % 16).sum()) and np.all(r[kvh, :, 65] == ((js // 16) % 16).sum())
                    assert np.all(r[kvh, :, 66] == (kvh + 1) * Pt) and np.all(r[kvh, :, 67] == Pt)


@pytest.mark.parametrize("gate", [False, True], ids=["plain", "gate"])
def test_fused_merge_matches_separate_combine(oracle_lib, gate):
    """Small split passes of flash_umma merge their records in the attention kernel (the CTA that
    finishes last for a job merges in record order) instead of launching attention_combine. Same
    arithmetic (the two routes may add the records' terms in a different order): the outputs
    must agree to one output ulp with the two-kernel route, repeat bit for bit from pass to pass
    (the arrival counters reset themselves; no result depends on which CTA came last), and match
    the oracle."""
    w = wl.make_pass("fused", 77, [(1500, 16), (777, 16), (2100, 9)], 32, 4, 128, 16, wl.BF16, mask="tree", gate=gate)
    ref, lse_ref = oracle_lib.attention_f64(w)
    outs = {}
    for fuse in (1, 0):
        op = host.AttnOp.for_workload(w, 16)
        try:
            op.set_option("umma_kernel", 1)
            op.set_option("fuse_combine", fuse)
            plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 24, 16)
            assert plan.n_parts > 0 and len(plan.tiles) <= 48
            dp = op.upload(w, plan)
            n0 = op.launch_count
            seen = []
            for _ in range(3):
                dp.O.zero_()
                op.forward(dp)
                op.check_status()
                seen.append(dp.O.cpu().numpy().view(np.uint16).copy())
            assert np.array_equal(seen[0], seen[1]) and np.array_equal(seen[0], seen[2])
            assert op.last_kernel == "flash_umma"
            assert op.launch_count - n0 == (3 if fuse else 6)   # one kernel per pass when fused
            outs[fuse] = (dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy())
        finally:
            op.close()
    fa, fb = wl.from_bits16(outs[1][0], w.q_dtype), wl.from_bits16(outs[0][0], w.q_dtype)
    assert np.all(np.abs(fa - fb) <= 2.0 ** -7 * np.maximum(np.abs(fa), np.abs(fb)) + 1e-30)
    assert np.abs(outs[1][1] - outs[0][1]).max() < 1e-5
    util.check_output(outs[1][0], ref, w)
    assert np.abs(outs[1][1] - lse_ref).max() < 2e-3


@pytest.mark.parametrize("case", ["prefill", "verify", "chunked_gate_f16", "forest"])
def test_hd512_on_tensor_cores(oracle_lib, case):
    """512-dim heads (the global layers of kernels/80_gemma.metal, src/model/impl/gemma.h:119-147) on the tcgen05 kernel:
    two CTAs per tile, each with one 256-dim half of the output and the whole 512-dim scores."""
    if case == "prefill":
        w, tr = wl.make_pass("hd512_prefill", 111, [(0, 300), (0, 77)], 4, 2, 512, 16, wl.BF16), 128
    elif case == "verify":
        w, tr = wl.make_pass("hd512_verify", 112, [(1000, 16), (333, 16), (64, 9)], 16, 2, 512, 16, wl.BF16, mask="tree"), 16
    elif case == "chunked_gate_f16":
        w, tr = wl.make_pass("hd512_chunk", 113, [(500, 200)], 4, 2, 512, 16, wl.F16, gate=True), 128
    else:
        w, tr = wl.make_pass("hd512_forest", 114, [(70, 40), (0, 33)], 8, 2, 512, 16, wl.BF16, mask="forest"), 32
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    for groups in (8, 592):                                  # unsplit, and split with records + merge
        O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_B200, tile_rows=tr, split=1 << 20, groups=groups)
        assert kernel == "flash_umma_pair"
        util.check_output(O, ref, w, ref_abs=ref_abs, what=f"{w.name}/g{groups}")
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3


@pytest.mark.parametrize("case", ["prefill", "verify", "chunked_gate_f16", "forest"])
def test_hd64_on_tensor_cores(oracle_lib, case):
    """64-dim heads (kernels/90_lfm2.metal:160-161) on the tcgen05 kernel: one 64-dim chunk per row, two CTAs per SM."""
    if case == "prefill":
        w, tr = wl.make_pass("hd64_prefill", 81, [(0, 300), (0, 77)], 8, 2, 64, 16, wl.BF16), 128
    elif case == "verify":
        w, tr = wl.make_pass("hd64_verify", 82, [(1000, 16), (333, 16), (64, 9)], 32, 4, 64, 16, wl.BF16, mask="tree"), 16
    elif case == "chunked_gate_f16":
        w, tr = wl.make_pass("hd64_chunk", 83, [(500, 200)], 8, 2, 64, 16, wl.F16, gate=True), 128
    else:
        w, tr = wl.make_pass("hd64_forest", 84, [(70, 40), (0, 33)], 8, 2, 64, 16, wl.BF16, mask="forest"), 32
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    for groups in (8, 592):                                  # unsplit, and split with records + merge
        O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_B200, tile_rows=tr, split=1 << 20, groups=groups)
        assert kernel == "flash_umma_pair"
        util.check_output(O, ref, w, ref_abs=ref_abs, what=f"{w.name}/g{groups}")
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3


@pytest.mark.parametrize("gate,dt", [(False, wl.BF16), (True, wl.F16)], ids=["bf16", "f16_gate"])
def test_hd256_verify_merges_inside_the_kernel(oracle_lib, gate, dt):
    """256-dim verify passes of one wave (flash_umma_pair, tiles of 16 rows x 8 heads): the CTA that draws the last
    ticket of a (job, kv head) folds the job's records in record order and writes the rows - one launch per pass.
    Same contract as the two-kernel route: agreement to one output ulp, bit-identical repeats, and the oracle."""
    w = wl.make_pass("fused256", 78, [(1500, 16), (777, 16), (2100, 9)], 32, 4, 256, 16, dt, mask="tree", gate=gate)
    ref, lse_ref = oracle_lib.attention_f64(w)
    outs = {}
    for fuse in (1, 0):
        op = host.AttnOp.for_workload(w, 16)
        try:
            op.set_option("fuse_combine", fuse)
            plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 28, 16)
            assert plan.n_parts > 0 and len(plan.tiles) * w.Hkv <= 148
            assert max(int(j["nparts"]) for j in plan.jobs) >= 3      # more than a pair: the fold runs over several records
            dp = op.upload(w, plan)
            n0 = op.launch_count
            seen = []
            for _ in range(3):
                dp.O.zero_()
                op.forward(dp)
                op.check_status()
                seen.append(dp.O.cpu().numpy().view(np.uint16).copy())
            assert np.array_equal(seen[0], seen[1]) and np.array_equal(seen[0], seen[2])
            assert op.last_kernel == "flash_umma_pair"
            assert op.launch_count - n0 == (3 if fuse else 6)
            outs[fuse] = (dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy())
        finally:
            op.close()
    fa, fb = wl.from_bits16(outs[1][0], w.q_dtype), wl.from_bits16(outs[0][0], w.q_dtype)
    ulp = 2.0 ** -7 if dt == wl.BF16 else 2.0 ** -10
    assert np.all(np.abs(fa - fb) <= ulp * np.maximum(np.abs(fa), np.abs(fb)) + 1e-30)
    assert np.abs(outs[1][1] - outs[0][1]).max() < 1e-5
    util.check_output(outs[1][0], ref, w)
    assert np.abs(outs[1][1] - lse_ref).max() < 2e-3


@pytest.mark.parametrize("case", ["prefill", "verify", "chunked_gate_f16", "forest"])
def test_hd256_on_tensor_cores(oracle_lib, case):
    """256-dim heads (the head dim of the reference's flash_attention, kernels/40_attention.metal:156)
    on the tcgen05 kernel: one CTA per SM, four 64-dim chunks per row, a 256-column accumulator."""
    if case == "prefill":
        w, tr = wl.make_pass("hd256_prefill", 91, [(0, 300), (0, 77)], 8, 2, 256, 16, wl.BF16), 128
    elif case == "verify":
        w, tr = wl.make_pass("hd256_verify", 92, [(1000, 16), (333, 16), (64, 9)], 32, 4, 256, 16, wl.BF16, mask="tree"), 16
    elif case == "chunked_gate_f16":
        w, tr = wl.make_pass("hd256_chunk", 93, [(500, 200)], 8, 2, 256, 16, wl.F16, gate=True), 128
    else:
        w, tr = wl.make_pass("hd256_forest", 94, [(70, 40), (0, 33)], 8, 2, 256, 16, wl.BF16, mask="forest"), 32
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    # unsplit; split with records + merge; split with the merge forced into the kernel whatever the number of CTAs
    for groups, options in ((8, None), (592, None), (592, {"fuse_combine": 2})):
        O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_B200, tile_rows=tr, split=1 << 20, groups=groups, options=options)
        assert kernel == "flash_umma_pair"
        util.check_output(O, ref, w, ref_abs=ref_abs, what=f"{w.name}/g{groups}")
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3


@pytest.mark.parametrize("case", ["verify128", "verify128_f16", "verify256", "verify256_bf16", "chunked_prefill"])
def test_e4m3_pool_on_tensor_cores(oracle_lib, case):
    """Multi-row passes over an E4M3 pool. Mostly cached keys: flash_umma (128-dim heads) and flash_umma_pair (256-dim
    heads) read the codes themselves
    (raw pages by TMA, converter warps, fp16 MMAs; option fp8_direct, default on) - no scratch needed. Otherwise, and
    with fp8_direct = 0: with the caller's scratch the blocks of the pass are widened to the 16-bit type (code * scale)
    and the tcgen05 kernels run on that copy; without scratch the pass runs on the general kernel. All within the E4M3
    tolerance of the oracle, which reads the codes."""
    if case == "verify128":
        w, tr = wl.make_pass("fp8_v128", 95, [(1500, 16), (333, 16), (70, 5)], 32, 4, 128, 16, wl.BF16, wl.E4M3, mask="tree"), 16
    elif case == "verify128_f16":
        w, tr = wl.make_pass("fp8_v128h", 98, [(2100, 16), (128, 16), (15, 3)], 16, 2, 128, 16, wl.F16, wl.E4M3, mask="tree"), 16
    elif case == "verify256":
        w, tr = wl.make_pass("fp8_v256", 96, [(900, 16), (200, 16)], 32, 8, 256, 16, wl.F16, wl.E4M3, mask="tree"), 32
    elif case == "verify256_bf16":   # 16 rows x 8 heads, a ragged tree, prefixes that end inside a page and inside a block
        w, tr = wl.make_pass("fp8_v256b", 99, [(1500, 16), (333, 16), (70, 5)], 32, 4, 256, 16, wl.BF16, wl.E4M3, mask="tree", gate=True), 16
    else:
        w, tr = wl.make_pass("fp8_chunk", 97, [(700, 150)], 8, 2, 128, 16, wl.BF16, wl.E4M3, gate=True), 128
    direct_ok = True
    direct_kernel = "flash_umma" if w.HD == 128 else "flash_umma_pair"
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    for groups in (8, 592):
        op = host.AttnOp.for_workload(w, tr)
        try:
            plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, groups, tr)
            dp = op.upload(w, plan)
            assert dp.scratch is not None
            for direct in ((1, 0) if direct_ok else (0,)):
                op.set_option("fp8_direct", direct)
                dp.O.zero_()
                op.forward(dp)
                op.check_status()
                assert op.last_kernel == (direct_kernel if direct else op.last_kernel)
                assert op.last_kernel in ("flash_umma", "flash_umma_pair", "flash_umma_duo")
                O, lse = dp.O.cpu().numpy().view(np.uint16), dp.lse.cpu().numpy()
                util.check_output(O, ref, w, ref_abs=ref_abs, what=f"{w.name}/g{groups}/direct{direct}")
                assert np.abs(lse - lse_ref).max() < 1e-2
            a = op.make_args(dp)
            a.dequant_scratch, a.dequant_scratch_bytes = None, 0          # no scratch
            for direct in ((1, 0) if direct_ok else (0,)):
                op.set_option("fp8_direct", direct)
                dp.O.zero_()
                op.forward(dp, a)
                op.check_status()
                assert op.last_kernel == (direct_kernel if direct else "flash_general")
                util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what=f"{w.name}/noscratch/direct{direct}")
        finally:
            op.close()


@pytest.mark.parametrize("HD,expect", [(128, "flash_umma"), (256, "flash_umma_pair")])
def test_chunked_prefill_over_few_e4m3_keys_without_scratch(oracle_lib, HD, expect):
    """A pass over mostly its own rows behind a short E4M3 prefix: with scratch it widens the prefix and runs the 16-bit
    kernels; without scratch the tcgen05 kernels read the codes themselves (batch keys through the converter warps)
    rather than falling onto the CUDA-core kernel."""
    w = wl.make_pass("fp8_short", 102, [(100, 400), (37, 130)], 8, 2, HD, 16, wl.BF16, wl.E4M3)
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    op = host.AttnOp.for_workload(w, 128)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 8, 128)
        dp = op.upload(w, plan)
        op.forward(dp)                                       # with the scratch
        op.check_status()
        assert op.last_kernel in ("flash_umma_duo", "flash_umma_pair")
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what="fp8_short/widened")
        a = op.make_args(dp)
        a.dequant_scratch, a.dequant_scratch_bytes = None, 0
        dp.O.zero_()
        n0 = op.launch_count
        op.forward(dp, a)
        op.check_status()
        assert op.last_kernel == expect and op.launch_count - n0 == 1
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what="fp8_short/direct")
        assert np.abs(dp.lse.cpu().numpy() - lse_ref).max() < 1e-2
    finally:
        op.close()


@pytest.mark.parametrize("HD,expect", [(128, "flash_umma_duo"), (256, "flash_umma_pair")])
def test_prefill_from_position_zero_ignores_the_pool_type(oracle_lib, HD, expect):
    """A prefill with no cached keys over an E4M3 pool reads nothing from the pool: it runs on the tcgen05 kernels as over
    a 16-bit pool - no scratch, no widening pass, one launch."""
    w = wl.make_pass("fp8_prefill", 101, [(0, 300), (0, 130)], 8, 2, HD, 16, wl.BF16, wl.E4M3)
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    op = host.AttnOp.for_workload(w, 128)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 8, 128)
        dp = op.upload(w, plan)
        a = op.make_args(dp)
        a.dequant_scratch, a.dequant_scratch_bytes = None, 0
        n0 = op.launch_count
        op.forward(dp, a)
        op.check_status()
        assert op.last_kernel == expect and op.launch_count - n0 == 1
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what="fp8_prefill")
        assert np.abs(dp.lse.cpu().numpy() - lse_ref).max() < 2e-3
    finally:
        op.close()


@pytest.mark.parametrize("case", ["prefill", "verify", "chunked", "ragged"])
def test_reference_shaped_plans_reach_the_tensor_cores(oracle_lib, case):
    """A drop-in caller plans the reference's way: a context with 8-row tiles and plan_tiles
    (src/model/impl/forest.h:1378-1433). Such a plan is plain full attention, so the library plans the
    pass again for the tcgen05 kernels; it must not fall onto the CUDA-core kernel, and O / lse must be
    the same results (against the float64 oracle, and against the general kernel on the caller's own plan)."""
    if case == "prefill":
        w = wl.config_c3(n_seqs=2, rows=1024)               # M = 1024, HD 128: 256 unsplit 8-row tiles
        expect = "flash_umma_duo"
    elif case == "verify":
        w = wl.config_c4(n_seqs=4, prefix=2048)             # split by the reference planner: records + combine
        expect = "flash_umma"
    elif case == "chunked":
        w = wl.make_pass("chunk", 501, [(900, 200), (64, 77)], 16, 4, 128, 16, wl.BF16, gate=True)
        expect = None
    else:
        w = wl.make_pass("ragged", 502, [(300, 13), (0, 3), (1000, 16), (17, 9)], 32, 4, 128, 16, wl.F16, mask="forest")
        expect = None
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    op = host.AttnOp.for_workload(w, 8)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_REFERENCE)
        assert plan.tile_rows == 8
        if case == "verify":
            assert plan.n_parts > 0
        dp = op.upload(w, plan)
        tiles_before = dp.tiles.clone()
        op.forward(dp)
        op.check_status()
        torch.cuda.synchronize()
        assert op.last_kernel != "flash_general", "a reference-shaped plan fell onto the CUDA-core kernel"
        if expect:
            assert op.last_kernel == expect
        assert torch.equal(dp.tiles, tiles_before)          # the caller's plan is read, never written
        O, lse = dp.O.cpu().numpy().view(np.uint16), dp.lse.cpu().numpy()
        util.check_output(O, ref, w, ref_abs=ref_abs, what=case)
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3
        # several passes in a row reuse the staging slots
        for _ in range(6):
            op.forward(dp)
        op.check_status()
        torch.cuda.synchronize()
        assert np.array_equal(dp.O.cpu().numpy().view(np.uint16), O)
        # the same plan with re-planning off runs as given, on the general kernel
        op.set_option("replan", 0)
        dp.O.zero_()
        op.forward(dp)
        op.check_status()
        assert op.last_kernel == "flash_general"
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, ref_abs=ref_abs, what=case + "/general")
    finally:
        op.close()


def test_records_only_plans_are_not_replanned():
    """Tiles whose records no job of the pass merges (the first level of a multi-GPU merge) are results
    of the pass in the caller's layout: such a plan runs as given."""
    w = wl.config_c4(n_seqs=2, prefix=512)
    op = host.AttnOp.for_workload(w, 8)
    try:
        plan = host.force_partial_records(host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_REFERENCE, split=0), w.trees)
        plan = host.Plan(plan.tiles, np.zeros(0, dtype=wl.COMBINE_DT), plan.n_parts, 8)
        dp = op.upload(w, plan)
        op.forward(dp)
        op.check_status()
        assert op.last_kernel == "flash_general"
    finally:
        op.close()


@pytest.mark.parametrize("gate", [False, True], ids=["plain", "gate"])
def test_two_record_jobs_merge_inside_a_cluster_pair(oracle_lib, gate):
    """A verify pass whose every row group is split in two: the two CTAs of a job run as a thread-block cluster and
    merge through distributed shared memory (option pair_merge, on by default) - one launch, nothing written to
    `parts`. Same results as the ticket merge through global memory (pair_merge 0) and as the combine kernel
    (fuse_combine 0), all within tolerance of the float64 oracle; rows of short trees and an odd tree out included."""
    trees = [(2048, 16), (1500, 16), (2048, 7), (2048, 16)]
    w = wl.make_pass("pairs", 601, trees, 32, 4, 128, 16, wl.BF16, mask="tree", gate=gate)
    ref, lse_ref = oracle_lib.attention_f64(w)
    outs = {}
    for name, options in (("pair", {}), ("ticket", {"pair_merge": 0}), ("combine", {"fuse_combine": 0})):
        op = host.AttnOp.for_workload(w, 16)
        try:
            for k, v in options.items():
                op.set_option(k, v)
            plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1024, 32, 32, 16)
            assert len(plan.tiles) == 8 and all(int(j["nparts"]) == 2 for j in plan.jobs)
            dp = op.upload(w, plan)
            dp.parts.fill_(-7.0)
            n0 = op.launch_count
            op.forward(dp)
            op.check_status()
            torch.cuda.synchronize()
            assert op.last_kernel == "flash_umma" and op.launch_count - n0 == (2 if name == "combine" else 1)
            if name == "pair":
                assert bool((dp.parts == -7.0).all()), "the pair merge wrote records to global memory"
            O, lse = dp.O.cpu().numpy().view(np.uint16), dp.lse.cpu().numpy()
            util.check_output(O, ref, w, what=name)
            assert np.abs(lse - lse_ref).max() < 2e-3
            outs[name] = wl.from_bits16(O, w.q_dtype)
            for _ in range(3):                               # back to back on the same context
                op.forward(dp)
            op.check_status()
            assert np.array_equal(dp.O.cpu().numpy().view(np.uint16), O)
        finally:
            op.close()
    assert np.abs(outs["pair"] - outs["ticket"]).max() <= 2.0 ** -7 * np.abs(outs["pair"]).max()
    assert np.abs(outs["pair"] - outs["combine"]).max() <= 2.0 ** -7 * np.abs(outs["pair"]).max()


@pytest.mark.parametrize("umma_kernel", [1, 2, 3], ids=["stream", "pair", "duo"])
def test_prefill_records_meet_the_plain_tolerance(oracle_lib, umma_kernel):
    """A causal prefill tile forced to write its fp32 records (no rounding of the output). Against the float64 oracle
    every element stays within the rigorous bound on rounding P to bf16, 2e-3 + 2^-9 * sum_j p_j |v_j| (the reference
    rounds P too, to fp16, kernels/40_attention.metal:297); beyond the first 128 rows, where a row averages over more
    than a block of keys, all but a handful of elements (a peaked row whose dominant p rounds badly: fewer than 1 in
    10 000) meet the plain 2e-3, and the share and the last such row are printed."""
    w = wl.config_c3(n_seqs=1, rows=512)
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_B200, tile_rows=128, force_parts=True, split=0, groups=592,
                                                options={"umma_kernel": umma_kernel})
    assert kernel == (KERNELS[umma_kernel] if umma_kernel in KERNELS else "flash_umma_duo")
    O64, lse64 = util.records_to_output(parts, w, plan.tiles, plan.jobs, 128)
    err = np.abs(O64 - ref)
    assert (err <= util.TOL_16 + 2.0 ** -9 * ref_abs).all()
    late = (err[128:] > util.TOL_16).mean()
    assert late < 1e-4, f"rows with 129+ keys: {late:.2e} of the elements beyond plain 2e-3, max abs err {err[128:].max():.3e}"
    assert np.abs(lse64 - lse_ref).max() < 1e-3
    over = (err > util.TOL_16).any(axis=1)
    print(f"prefill records ({kernel}): {(err > util.TOL_16).mean():.2e} of the elements beyond plain 2e-3, the last such row is {int(np.flatnonzero(over).max()) if over.any() else -1}")


@pytest.mark.parametrize("kv", [None, wl.E4M3], ids=["bf16", "fp8"])
def test_stable_cache_option_gives_the_same_results(oracle_lib, kv):
    """Option stable_cache lets the verify kernel fetch cached key blocks before the previous kernel of the stream has
    completed; with a pool nobody writes between the passes the results are those of the default order, pass after pass
    (several passes back to back on one stream, so that the early fetches do overlap a running kernel)."""
    w = wl.make_pass("stable", 99, [(3000, 16), (1500, 16), (700, 9)], 32, 4, 128, 16, wl.BF16, kv, mask="tree")
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    op = host.AttnOp.for_workload(w, 16)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 148, 16)
        dp = op.upload(w, plan)
        outs = {}
        for stable in (0, 1):
            op.set_option("stable_cache", stable)
            for _ in range(6):
                op.forward(dp)
            op.check_status()
            assert op.last_kernel == "flash_umma"
            outs[stable] = dp.O.cpu().numpy().view(np.uint16).copy()
            util.check_output(outs[stable], ref, w, ref_abs=ref_abs, what=f"stable_cache={stable}")
        assert np.array_equal(outs[0], outs[1])
    finally:
        op.close()
