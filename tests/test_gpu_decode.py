"""Parity of the CUDA decode path (esp_attn_forward -> decode_gqa / flash_general ->
attention_combine) with the oracle, through the C ABI. Tolerances: max abs error <= 2e-3
(fp16 / bf16 pools) and <= 1e-2 (E4M3 pools) against float64, plus half an output ulp for
storing the result in 16 bits; page-table indexing bit-exact through integer probes."""
import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


def _run(w, mode=capi.ESP_PLAN_REFERENCE, options=None, split=512, groups=256, force_parts=False, tile_rows=8):
    return host.run_pass(w, mode=mode, tile_rows=tile_rows, split=split, groups=groups, options=options, force_parts=force_parts)


CASES = [
    # name, trees, H, Hkv, HD, bt, q dtype, kv dtype, gate
    ("c1_f16", [(1024, 1)], 8, 2, 128, 16, wl.F16, None, False),
    ("c2_small_bf16", [(p, 1) for p in (512, 777, 1500, 2048, 3000)], 32, 4, 128, 16, wl.BF16, None, False),
    ("c5_small_fp8", [(8192, 1)], 32, 8, 256, 16, wl.BF16, wl.E4M3, False),
    ("hd256_bf16", [(900, 1), (64, 1)], 16, 4, 256, 16, wl.BF16, None, False),
    ("hd256_f16_gate", [(300, 1), (1000, 1)], 16, 4, 256, 16, wl.F16, None, True),
    ("hd128_fp8_f16q", [(700, 1), (5000, 1)], 16, 2, 128, 16, wl.F16, wl.E4M3, False),
    ("g1_bt64", [(1000, 1), (130, 1)], 4, 4, 128, 64, wl.BF16, None, True),
    ("g2_bt32", [(555, 1)], 8, 4, 128, 32, wl.F16, None, False),
    # 512-dim heads: the global layers of kernels/80_gemma.metal (HD = 512 instantiations, gemma.h:119-147)
    ("hd512_bf16", [(900, 1), (64, 1), (5000, 1)], 8, 2, 512, 16, wl.BF16, None, False),
    ("hd512_f16_gate_g8", [(300, 1), (1000, 1)], 16, 2, 512, 16, wl.F16, None, True),
    ("hd512_fp8", [(700, 1), (3000, 1)], 8, 1, 512, 16, wl.BF16, wl.E4M3, False),
    ("hd512_fp8_f16q_bt32", [(2100, 1)], 4, 2, 512, 32, wl.F16, wl.E4M3, False),
    # 64-dim heads (kernels/90_lfm2.metal:160-161), 16-bit pools
    ("hd64_bf16", [(900, 1), (64, 1), (7000, 1)], 16, 4, 64, 16, wl.BF16, None, False),
    ("hd64_f16_gate_g8", [(300, 1), (1000, 1)], 16, 2, 64, 16, wl.F16, None, True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
@pytest.mark.parametrize("mode", [capi.ESP_PLAN_REFERENCE, capi.ESP_PLAN_B200], ids=["refplan", "b200plan"])
def test_decode_matches_oracle(oracle_lib, case, mode):
    name, trees, H, Hkv, HD, bt, dt, kvdt, gate = case
    w = wl.make_pass(name, 1000 + len(name), trees, H, Hkv, HD, bt, dt, kvdt, gate=gate)
    ref, lse_ref = oracle_lib.attention_f64(w)
    groups = 256 if mode == capi.ESP_PLAN_REFERENCE else 592
    O, lse, parts, plan, kernel = _run(w, mode=mode, groups=groups, split=512 if mode == capi.ESP_PLAN_REFERENCE else 1 << 20)
    assert kernel == "decode_gqa"
    util.check_output(O, ref, w, what=name)
    assert np.abs(lse - lse_ref).max() < 2e-3
    # the general kernel is an independent second implementation of the same contract
    O2, lse2, _, _, kernel2 = _run(w, mode=mode, groups=groups, options={"attn_gqa": 0})
    assert kernel2 == "flash_general"
    util.check_output(O2, ref, w, what=name + "/general")
    assert np.abs(lse2 - lse_ref).max() < 2e-3


@pytest.mark.parametrize("P", [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100])
def test_decode_edge_context_lengths(oracle_lib, P):
    for dt, kvdt, HD in ((wl.BF16, None, 128), (wl.F16, wl.E4M3, 256), (wl.F16, None, 512), (wl.BF16, wl.E4M3, 512), (wl.BF16, None, 64)):
        w = wl.make_pass("edge", 77 + P, [(P, 1), (max(0, P - 1), 1)], 8, 2, HD, 16, dt, kvdt)
        ref, lse_ref = oracle_lib.attention_f64(w)
        O, lse, _, plan, kernel = _run(w)
        assert kernel == "decode_gqa"
        util.check_output(O, ref, w, what=f"P={P}")
        assert np.abs(lse - lse_ref).max() < 2e-3


def test_unsplit_and_record_paths_agree_with_f64(oracle_lib):
    """Every tile forced to write its fp32 record: the records merged in float64 on the host are
    the unrounded result, compared with no output-rounding allowance."""
    w = wl.make_pass("rec", 31, [(2000, 1), (40, 1), (0, 1)], 16, 2, 128, 16, wl.BF16)
    ref, lse_ref = oracle_lib.attention_f64(w)
    O, lse, parts, plan, kernel = _run(w, force_parts=True)
    assert kernel == "decode_gqa"
    O64, lse64 = util.records_to_output(parts, w, plan.tiles, plan.jobs, 8)
    assert np.abs(O64 - ref).max() <= util.TOL_16
    assert np.abs(lse64 - lse_ref).max() < 1e-3
    util.check_output(O, ref, w)


def test_decode_matches_reference_restatement(oracle_lib):
    """Against the fp32 restatement of attn_decode_gqa on the same plan (same record layout)."""
    w = wl.make_pass("restate", 32, [(1024, 1)], 8, 2, 128, 16, wl.F16)
    O, lse, parts, plan, _ = _run(w)
    O_r, lse_r, parts_r = oracle_lib.decode_gqa_f32(w, plan.tiles, 8, plan.n_parts)
    n = plan.n_parts * w.Hkv * 8 * w.G
    rec = parts[: n * (w.HD + 2)].reshape(-1, 8, w.G, w.HD + 2)[:, 0]      # row 0 of each 8-row slot
    rec_r = parts_r[: n * (w.HD + 2)].reshape(-1, 8, w.G, w.HD + 2)[:, 0]
    # normalised records agree to fp32 softmax accuracy
    assert np.abs(rec[..., :w.HD] / rec[..., w.HD + 1:] - rec_r[..., :w.HD] / rec_r[..., w.HD + 1:]).max() < 2e-3
    lse_rec = rec[..., w.HD] + np.log(rec[..., w.HD + 1])
    lse_rec_r = rec_r[..., w.HD] + np.log(rec_r[..., w.HD + 1])
    assert np.abs(lse_rec - lse_rec_r).max() < 1e-3


@pytest.mark.parametrize("kvdt", [None, wl.E4M3], ids=["bf16", "fp8"])
def test_page_table_probe_is_exact(kvdt):
    """Q = 0: every key weighs exactly 1, the fp32 record is the integer sum of the V rows of the
    keys the tile covers. V encodes (key mod 16, key / 16 mod 16, key / 256, kv head) in values
    exactly representable in bf16 and E4M3; the pool is otherwise filled with a poison value, so a
    wrong block, row, head or range changes an integer."""
    P, H, Hkv, HD, bt = 1000, 16, 2, 128, 16
    w = wl.make_pass("probe", 55, [(P, 1), (333, 1)], H, Hkv, HD, bt, wl.BF16, kvdt, spare_blocks=5)
    w.Q[:] = 0
    pool = np.full((w.n_blocks, 2, bt, Hkv, HD), 7.0, dtype=np.float32)  # poison
    for ti, t in enumerate(w.trees):
        for j in range(int(t["P"])):
            b = int(w.blocks[int(t["table"]) + j // bt])
            pool[b, 1, j % bt, :, :] = 0
            for kvh in range(Hkv):
                pool[b, 1, j % bt, kvh, 0:5] = [j % 16, (j // 16) % 16, j // 256, kvh + 1, ti + 1]
    if kvdt is None:
        w.kv = wl.f32_to_bf16_bits(pool.reshape(-1))
    else:
        w.kv_scales[:] = 1.0
        w.kv = wl.e4m3_encode(pool.reshape(-1))
    w.Vb[:] = 0
    O, lse, parts, plan, kernel = _run(w, force_parts=True, split=128)
    assert kernel == "decode_gqa"
    rec = parts[: plan.n_parts * Hkv * 8 * w.G * (HD + 2)].reshape(plan.n_parts, Hkv, 8, w.G, HD + 2)
    for t in plan.tiles:
        ti, k0, k1, part = int(t["tree"]), int(t["k0"]), int(t["k1"]), int(t["part"])
        js = np.arange(k0, k1)
        n = len(js) + int(t["last"])
        for kvh in range(Hkv):
            r = rec[part, kvh, 0]
            assert np.all(r[:, HD] == 0.0), "m must be exactly 0"
            assert np.all(r[:, HD + 1] == n), (r[:, HD + 1], n)
            want = [float((js % 16).sum()), float(((js // 16) % 16).sum()), float((js // 256).sum()), float((kvh + 1) * len(js)),
                    float((ti + 1) * len(js))]
            assert np.all(r[:, 0:5] == np.array(want, dtype=np.float32)), (r[0, 0:5], want)
            assert np.all(r[:, 5:HD] == 0.0)


def test_fail_pass_injection_and_validation():
    w = wl.make_pass("inject", 5, [(128, 1)] * 64, 8, 2, 128, 16, wl.BF16)
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv)
        dp = op.upload(w, plan)
        op.set_option("fail_pass", 2)
        op.forward(dp)
        with pytest.raises(capi.EspError) as ei:
            op.forward(dp)
        assert ei.value.code == capi.ESP_ERR_INJECTED and "injected" in str(ei.value)
        op.set_option("fail_pass", 0)
        # validation: a tile whose key range passes the tree's cached keys is refused before launch
        bad = host.Plan(plan.tiles.copy(), plan.jobs, plan.n_parts, plan.tile_rows)
        bad.tiles[0]["k1"] = 999
        dp2 = op.upload(w, bad)
        n0 = op.launch_count
        with pytest.raises(capi.EspError) as ei:
            op.forward(dp2)
        assert ei.value.code == capi.ESP_ERR_INVALID and op.launch_count == n0
        op.forward(dp)
        op.check_status()
    finally:
        op.close()


@pytest.mark.parametrize("shape", [(32, 4, 128, None, False), (32, 8, 256, wl.E4M3, False), (16, 4, 128, None, True),
                                   (8, 8, 128, None, False), (16, 8, 128, None, False)], ids=["hd128", "hd256-fp8", "gate", "g1", "g2"])
def test_decode_fused_merge_matches_combine_kernel(oracle_lib, shape):
    """ESP_PLAN_B200 tiles name their combine job: the decode kernel then merges the records itself
    (the CTA that finishes a job last, in record order) and no combine kernel is launched. With
    the option off the same plan takes the two-kernel route; both must match the oracle, agree with
    each other to an output ulp, and the fused route must repeat bit for bit."""
    H, Hkv, HD, kvdt, gate = shape
    w = wl.make_pass("fused_dec", 11, [(9000, 1), (70, 1), (3333, 1), (64, 1), (20000, 1), (5, 1)], H, Hkv, HD, 16, wl.BF16, kvdt,
                     gate=gate)
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    outs = {}
    for fuse in (1, 0):
        op = host.AttnOp.for_workload(w, 8)
        try:
            op.set_option("fuse_combine", fuse)
            plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 128, 8)  # at most 128 CTAs: a small pass
            assert plan.n_parts > 4 and len(plan.jobs) >= 2
            assert all(int(t["pad1"]) >= 1 for t in plan.tiles if t["part"] >= 0)
            dp = op.upload(w, plan)
            n0 = op.launch_count
            seen = []
            for _ in range(3):
                dp.O.zero_()
                dp.lse.zero_()
                op.forward(dp)
                op.check_status()
                seen.append((dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy()))
            assert op.last_kernel == "decode_gqa"
            fused_here = fuse and (H // Hkv) % 2 == 0          # a single head per kv head keeps the combine kernel
            assert op.launch_count - n0 == (3 if fused_here else 6)
            assert all(np.array_equal(seen[0][0], s[0]) and np.array_equal(seen[0][1], s[1]) for s in seen[1:])
            outs[fuse] = seen[0]
        finally:
            op.close()
    util.check_output(outs[1][0], ref, w, ref_abs=ref_abs)   # the 5-key row needs the P-rounding allowance
    util.check_output(outs[0][0], ref, w, ref_abs=ref_abs)
    assert np.abs(outs[1][1] - lse_ref).max() < 2e-3
    fa, fb = wl.from_bits16(outs[1][0], w.q_dtype), wl.from_bits16(outs[0][0], w.q_dtype)
    assert np.all(np.abs(fa - fb) <= 2.0 ** -7 * np.maximum(np.abs(fa), np.abs(fb)) + 1e-30)
    assert np.abs(outs[1][1] - outs[0][1]).max() < 1e-5


def test_in_kernel_merge_is_deterministic():
    """A batched decode whose many jobs are merged inside the kernel by whichever CTA finishes a job
    last: forty passes must give the same bits (no result may depend on that order) with one launch each."""
    import torch
    w = wl.config_c2(n_seqs=16, hi=8192)
    op = host.AttnOp.for_workload(w, 8)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 2368, 8)
        assert len(plan.jobs) * w.Hkv >= 32
        dp = op.upload(w, plan)
        op.forward(dp)
        ref_O, ref_lse = dp.O.clone(), dp.lse.clone()
        n0 = op.launch_count
        for _ in range(40):
            dp.O.zero_()
            op.forward(dp)
            assert torch.equal(dp.O, ref_O) and torch.equal(dp.lse, ref_lse)
        op.check_status()
        assert op.launch_count - n0 == 40 and op.last_kernel == "decode_gqa"
    finally:
        op.close()
