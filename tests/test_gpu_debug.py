"""Debug and robustness surfaces of the C ABI on the GPU: the NaN / Inf detector over the attention
output (the reference's finite_check, site "attn_out"), block ids outside the pool caught by the
general kernel instead of read, 64- and 512-dim heads, and the attn_vec option."""
import ctypes as C

import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


def test_finite_check_record_matches_a_host_scan():
    lib = capi.load()
    rows, cols, ld = 37, 200, 256
    rng = np.random.default_rng(5)
    x = rng.standard_normal((rows, ld)).astype(np.float32)
    x[:, cols:] = np.nan                                   # padding columns are not scanned
    bad = [(3, 7, np.inf), (3, 9, np.nan), (20, 199, -np.inf), (36, 0, 5e12)]
    for r, c, v in bad:
        x[r, c] = v
    rec = torch.zeros(4, dtype=torch.int32, device="cuda")
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for dtype, t in ((0, torch.from_numpy(x).cuda()), (2, torch.from_numpy(x).cuda().bfloat16()), (1, torch.from_numpy(x).cuda().half())):
        for thr, want in ((float("inf"), 3 if dtype != 1 else 4), (1e11, 4)):   # 5e12 overflows fp16 to Inf
            capi.check(lib.esp_attn_finite_check(s, C.c_void_p(t.data_ptr()), rows, cols, ld, dtype, thr, C.c_void_p(rec.data_ptr())))
            torch.cuda.synchronize()
            hits, idx, done, val = (int(v) & 0xFFFFFFFF for v in rec.cpu().numpy())
            assert hits == want and idx == 3 * cols + 7 and done > 0
            assert np.isinf(np.uint32(val).view(np.float32))
    clean = torch.from_numpy(np.ascontiguousarray(x[:, :cols])).cuda()
    clean[torch.isnan(clean) | torch.isinf(clean)] = 0
    clean[36, 0] = 1.0
    capi.check(lib.esp_attn_finite_check(s, C.c_void_p(clean.data_ptr()), rows, cols, cols, 0, float("inf"), C.c_void_p(rec.data_ptr())))
    torch.cuda.synchronize()
    hits, idx, _, _ = (int(v) & 0xFFFFFFFF for v in rec.cpu().numpy())
    assert hits == 0 and idx == 0xFFFFFFFF


def test_check_finite_option_reports_the_first_bad_output_element():
    """A NaN planted in one value row of the pool reaches O; with the option on, check_status names it."""
    w = wl.make_pass("finite", 70, [(200, 1), (100, 1)], 8, 2, 128, 16, wl.BF16)
    blk = int(w.blocks[int(w.trees[1]["table"])])
    kv = w.kv.reshape(w.n_blocks, 2, w.bt, w.kv_ld)
    kv[blk, 1, 3, 5] = 0x7FC0                              # V of key 3 of sequence 1, kv head 0, dim 5: NaN
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv)
        dp = op.upload(w, plan)
        op.forward(dp)
        op.check_status()                                  # the option is off: nothing is reported
        op.set_option("check_finite", 1)
        op.forward(dp)
        with pytest.raises(capi.EspError) as e:
            op.check_status()
        assert "attn_out" in str(e.value) and "row 1, column 5" in str(e.value)
        op.check_status()                                  # read once, then cleared
    finally:
        op.close()


def test_block_id_outside_the_pool_is_caught_not_read():
    w = wl.make_pass("badblock", 71, [(300, 4)], 8, 2, 128, 16, wl.BF16)
    w.blocks[2] = w.n_blocks + 1000                        # what a corrupted table would hold
    op = host.AttnOp.for_workload(w)
    try:
        op.set_option("attn_umma", 0)
        plan = host.plan_tiles(w.trees, w.Hkv)
        dp = op.upload(w, plan)
        op.forward(dp)
        assert op.last_kernel == "flash_general"
        with pytest.raises(capi.EspError) as e:
            op.check_status()
        assert "bad block id" in str(e.value)
        torch.cuda.synchronize()                           # the context is alive: no fault happened
        dp2 = op.upload(wl.make_pass("ok", 72, [(300, 4)], 8, 2, 128, 16, wl.BF16), plan)
        op.forward(dp2)
        op.check_status()
    finally:
        op.close()


def test_512_dim_heads(oracle_lib):
    """The reference's Gemma global layers (src/model/impl/gemma.h:119-147): HD 512. Single-row trees take the decode
    kernel, multi-row tiles the tcgen05 kernel (re-planned from 8-row tiles); the general one is the cross-check of both."""
    for trees, options, want in (([(700, 1), (33, 1)], None, "decode_gqa"), ([(700, 1), (33, 1)], {"attn_gqa": 0}, "flash_general"),
                                 ([(100, 9)], None, "flash_umma_pair"), ([(100, 9)], {"attn_umma": 0}, "flash_general")):
        w = wl.make_pass("hd512", 73, trees, 4, 2, 512, 16, wl.BF16, scale=1.0 / np.sqrt(512.0))
        ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
        O, lse, _, plan, kernel = host.run_pass(w, options=options)
        assert kernel == want
        util.check_output(O, ref, w, what="hd512", ref_abs=ref_abs if want == "flash_umma_pair" else None)
        assert np.abs(lse - lse_ref).max() < 2e-3


def test_64_dim_heads(oracle_lib):
    """64-dim heads (kernels/90_lfm2.metal:160-161): single-row trees over 16-bit pools take the decode kernel; E4M3
    pools (a row is half a 128-byte line) the general one, multi-row tiles the tcgen05 kernel (re-planned from 8-row tiles)."""
    for trees, kvdt, options, want in (([(700, 1), (33, 1)], None, None, "decode_gqa"), ([(700, 1), (33, 1)], wl.E4M3, None, "flash_general"),
                                       ([(100, 9), (0, 40)], None, None, "flash_umma_pair"), ([(100, 9), (0, 40)], None, {"attn_umma": 0}, "flash_general")):
        w = wl.make_pass("hd64", 76, trees, 8, 2, 64, 16, wl.BF16, kvdt)
        ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
        O, lse, _, plan, kernel = host.run_pass(w, options=options)
        assert kernel == want
        # (the tensor-core kernel rounds P to bf16 before P.V: the allowance 2^-9 * sum_j p_j |v_j| of the tcgen05 tests)
        util.check_output(O, ref, w, what="hd64", ref_abs=ref_abs if want == "flash_umma_pair" else None)
        assert np.abs(lse - lse_ref).max() < 2e-3


def test_attn_vec_option_has_a_defined_answer():
    w = wl.make_pass("vec", 74, [(64, 1)], 8, 2, 128, 16, wl.BF16)
    op = host.AttnOp.for_workload(w)
    try:
        op.set_option("attn_vec", 0)
        with pytest.raises(capi.EspError) as e:
            op.set_option("attn_vec", 1)
        assert e.value.code == capi.ESP_ERR_UNSUPPORTED
    finally:
        op.close()


def test_profile_reports_gpu_time_per_kernel():
    """esp_attn_set_profile / esp_attn_get_profile (the reference's set_profile, src/model/model.mm:1041-1054): every
    launch timed on its own, summed per kernel name."""
    lib = capi.load()
    w = wl.make_pass("prof", 75, [(5000, 1), (3000, 1)], 32, 8, 256, 16, wl.BF16, wl.E4M3)
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv)               # split by the reference planner: decode + combine
        dp = op.upload(w, plan)
        op.forward(dp)                                       # not profiled
        capi.check(lib.esp_attn_set_profile(op.ctx, 1))
        for _ in range(5):
            op.forward(dp)
        ents = (capi.ProfileEntry * 8)()
        n = C.c_int32()
        capi.check(lib.esp_attn_get_profile(op.ctx, ents, 8, C.byref(n)))
        got = {ents[i].kernel.decode(): (ents[i].launches, ents[i].gpu_ms) for i in range(n.value)}
        assert set(got) == {"decode_gqa", "attention_combine"}
        assert got["decode_gqa"][0] == 5 and got["attention_combine"][0] == 5
        assert 0.0 < got["attention_combine"][1] < got["decode_gqa"][1] < 50.0
        capi.check(lib.esp_attn_set_profile(op.ctx, 0))      # off: the sums are cleared, nothing more is recorded
        op.forward(dp)
        capi.check(lib.esp_attn_get_profile(op.ctx, ents, 8, C.byref(n)))
        assert n.value == 0
        op.check_status()
    finally:
        op.close()
