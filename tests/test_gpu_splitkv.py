"""Split-KV over several ranks, emulated on ONE GPU (ranks as consecutive passes over their key
ranges): every rank writes partial records for its keys, reduces them to one record per (row,
head) (esp_attn_reduce_parts), the records are laid side by side as an all-gather would, and
the final merge (esp_attn_combine_parts) must reproduce attention over the whole sequence."""
import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, shard, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


def _rank_workload(w, lo, hi):
    """The part of a single-sequence decode workload a rank holds: keys [lo, hi) with their pages."""
    bt = w.bt
    pages = list(range(lo // bt, (hi + bt - 1) // bt))
    pool = w.kv.reshape(w.n_blocks, -1)
    sub = wl.make_pass(w.name + "_r", 1, [(hi - lo, 1)], w.H, w.Hkv, w.HD, bt, w.q_dtype, w.kv_dtype, spare_blocks=1)
    sub.Q, sub.Kb, sub.Vb = w.Q, w.Kb, w.Vb
    kv = sub.kv.reshape(sub.n_blocks, -1)
    for i, pg in enumerate(pages):
        kv[int(sub.blocks[i])] = pool[int(w.blocks[pg])]
        if w.kv_scales is not None:
            sub.kv_scales[int(sub.blocks[i])] = w.kv_scales[int(w.blocks[pg])]
    return sub


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8"])
def test_split_kv_ranks_match_whole_sequence(oracle_lib, world, fp8):
    P = 6000 + 16 * world + 5
    w = wl.make_pass("splitkv", 60 + world, [(P, 1)], 32, 8, 256 if fp8 else 128, 16, wl.BF16, wl.E4M3 if fp8 else None)
    ref, lse_ref = oracle_lib.attention_f64(w)
    ranges = shard.split_kv_range(P, world, w.bt)
    assert ranges[0][0] == 0 and ranges[-1][1] == P and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    op = host.AttnOp.for_workload(w)
    try:
        rec_floats = op.parts_floats(1)
        gathered = torch.zeros(world * rec_floats, dtype=torch.float32, device=op.device)
        for r, (lo, hi) in enumerate(ranges):
            sub = _rank_workload(w, lo, hi)
            plan = host.plan_tiles(sub.trees, sub.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
            tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=(r == world - 1))
            dp = op.upload(sub, host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, 8))
            op.forward(dp)                                   # records only, no local combine
            assert op.last_kernel == "decode_gqa"
            jobs_dev = host._dev(jobs, op.device)
            op.reduce_parts(dp, dp.parts, jobs_dev, len(jobs), gathered, out_part0=r)
            torch.cuda.synchronize()
        merge = shard.world_merge_jobs(1, world)
        dpw = op.upload(w)
        op.combine(dpw, gathered, host._dev(merge, op.device), len(merge))
        op.check_status()
        torch.cuda.synchronize()
        O = dpw.O.cpu().numpy().view(np.uint16)
        lse = dpw.lse.cpu().numpy()
    finally:
        op.close()
    util.check_output(O, ref, w)
    assert np.abs(lse - lse_ref).max() < 2e-3


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8"])
def test_peer_exchange_emulated_ranks(oracle_lib, world, fp8):
    """esp_attn_exchange_parts with the ranks emulated on one GPU: every emulated rank runs the
    publishing phase (merge + stores into all ranks' buffers + flags), then every rank runs the
    waiting phase, whose flags are all set by then (no kernel ever waits for a later launch).
    All ranks must produce identical bits, equal to attention over the whole sequence; a second
    epoch on the same buffers (other parity) must do so again."""
    P = 5000 + 16 * world + 3
    w = wl.make_pass("xch", 80 + world, [(P, 1)], 32, 8, 256 if fp8 else 128, 16, wl.BF16, wl.E4M3 if fp8 else None)
    ref, lse_ref = oracle_lib.attention_f64(w)
    ranges = shard.split_kv_range(P, world, w.bt)
    op = host.AttnOp.for_workload(w)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=world)
    try:
        passes = []
        for r, (lo, hi) in enumerate(ranges):
            sub = _rank_workload(w, lo, hi)
            plan = host.plan_tiles(sub.trees, sub.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
            tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=(r == world - 1))
            dp = op.upload(sub, host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, 8))
            passes.append((dp, host._dev(jobs, op.device), len(jobs), n_parts))
        for epoch in range(3):
            xch.next_epoch()
            for r, (dp, jobs_dev, n_jobs, n_parts) in enumerate(passes):
                dp.O.zero_()
                op.forward(dp)
                op.exchange_parts(dp, dp.parts, jobs_dev, n_jobs, xch, rank=r, phases=1, parts_max=n_parts)
            torch.cuda.synchronize()
            outs = []
            for r, (dp, jobs_dev, n_jobs, n_parts) in enumerate(passes):
                op.exchange_parts(dp, dp.parts, jobs_dev, n_jobs, xch, rank=r, phases=2, parts_max=n_parts)
                op.check_status()
                outs.append((dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy()))
            for O, lse in outs[1:]:
                assert np.array_equal(O, outs[0][0]) and np.array_equal(lse, outs[0][1])
            util.check_output(outs[0][0], ref, w)
            assert np.abs(outs[0][1] - lse_ref).max() < 2e-3
    finally:
        xch.close()
        op.close()


def test_peer_exchange_single_rank_one_launch(oracle_lib):
    """world = 1, phases = 3: the fused kernel publishes to itself and finishes in the same launch."""
    w = wl.make_pass("xch1", 91, [(3000, 1), (1234, 1)], 32, 8, 128, 16, wl.BF16, None)
    ref, _ = oracle_lib.attention_f64(w)
    op = host.AttnOp.for_workload(w)
    plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
    tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=True)
    xch = host.PeerExchange.emulated(op, n_jobs=len(jobs), rows_max=1, world=1)
    try:
        dp = op.upload(w, host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, 8))
        jobs_dev = host._dev(jobs, op.device)
        for _ in range(2):
            xch.next_epoch()
            dp.O.zero_()
            op.forward(dp)
            op.exchange_parts(dp, dp.parts, jobs_dev, len(jobs), xch, rank=0, phases=3, parts_max=n_parts)
            op.check_status()
            util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w)
    finally:
        xch.close()
        op.close()


def test_peer_exchange_wait_runs_out(oracle_lib):
    """A peer that never publishes: the waiting phase gives up after wait_ms, leaves O alone, the
    status word reports it, and the context keeps working afterwards (host-visible failure, no fault)."""
    w = wl.make_pass("xchT", 92, [(777, 1)], 32, 8, 128, 16, wl.BF16, None)
    ref, _ = oracle_lib.attention_f64(w)
    op = host.AttnOp.for_workload(w)
    plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
    tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=True)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=2)
    try:
        dp = op.upload(w, host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, 8))
        jobs_dev = host._dev(jobs, op.device)
        xch.next_epoch()
        op.forward(dp)
        dp.O.fill_(7.0)
        op.exchange_parts(dp, dp.parts, jobs_dev, 1, xch, rank=0, phases=1, parts_max=n_parts)   # rank 1 stays silent
        op.exchange_parts(dp, dp.parts, jobs_dev, 1, xch, rank=0, phases=2, parts_max=n_parts, wait_ms=50)
        with pytest.raises(capi.EspError, match="peer GPU never published"):
            op.check_status()
        assert bool((dp.O == 7.0).all())
        op.check_status()                      # cleared
        dpw = op.upload(w, plan)
        op.forward(dpw)                        # an ordinary pass still runs on the same context
        op.check_status()
        util.check_output(dpw.O.cpu().numpy().view(np.uint16), ref, w)
    finally:
        xch.close()
        op.close()


def _rank_pass(op, sub, last, groups=64):
    """A rank's records-only plan with its reduce job, uploaded: (dp, args for esp_attn_forward_exchange)."""
    plan = host.plan_tiles(sub.trees, sub.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, groups, 8)
    tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=last)
    dp = op.upload(sub, host.Plan(tiles, jobs, n_parts, 8))
    return dp, op.make_args(dp)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8"])
@pytest.mark.parametrize("groups", [16, 64, 296])
def test_fused_exchange_emulated_ranks(oracle_lib, world, fp8, groups):
    """esp_attn_forward_exchange with the ranks emulated on one GPU: every rank's ONE launch computes its
    records, folds them in two levels inside the decode kernel and stores the result into all ranks'
    buffers (phase 1: it does not wait); then every rank runs the second half (phase 2), whose words are
    all there by then - no launch ever waits for a later one. All ranks must hold identical bits, equal
    to attention over the whole sequence, for three epochs on the same buffers; and the bits must be the
    ones the two-kernel route (esp_attn_forward + esp_attn_exchange_parts) stores in the buffers, up to
    the order of the folds (same tolerance)."""
    P = 7000 + 16 * world + 9
    w = wl.make_pass("fxch", 180 + world, [(P, 1)], 32, 8, 256 if fp8 else 128, 16, wl.BF16, wl.E4M3 if fp8 else None)
    ref, lse_ref = oracle_lib.attention_f64(w)
    ranges = shard.split_kv_range(P, world, w.bt)
    op = host.AttnOp.for_workload(w)
    op.set_option("fuse_exchange", 1)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=world)
    try:
        passes = [_rank_pass(op, _rank_workload(w, lo, hi), r == world - 1, groups) for r, (lo, hi) in enumerate(ranges)]
        for epoch in range(3):
            xch.next_epoch()
            launches0 = op.launch_count
            for r, (dp, args) in enumerate(passes):
                dp.O.zero_()
                op.forward_exchange(dp, args, xch, rank=r, phases=1)
            assert op.launch_count - launches0 == world and op.last_kernel == "decode_gqa"   # one launch per rank
            torch.cuda.synchronize()
            outs = []
            for r, (dp, args) in enumerate(passes):
                op.forward_exchange(dp, args, xch, rank=r, phases=2)
                op.check_status()
                outs.append((dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy()))
            for O, lse in outs[1:]:
                assert np.array_equal(O, outs[0][0]) and np.array_equal(lse, outs[0][1])
            util.check_output(outs[0][0], ref, w)
            assert np.abs(outs[0][1] - lse_ref).max() < 2e-3
    finally:
        xch.close()
        op.close()


def test_fused_exchange_one_rank_one_launch_and_many_parts(oracle_lib):
    """world = 1, phases = 3: one launch publishes to itself, reads its own words and writes the row. Also with
    a plan of 64 records (8 groups of 8 in the two-level fold) and with few records (a single level)."""
    w = wl.make_pass("fxch1", 191, [(9000, 1)], 32, 8, 128, 16, wl.BF16, None)
    ref, lse_ref = oracle_lib.attention_f64(w)
    op = host.AttnOp.for_workload(w)
    op.set_option("fuse_exchange", 1)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=1)
    try:
        for groups in (8, 40, 296, 512):
            dp, args = _rank_pass(op, w, True, groups)
            for _ in range(2):
                xch.next_epoch()
                dp.O.zero_()
                n0 = op.launch_count
                op.forward_exchange(dp, args, xch, rank=0, phases=3)
                op.check_status()
                torch.cuda.synchronize()
                resident = len(dp.plan.tiles) * w.Hkv <= 2 * 148        # the waiting CTAs need the whole grid on the GPU at once
                assert op.launch_count - n0 == (1 if resident else 2), f"groups={groups}: {op.launch_count - n0} launches"
                util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w, what=f"groups={groups}")
                assert np.abs(dp.lse.cpu().numpy() - lse_ref).max() < 2e-3
    finally:
        xch.close()
        op.close()


def test_fused_exchange_wait_runs_out(oracle_lib):
    """One launch that waits for a peer which never publishes: after wait_ms it leaves O alone and the status
    word reports it; the context keeps working (a bounded wait that runs out - no fault, no hang)."""
    w = wl.make_pass("fxchT", 192, [(2000, 1)], 32, 8, 128, 16, wl.BF16, None)
    ref, _ = oracle_lib.attention_f64(w)
    op = host.AttnOp.for_workload(w)
    op.set_option("fuse_exchange", 1)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=2)
    try:
        dp, args = _rank_pass(op, w, True)
        xch.next_epoch()
        dp.O.fill_(7.0)
        op.forward_exchange(dp, args, xch, rank=0, phases=3, wait_ms=50)     # rank 1 stays silent
        with pytest.raises(capi.EspError, match="peer GPU never published"):
            op.check_status()
        assert bool((dp.O == 7.0).all())
        op.check_status()
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
        dpw = op.upload(w, plan)
        op.forward(dpw)                                                       # merges in the kernel with the same counters
        op.check_status()
        util.check_output(dpw.O.cpu().numpy().view(np.uint16), ref, w)
    finally:
        xch.close()
        op.close()


def test_two_level_merge_matches_the_combine_kernel(oracle_lib):
    """The in-kernel merge (fuse_combine 2: groups folded as they finish, then the groups) against the
    combine kernel (fuse_combine 0) on plans of 2 to 64 records per sequence: both within tolerance of the
    float64 oracle, and equal to each other to fp32 rounding of the fold order."""
    w = wl.make_pass("twolevel", 193, [(30000, 1), (700, 1), (5000, 1), (64, 1)], 32, 4, 128, 16, wl.BF16)
    ref, lse_ref = oracle_lib.attention_f64(w)
    for groups in (16, 128, 1184, 4096):
        res = {}
        for fuse in (0, 2):
            O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_B200, tile_rows=8, groups=groups, split=1 << 20,
                                                        options={"fuse_combine": fuse})
            assert kernel == "decode_gqa"
            util.check_output(O, ref, w, what=f"groups={groups} fuse={fuse}")
            assert np.abs(lse - lse_ref).max() < 2e-3
            res[fuse] = wl.from_bits16(O, w.q_dtype)
        assert np.abs(res[0] - res[2]).max() <= 2.0 ** -7 * np.abs(res[0]).max()


def test_forward_exchange_default_route_is_two_kernels(oracle_lib):
    """Without the option esp_attn_forward_exchange runs the records-only pass and the exchange kernel (the route
    that measured faster); same result."""
    w = wl.make_pass("fxch2k", 194, [(6000, 1)], 32, 8, 128, 16, wl.BF16, None)
    ref, _ = oracle_lib.attention_f64(w)
    op = host.AttnOp.for_workload(w)
    xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=1)
    try:
        dp, args = _rank_pass(op, w, True)
        xch.next_epoch()
        n0 = op.launch_count
        op.forward_exchange(dp, args, xch, rank=0, phases=3)
        op.check_status()
        assert op.launch_count - n0 == 2
        util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w)
    finally:
        xch.close()
        op.close()
