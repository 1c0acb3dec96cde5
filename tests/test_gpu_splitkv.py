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
