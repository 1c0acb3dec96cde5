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
