"""Child process of tests/test_gpu_multi.py: one rank of a split-KV decode over several GPUs.

Launched with torch.distributed.run (one process per GPU, NCCL, rendezvous on 127.0.0.1). Every rank
builds the same seeded single-sequence decode workload, keeps the pages of its own key range, and
the ranks finish it twice: with the fused peer exchange kernel (esp_attn_exchange_parts), with the
one-launch route (esp_attn_forward_exchange) and with reduce + NCCL all-gather + combine. Both must match the float64 oracle over the whole sequence,
every rank must hold identical bits, and a few more epochs on the same buffers must repeat them.
Rank 0 prints one line "MULTI_GPU_OK ..." on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from espetero_b200 import capi, host, shard, workloads as wl  # noqa: E402
import oracle  # noqa: E402
from tests import util  # noqa: E402
from tests.test_gpu_splitkv import _rank_workload  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    fp8 = len(sys.argv) > 1 and sys.argv[1] == "fp8"
    P = 9000 + 16 * world + 7
    w = wl.make_pass("multi", 300 + world, [(P, 1)], 32, 8, 256 if fp8 else 128, 16, wl.BF16, wl.E4M3 if fp8 else None)
    oracle.load()
    ref, lse_ref = oracle.attention_f64(w)
    lo, hi = shard.split_kv_range(P, world, w.bt)[rank]
    sub = _rank_workload(w, lo, hi)
    op = host.AttnOp.for_workload(w, 8, local)
    plan = host.plan_tiles(sub.trees, sub.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, 64, 8)
    tiles, jobs, n_parts = shard.local_decode_plan(plan.tiles, is_last_rank=(rank == world - 1))
    dp = op.upload(sub, host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, 8))
    jobs_dev = host._dev(jobs, dev)
    xch = host.PeerExchange(op, n_jobs=1, rows_max=1)
    outs = []
    for _ in range(5):
        xch.next_epoch()
        dp.O.zero_()
        op.forward(dp)
        op.exchange_parts(dp, dp.parts, jobs_dev, len(jobs), xch, parts_max=n_parts)
        op.check_status()
        outs.append((dp.O.cpu().numpy().view(np.uint16).copy(), dp.lse.cpu().numpy().copy()))
    for O, lse in outs[1:]:
        assert np.array_equal(O, outs[0][0]) and np.array_equal(lse, outs[0][1]), "epochs differ"
    util.check_output(outs[0][0], ref, w)
    assert np.abs(outs[0][1] - lse_ref).max() < 2e-3
    # identical bits on every rank
    mine = torch.from_numpy(outs[0][0].astype(np.int32)).to(dev)
    every = torch.empty(world * mine.numel(), dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(every, mine.flatten())
    every = every.view(world, -1)
    assert bool((every == every[0]).all()), "ranks hold different outputs"
    # the one-launch route (esp_attn_forward_exchange: records, two-level fold, peer stores, wait and final fold in
    # the decode kernel): correct, identical on every rank, the same over several epochs, and one launch per step
    op.set_option("fuse_exchange", 1)
    dpf = op.upload(sub, host.Plan(tiles, jobs, n_parts, 8))
    args_f = op.make_args(dpf)
    fused = []
    for _ in range(4):
        xch.next_epoch()
        dpf.O.zero_()
        n0 = op.launch_count
        op.forward_exchange(dpf, args_f, xch)
        op.check_status()
        assert op.launch_count - n0 == 1, "the fused exchange took the two-kernel route"
        fused.append((dpf.O.cpu().numpy().view(np.uint16).copy(), dpf.lse.cpu().numpy().copy()))
    for O, lse in fused[1:]:
        assert np.array_equal(O, fused[0][0]) and np.array_equal(lse, fused[0][1]), "fused epochs differ"
    util.check_output(fused[0][0], ref, w)
    assert np.abs(fused[0][1] - lse_ref).max() < 2e-3
    mine = torch.from_numpy(fused[0][0].astype(np.int32)).to(dev)
    dist.all_gather_into_tensor(every.view(-1), mine.flatten())
    assert bool((every.view(world, -1) == every.view(world, -1)[0]).all()), "ranks hold different outputs (fused exchange)"
    dist.barrier()
    # a silent peer on the one-launch route: the waiting CTAs give up after 100 ms, O stays untouched
    xch.next_epoch()
    dpf.O.fill_(0x3C00)
    if rank != world - 1:
        op.forward_exchange(dpf, args_f, xch, wait_ms=100)
        try:
            op.check_status()
            raise AssertionError("the fused wait for a silent peer did not report")
        except capi.EspError as e:
            assert "never published" in str(e), str(e)
        assert bool((dpf.O == 0x3C00).all()), "O was written although a peer was missing (fused exchange)"
    torch.cuda.synchronize()
    dist.barrier()
    xch.next_epoch()
    dpf.O.zero_()
    op.forward_exchange(dpf, args_f, xch)
    op.check_status()
    util.check_output(dpf.O.cpu().numpy().view(np.uint16), ref, w)
    dist.barrier()
    # the library-collective route gives the same answer within the tolerance
    rec_local = torch.zeros(op.parts_floats(1), dtype=torch.float32, device=dev)
    rec_world = torch.zeros(world * op.parts_floats(1), dtype=torch.float32, device=dev)
    dp.O.zero_()
    op.forward(dp)
    op.reduce_parts(dp, dp.parts, jobs_dev, len(jobs), rec_local, 0)
    dist.all_gather_into_tensor(rec_world, rec_local)
    op.combine(dp, rec_world, host._dev(shard.world_merge_jobs(1, world), dev), 1)
    op.check_status()
    util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w)
    dist.barrier()
    # A rank that sits a step out (decided on the host: it simply does not launch): the others'
    # wait runs out after 100 ms, they leave O alone and report it; the silent rank reports nothing.
    # The next step, with every rank back, is correct again on the same buffers and contexts.
    xch.next_epoch()
    silent = world - 1
    dp.O.fill_(0x3C00)
    op.forward(dp)
    if rank != silent:
        op.exchange_parts(dp, dp.parts, jobs_dev, len(jobs), xch, parts_max=n_parts, wait_ms=100)
        try:
            op.check_status()
            raise AssertionError("the wait for a silent peer did not report")
        except capi.EspError as e:
            assert "never published" in str(e), str(e)
        assert bool((dp.O == 0x3C00).all()), "O was written although a peer was missing"
    else:
        op.check_status()
    torch.cuda.synchronize()
    dist.barrier()   # the ranks learn of each other on the host before the next launch
    xch.next_epoch()
    dp.O.zero_()
    op.forward(dp)
    op.exchange_parts(dp, dp.parts, jobs_dev, len(jobs), xch, parts_max=n_parts)
    op.check_status()
    util.check_output(dp.O.cpu().numpy().view(np.uint16), ref, w)
    dist.barrier()
    xch.close()
    op.close()
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} fp8={fp8} silent-peer step reported and recovered", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
