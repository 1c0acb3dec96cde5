"""The multi-rank host logic on CPU: two gloo ranks shard a workload as bench.py does on GPUs
(sequences by longest-processing-time; one long sequence by KV range), exchange what the GPU
path exchanges (nothing for sequences, one reduced record per rank for split-KV, all-gathered),
and the merged result must equal the single-rank result. The arithmetic is done by the oracle
here: this test is about partitioning, record layout and merge order, not about kernels."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from espetero_b200 import shard, workloads as wl


def test_lpt_partition_and_ranges():
    lens = [32768, 512, 9000, 9000, 100, 20000, 15000, 700]
    parts = shard.lpt_partition(lens, 4)
    assert sorted(i for p in parts for i in p) == list(range(8))
    loads = [sum(lens[i] for i in p) for p in parts]
    assert max(loads) <= 32768 + 100 and max(loads) - min(loads) <= 32768 - min(loads)  # the longest alone bounds it
    assert shard.lpt_partition([5, 5, 5, 5], 2) == [[0, 2], [1, 3]]
    r = shard.split_kv_range(131072, 8, 16)
    assert r[0] == (0, 16384) and r[-1] == (114688, 131072)
    r = shard.split_kv_range(100, 4, 16)          # 7 pages over 4 ranks, cut on page boundaries
    assert r == [(0, 16), (16, 48), (48, 80), (80, 100)]
    assert shard.split_kv_range(10, 4, 16) == [(0, 0), (0, 0), (0, 0), (0, 10)]


def _worker(rank, world, port, q):
    import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- split-KV: one sequence, each rank holds a key range
        P, H, Hkv, HD, bt = 777, 8, 2, 128, 16
        w = wl.make_pass("cpu_split", 5, [(P, 1)], H, Hkv, HD, bt, wl.BF16)
        lo, hi = shard.split_kv_range(P, world, bt)[rank]
        tile = np.zeros(1, dtype=wl.TILE_DT)
        tile[0] = (0, 0, lo, hi, -1, 1, 0, 0)   # the rank's whole range as one unsplit tile
        tiles, jobs, n_parts = shard.local_decode_plan(tile, is_last_rank=(rank == world - 1))
        _, _, parts = oracle.decode_gqa_f32(w, tiles, 8, n_parts, threads=1)
        local = torch.from_numpy(parts.copy())
        gathered = [torch.zeros_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        allrec = torch.cat(gathered).numpy()
        O = np.zeros((1, w.q_ld), dtype=np.uint16)
        lse = np.zeros((1, H), dtype=np.float32)
        oracle.combine_f32(w, allrec, shard.world_merge_jobs(1, world), O, lse, 8)
        ref, lse_ref = oracle.attention_f64(w, threads=1)
        err = float(np.abs(wl.from_bits16(O, wl.BF16) - ref).max())
        # every rank must hold identical bits after the merge
        mine = torch.from_numpy(O.astype(np.int32))
        other = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(other, mine)
        same = all(bool((o == mine).all()) for o in other)
        # ---- sequences: each rank takes its share, nothing is exchanged
        lens = [300, 50, 1000, 640, 16, 900]
        share = shard.lpt_partition(lens, world)[rank]
        q.put((rank, err, same, float(np.abs(lse - lse_ref).max()), share))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_split_kv_and_sequences():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, same, lse_err, share in res:
        assert err <= 2e-3 + 2.0 ** -9 and same and lse_err < 2e-3
    assert sorted(res[0][4] + res[1][4]) == list(range(6))


def test_c_abi_sharding_planners_match_a_python_restatement():
    """esp_shard_lpt / esp_attn_split_kv_ranges / esp_attn_plan_split_kv against the rules stated in
    the header, restated here in a few lines of Python, on random inputs."""
    rng = np.random.default_rng(7)
    for _ in range(50):
        n, world = int(rng.integers(0, 40)), int(rng.integers(1, 9))
        lens = rng.integers(1, 40000, size=n)
        order = sorted(range(n), key=lambda i: (-int(lens[i]), i))
        load, want = [0] * world, [[] for _ in range(world)]
        for i in order:
            r = min(range(world), key=lambda k: (load[k], k))
            want[r].append(i)
            load[r] += int(lens[i])
        assert shard.lpt_partition(lens, world) == [sorted(x) for x in want]
        P, bt = int(rng.integers(0, 200000)), int(rng.choice([16, 32, 64]))
        pages = (P + bt - 1) // bt
        cuts = [(pages * r) // world for r in range(world + 1)]
        assert shard.split_kv_range(P, world, bt) == [(min(P, cuts[r] * bt), min(P, cuts[r + 1] * bt)) for r in range(world)]
    # records-only plan: two row groups, one split in three (tagged for a fused merge), one unsplit
    tiles = np.zeros(4, dtype=wl.TILE_DT)
    tiles[0] = (0, 0, 0, 64, 0, 0, 0, 1)
    tiles[1] = (0, 0, 64, 128, 1, 0, 0, 1)
    tiles[2] = (0, 0, 128, 150, 2, 1, 0, 1)
    tiles[3] = (1, 1, 0, 40, -1, 1, 0, 0)
    for last in (False, True):
        t, jobs, n_parts = shard.local_decode_plan(tiles, is_last_rank=last)
        assert n_parts == 4 and list(t["part"]) == [0, 1, 2, 3] and list(t["pad1"]) == [1, 1, 1, 2]   # every tile names its reduce job
        assert list(t["last"]) == ([0, 0, 1, 1] if last else [0, 0, 0, 0])
        assert [tuple(j) for j in jobs] == [(0, 1, 0, 3), (1, 1, 3, 1)]
    assert [tuple(j) for j in shard.world_merge_jobs(1, 4)] == [(0, 1, 0, 4)]
