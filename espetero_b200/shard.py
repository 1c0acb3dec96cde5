"""How the attention path is spread over the GPUs of one box (one process per GPU).

The reference is single-GPU; this is the multi-GPU layer the B200 build adds:
 - independent sequences (batched decode, verify, prefill) go to ranks whole: each rank owns its
   sequences' pages in its own pool and runs its own plan; nothing is exchanged on the data path;
 - one very long sequence is split by KV range: rank r holds the pages of keys
   [lo_r, hi_r) on page boundaries, writes partial records for them, reduces them to one record
   per (row, head), the ranks all-gather those records and every rank finishes the merge
   (esp_attn_combine_parts) over the world's records in rank order, so all ranks get identical bits.
Pure integer helpers; no GPU needed.
"""
from __future__ import annotations

import numpy as np

from .workloads import COMBINE_DT, TILE_DT


def lpt_partition(lengths, world: int):
    """Longest-processing-time greedy: sequence -> rank so that the ranks' total context lengths are
    near equal. Returns a list of index lists, one per rank (indices ascending inside a rank)."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def split_kv_range(P: int, world: int, bt: int):
    """Key ranges [lo, hi) per rank, cut on page boundaries, pages spread as evenly as possible."""
    pages = (P + bt - 1) // bt
    cuts = [(pages * r) // world for r in range(world + 1)]
    return [(min(P, cuts[r] * bt), min(P, cuts[r + 1] * bt)) for r in range(world)]


def local_decode_plan(plan_tiles: np.ndarray, is_last_rank: bool):
    """Turn a rank's plan over its local key range into "records only": every tile writes a partial
    record (unsplit tiles get one), only the rank that holds the end of the sequence keeps the
    `last` flag (the row's own batch key is counted once), and ONE reduce job per row group merges
    the rank's records. Returns (tiles, jobs, n_parts)."""
    tiles = np.array(plan_tiles, dtype=TILE_DT, copy=True)
    n_parts = int(tiles["part"].max()) + 1 if len(tiles) and tiles["part"].max() >= 0 else 0
    for t in tiles:
        if t["part"] < 0:
            t["part"] = n_parts
            n_parts += 1
        if not is_last_rank:
            t["last"] = 0
    jobs = []
    groups = {}
    for t in tiles:
        groups.setdefault((int(t["tree"]), int(t["r0"])), []).append(int(t["part"]))
    for (tree, r0), parts in sorted(groups.items()):
        parts.sort()
        assert parts == list(range(parts[0], parts[0] + len(parts))), "a row group's records must be consecutive"
        jobs.append((r0, 1, parts[0], len(parts)))
    return tiles, np.array(jobs, dtype=COMBINE_DT), n_parts


def world_merge_jobs(n_row_groups: int, world: int, rows: int = 1):
    """The final merge over the gathered records: rank r's reduced record of row group g is record
    r * n_row_groups + g; merging needs them consecutive per group, so the gathered buffer is laid
    out group-major by the caller when n_row_groups > 1. For one row group: one job over records
    0 .. world-1."""
    assert n_row_groups == 1, "split-KV sharding is used for a single long sequence"
    return np.array([(0, rows, 0, world)], dtype=COMBINE_DT)
