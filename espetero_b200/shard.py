"""How the attention path is spread over the GPUs of one box (one process per GPU).

The reference is single-GPU; this is the multi-GPU layer the B200 build adds:
 - independent sequences (batched decode, verify, prefill) go to ranks whole: each rank owns its
   sequences' pages in its own pool and runs its own plan; nothing is exchanged on the data path;
 - one very long sequence is split by KV range: rank r holds the pages of keys [lo_r, hi_r) on
   page boundaries and writes partial records for them; one kernel per rank then reduces them,
   stores the reduced record into every rank's exchange buffer over NVLink peer mappings and
   finishes the merge over the world's records in rank order (esp_attn_exchange_parts), so all
   ranks get identical bits. A library all-gather of the reduced records followed by
   esp_attn_combine_parts is the fallback route where peer mappings cannot be set up.
The integer planning lives in the C library (csrc/shard_host.cpp): these are ctypes calls.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .workloads import COMBINE_DT, TILE_DT


def lpt_partition(lengths, world: int):
    """esp_shard_lpt: sequence -> rank so that the ranks' total context lengths are near equal.
    Returns a list of index lists, one per rank (indices ascending inside a rank)."""
    lens = np.ascontiguousarray(lengths, dtype=np.int64)
    rank_of = np.zeros(max(1, len(lens)), dtype=np.int32)
    capi.check(capi.load().esp_shard_lpt(C.c_void_p(lens.ctypes.data), len(lens), world, C.c_void_p(rank_of.ctypes.data)))
    return [[i for i in range(len(lens)) if rank_of[i] == r] for r in range(world)]


def split_kv_range(P: int, world: int, bt: int):
    """esp_attn_split_kv_ranges: key ranges [lo, hi) per rank, cut on page boundaries."""
    lo, hi = np.zeros(world, dtype=np.int32), np.zeros(world, dtype=np.int32)
    capi.check(capi.load().esp_attn_split_kv_ranges(P, world, bt, C.c_void_p(lo.ctypes.data), C.c_void_p(hi.ctypes.data)))
    return [(int(a), int(b)) for a, b in zip(lo, hi)]


def local_decode_plan(plan_tiles: np.ndarray, is_last_rank: bool):
    """esp_attn_plan_split_kv: a rank's plan over its local key range as "records only".
    Returns (tiles, reduce jobs, n_parts)."""
    lib = capi.load()
    tiles = np.array(plan_tiles, dtype=TILE_DT, copy=True)
    nj, npart = C.c_int32(), C.c_int32()
    jobs = np.zeros(max(1, len(tiles)), dtype=COMBINE_DT)
    capi.check(lib.esp_attn_plan_split_kv(C.c_void_p(tiles.ctypes.data), len(tiles), int(bool(is_last_rank)),
                                          C.c_void_p(jobs.ctypes.data), len(jobs), C.byref(nj), C.byref(npart)))
    return tiles, jobs[:nj.value].copy(), npart.value


def world_merge_jobs(n_row_groups: int, world: int, rows: int = 1):
    """esp_attn_world_merge_jobs: the final merge over the gathered (rank-major) reduced records."""
    jobs = np.zeros(1, dtype=COMBINE_DT)
    nj = C.c_int32()
    capi.check(capi.load().esp_attn_world_merge_jobs(n_row_groups, world, rows, C.c_void_p(jobs.ctypes.data), 1, C.byref(nj)))
    return jobs[:nj.value]
