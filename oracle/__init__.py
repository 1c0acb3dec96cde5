"""TEST INFRASTRUCTURE: ctypes binding of oracle/oracle.cpp (the CPU restatement of the
reference's attention path). Only tests/, the smoke check and bench.py's CPU-baseline and
reference arms may import this package; the product library never does.

PARITY UNPINNED: the reference has no golden vectors for this path (see oracle.cpp).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")


class Params(C.Structure):
    _fields_ = [("H", C.c_int32), ("Hkv", C.c_int32), ("q_ld", C.c_int32), ("kv_ld", C.c_int32), ("g_ld", C.c_int32),
                ("bt", C.c_int32), ("kv_base", C.c_uint64)]


class Problem(C.Structure):
    _fields_ = [("Q", C.c_void_p), ("Kb", C.c_void_p), ("Vb", C.c_void_p), ("kv", C.c_void_p), ("kv_scales", C.c_void_p),
                ("blocks", C.c_void_p), ("desc", C.c_void_p), ("anc_mask", C.c_void_p), ("X", C.c_void_p), ("trees", C.c_void_p),
                ("n_trees", C.c_int32), ("HD", C.c_int32), ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32),
                ("tile_rows", C.c_int32), ("scale", C.c_float), ("p", Params),
                ("pos", C.c_void_p), ("window", C.c_int32), ("ring", C.c_int32), ("bidi", C.c_int32), ("pad", C.c_int32)]


_lib = None


def build() -> None:
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        lib = C.CDLL(LIB_PATH)
        lib.orc_round_e4m3.restype = C.c_float
        lib.orc_round_e4m3.argtypes = [C.c_float]
        lib.orc_e4m3_encode.restype = C.c_uint8
        lib.orc_e4m3_encode.argtypes = [C.c_float]
        lib.orc_e4m3_decode.restype = C.c_float
        lib.orc_e4m3_decode.argtypes = [C.c_uint8]
        lib.orc_f16_encode.restype = C.c_uint16
        lib.orc_f16_encode.argtypes = [C.c_float]
        lib.orc_f16_decode.restype = C.c_float
        lib.orc_f16_decode.argtypes = [C.c_uint16]
        lib.orc_bf16_encode.restype = C.c_uint16
        lib.orc_bf16_encode.argtypes = [C.c_float]
        lib.orc_bf16_decode.restype = C.c_float
        lib.orc_bf16_decode.argtypes = [C.c_uint16]
        lib.orc_e4m3_encode_n.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.orc_hw_threads.restype = C.c_int
        _lib = lib
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data


def hw_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return load().orc_hw_threads()


def problem(w, tile_rows: int = 8) -> Problem:
    """Problem struct over a workload's host arrays (the arrays must outlive the struct)."""
    pb = Problem()
    pb.Q, pb.Kb, pb.Vb, pb.kv = _p(w.Q), _p(w.Kb), _p(w.Vb), _p(w.kv)
    pb.kv_scales, pb.blocks, pb.X, pb.trees = _p(w.kv_scales), _p(w.blocks), _p(w.X), _p(w.trees)
    pb.desc = _p(w.desc)
    pb.anc_mask = _p(w.anc_mask) if (w.flags & 2) else None
    pb.n_trees, pb.HD, pb.q_dtype, pb.kv_dtype, pb.tile_rows, pb.scale = len(w.trees), w.HD, w.q_dtype, w.kv_dtype, tile_rows, w.scale
    pb.p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    win = w.extra.get("window") if hasattr(w, "extra") else None
    if win:
        pb.pos, pb.window, pb.ring, pb.bidi = _p(win["pos"]), win["window"], win["ring"], win["bidi"]
    return pb


def attention_f64(w, rows=None, threads: int | None = None, with_abs: bool = False):
    """float64 direct softmax. Returns (O [n, H*HD] float64, lse [n, H] float64) for `rows`
    (absolute row indices; None = every row); with_abs adds sum_j softmax_j |v_j|."""
    lib = load()
    pb = problem(w)
    if rows is None:
        rows_a, n = None, w.n_rows
    else:
        rows_a = np.ascontiguousarray(rows, dtype=np.int32)
        n = len(rows_a)
    O = np.zeros((n, w.q_ld), dtype=np.float64)
    lse = np.zeros((n, w.H), dtype=np.float64)
    Oabs = np.zeros((n, w.q_ld), dtype=np.float64) if with_abs else None
    rc = lib.orc_attention_f64(C.byref(pb), C.c_void_p(_p(rows_a)), n, C.c_void_p(O.ctypes.data), C.c_void_p(lse.ctypes.data),
                               C.c_void_p(_p(Oabs)), threads or hw_threads())
    if rc != 0:
        raise RuntimeError("orc_attention_f64: a row belongs to no tree")
    return (O, lse, Oabs) if with_abs else (O, lse)


def _run_kernel(fn, w, tiles, tile_rows, n_parts, threads):
    pb = problem(w, tile_rows)
    tiles = np.ascontiguousarray(tiles)
    O = np.zeros((w.n_rows, w.q_ld), dtype=np.uint16)
    lse = np.full((w.n_rows, w.H), np.nan, dtype=np.float32)
    parts = np.zeros(max(1, n_parts) * w.Hkv * tile_rows * w.G * (w.HD + 2), dtype=np.float32)
    fn(C.byref(pb), C.c_void_p(tiles.ctypes.data), len(tiles), C.c_void_p(O.ctypes.data), C.c_void_p(lse.ctypes.data),
       C.c_void_p(parts.ctypes.data), threads or hw_threads())
    return O, lse, parts


def flash_f32(w, tiles, tile_rows: int = 8, n_parts: int = 0, threads: int | None = None):
    """fp32 restatement of flash_attention over `tiles`. Returns (O bits, lse, parts)."""
    return _run_kernel(load().orc_flash_f32, w, tiles, tile_rows, n_parts, threads)


def decode_gqa_f32(w, tiles, tile_rows: int = 8, n_parts: int = 0, threads: int | None = None):
    """fp32 restatement of attn_decode_gqa over `tiles` (single-row trees)."""
    return _run_kernel(load().orc_decode_gqa_f32, w, tiles, tile_rows, n_parts, threads)


def combine_f32(w, parts, jobs, O, lse, tile_rows: int = 8, threads: int = 1):
    """fp32 restatement of attention_combine; writes rows of O (uint16 bits) and lse in place."""
    p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    jobs = np.ascontiguousarray(jobs)
    load().orc_combine_f32(C.c_void_p(parts.ctypes.data), C.c_void_p(_p(w.X) if (w.flags & 1) else None), C.c_void_p(O.ctypes.data),
                           C.c_void_p(lse.ctypes.data), C.byref(p), w.HD, w.q_dtype, tile_rows, C.c_void_p(jobs.ctypes.data), len(jobs),
                           threads)


def plan_tiles(trees, Hkv, split=512, groups=256, min_chunk=32, tile_rows=8):
    from espetero_b200.workloads import COMBINE_DT, TILE_DT
    lib = load()
    trees = np.ascontiguousarray(trees)
    nt, nj, npart = C.c_int32(), C.c_int32(), C.c_int32()
    lib.orc_plan_tiles(C.c_void_p(trees.ctypes.data), len(trees), Hkv, split, groups, min_chunk, tile_rows, None, None, C.byref(nt),
                       C.byref(nj), C.byref(npart))
    tiles = np.zeros(max(1, nt.value), dtype=TILE_DT)
    jobs = np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    lib.orc_plan_tiles(C.c_void_p(trees.ctypes.data), len(trees), Hkv, split, groups, min_chunk, tile_rows, C.c_void_p(tiles.ctypes.data),
                       C.c_void_p(jobs.ctypes.data), C.byref(nt), C.byref(nj), C.byref(npart))
    return tiles[:nt.value], jobs[:nj.value], npart.value


def g4_plan_tiles(trees, groups, split=512, rows=8, window=0, pos=None):
    from espetero_b200.workloads import COMBINE_DT, TILE_DT
    lib = load()
    trees = np.ascontiguousarray(trees)
    pos = None if pos is None else np.ascontiguousarray(pos, dtype=np.int32)
    nt, nj, npart, pr = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
    lib.orc_g4_plan_tiles(C.c_void_p(trees.ctypes.data), len(trees), groups, split, rows, window, C.c_void_p(_p(pos)), None, None,
                          C.byref(nt), C.byref(nj), C.byref(npart), C.byref(pr))
    tiles = np.zeros(max(1, nt.value), dtype=TILE_DT)
    jobs = np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    lib.orc_g4_plan_tiles(C.c_void_p(trees.ctypes.data), len(trees), groups, split, rows, window, C.c_void_p(_p(pos)),
                          C.c_void_p(tiles.ctypes.data), C.c_void_p(jobs.ctypes.data), C.byref(nt), C.byref(nj), C.byref(npart),
                          C.byref(pr))
    return tiles[:nt.value], jobs[:nj.value], npart.value, pr.value


def kv_save(w, kv, entries):
    p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    entries = np.ascontiguousarray(entries)
    load().orc_kv_save(C.c_void_p(w.Kb.ctypes.data), C.c_void_p(w.Vb.ctypes.data), C.c_void_p(kv.ctypes.data),
                       C.c_void_p(_p(w.kv_scales)), C.c_void_p(entries.ctypes.data), len(entries), C.byref(p), w.HD, w.q_dtype, w.kv_dtype)


class PrepParams(C.Structure):
    _fields_ = [("H", C.c_int32), ("Hkv", C.c_int32), ("ld", C.c_int32), ("q_off", C.c_int32), ("q_stride", C.c_int32),
                ("k_off", C.c_int32), ("v_off", C.c_int32), ("q_ld", C.c_int32), ("kv_ld", C.c_int32), ("rot_half", C.c_int32),
                ("eps", C.c_float), ("qscale", C.c_float), ("bt", C.c_int32), ("reserved", C.c_int32), ("kv_base", C.c_uint64)]


def attn_prep_f64(X, qn_w, kn_w, pos, inv_freq, sel, rows, HD, pp: PrepParams):
    """attn_prep in double (40_attention.metal:23-102 / 82_qwen3_omni.metal:40-88): returns Q64, K64, V64."""
    Q = np.zeros((rows, pp.q_ld), dtype=np.float64)
    K = np.zeros((rows, pp.kv_ld), dtype=np.float64)
    V = np.zeros((rows, pp.kv_ld), dtype=np.float64)
    X, qn_w, kn_w, inv_freq = (np.ascontiguousarray(a, dtype=np.float32) for a in (X, qn_w, kn_w, inv_freq))
    pos, sel = np.ascontiguousarray(pos, dtype=np.int32), np.ascontiguousarray(sel, dtype=np.int32)
    load().orc_attn_prep_f64(C.c_void_p(X.ctypes.data), C.c_void_p(qn_w.ctypes.data), C.c_void_p(kn_w.ctypes.data),
                             C.c_void_p(pos.ctypes.data), C.c_void_p(inv_freq.ctypes.data), C.c_void_p(sel.ctypes.data),
                             C.c_void_p(Q.ctypes.data), C.c_void_p(K.ctypes.data), C.c_void_p(V.ctypes.data), rows, HD, C.byref(pp))
    return Q, K, V


def kv_copy_blocks(w, kv, pairs, region_elems, n_layers):
    p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    pairs = np.ascontiguousarray(pairs, dtype=np.int32)
    load().orc_kv_copy_blocks(C.c_void_p(kv.ctypes.data), C.c_void_p(pairs.ctypes.data), len(pairs), C.byref(p),
                              C.c_uint64(region_elems), n_layers, w.kv_elem_bytes)
