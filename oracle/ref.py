"""TEST INFRASTRUCTURE: loader of oracle/_ref/libplan_ref.so - the reference's own integer host code
(plan_tiles, g4_plan_tiles, the KV pool and target_blocks, kv_row_table, leaf hosting, row records,
block tables), its E4M3 codec and its three per-thread kernels (attention_combine, kv_save,
kv_copy_blocks), compiled from the reference tree by `make -C oracle ref` (extract_ref.py +
ref_glue.cpp). The library exists wherever the reference tree was present at build time and travels
with the working tree; only tests/ load it. Nothing of the reference is stored in the repository."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libplan_ref.so")
REFERENCE_ROOT = os.environ.get("ESPETERO_REFERENCE", "/root/reference")

_lib = None


def reference_present() -> bool:
    return os.path.exists(os.path.join(REFERENCE_ROOT, "src", "model", "impl", "forest.h"))


def build() -> bool:
    """Cut and compile when the reference tree is here; returns whether the library exists."""
    if reference_present():
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={REFERENCE_ROOT}"], check=True, capture_output=True)
    return os.path.exists(LIB_PATH)


def load():
    """The library, or None when it was never built (no reference tree on this machine)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH) and not build():
            return None
        lib = C.CDLL(LIB_PATH)
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_model_create.restype = C.c_void_p
        lib.ref_model_create.argtypes = [C.c_int, C.c_int]
        lib.ref_model_destroy.argtypes = [C.c_void_p]
        for name in ("ref_kv_free",):
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.ref_kv_refcount.argtypes = [C.c_void_p, C.c_int]
        lib.ref_kv_alloc.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        lib.ref_kv_retain.argtypes = [C.c_void_p, C.c_int]
        lib.ref_kv_release.argtypes = [C.c_void_p, C.c_int]
        lib.ref_target_blocks.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                          C.POINTER(C.c_int), C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        lib.ref_target_new_blocks.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        lib.ref_round_e4m3.restype = C.c_float
        lib.ref_round_e4m3.argtypes = [C.c_float]
        lib.ref_e4m3x2.argtypes = [C.c_uint, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.ref_block_tables.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6 + [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_void_p, C.c_int,
                                                                                      C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_void_p,
                                                                                      C.c_int, C.POINTER(C.c_int)]
        lib.ref_kv_copy_blocks.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_ulonglong, C.c_int]
        _lib = lib
    return _lib


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _check(rc):
    if rc != 0:
        raise RuntimeError(load().ref_last_error().decode())


def plan_tiles(trees, Hkv, split=512, groups=256, min_chunk=32, qt=None):
    """The reference's plan_tiles. qt: per tree, per 8-row group, the sparse list id (-1 dense), flattened; None = no sparse attention."""
    from espetero_b200.workloads import COMBINE_DT, TILE_DT
    lib = load()
    trees = np.ascontiguousarray(trees)
    qt = None if qt is None else np.ascontiguousarray(qt, dtype=np.int32)
    nt, nj, npart = C.c_int(), C.c_int(), C.c_int()
    _check(lib.ref_plan_tiles(_p(trees), len(trees), Hkv, split, groups, min_chunk, _p(qt), None, 0, None, 0, C.byref(nt), C.byref(nj), C.byref(npart)))
    tiles, jobs = np.zeros(max(1, nt.value), dtype=TILE_DT), np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    _check(lib.ref_plan_tiles(_p(trees), len(trees), Hkv, split, groups, min_chunk, _p(qt), _p(tiles), len(tiles), _p(jobs), len(jobs), C.byref(nt),
                              C.byref(nj), C.byref(npart)))
    return tiles[:nt.value], jobs[:nj.value], npart.value


def g4_plan_tiles(trees, groups, split=512, rows=8, window=0, pos=None):
    from espetero_b200.workloads import COMBINE_DT, TILE_DT
    lib = load()
    trees = np.ascontiguousarray(trees)
    pos = None if pos is None else np.ascontiguousarray(pos, dtype=np.int32)
    nt, nj, npart, pr = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    _check(lib.ref_g4_plan_tiles(_p(trees), len(trees), groups, split, window, _p(pos), rows, None, 0, None, 0, C.byref(nt), C.byref(nj), C.byref(npart),
                                 C.byref(pr)))
    tiles, jobs = np.zeros(max(1, nt.value), dtype=TILE_DT), np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    _check(lib.ref_g4_plan_tiles(_p(trees), len(trees), groups, split, window, _p(pos), rows, _p(tiles), len(tiles), _p(jobs), len(jobs), C.byref(nt),
                                 C.byref(nj), C.byref(npart), C.byref(pr)))
    return tiles[:nt.value], jobs[:nj.value], npart.value, pr.value


class Pool:
    """The reference's KVPool behind a Model (kv_alloc / kv_retain / kv_release, target_blocks)."""

    def __init__(self, n_blocks, bt):
        self.lib, self.n, self.bt = load(), n_blocks, bt
        self.h = C.c_void_p(self.lib.ref_model_create(n_blocks, bt))

    def alloc(self):
        b = C.c_int()
        _check(self.lib.ref_kv_alloc(self.h, C.byref(b)))
        return b.value

    def retain(self, b):
        self.lib.ref_kv_retain(self.h, b)

    def release(self, b):
        self.lib.ref_kv_release(self.h, b)

    def refs(self):
        return [self.lib.ref_kv_refcount(self.h, b) for b in range(self.n)]

    def free(self):
        return self.lib.ref_kv_free(self.h)

    def target_blocks(self, parent, P, w0, end, in_place):
        pa = np.asarray(parent, dtype=np.int32)
        out = np.zeros(max(1, (end + self.bt - 1) // self.bt + len(parent) + 2), dtype=np.int32)
        cow = np.zeros((len(out), 2), dtype=np.int32)
        no, nc = C.c_int(), C.c_int()
        _check(self.lib.ref_target_blocks(self.h, _p(pa), len(pa), P, w0, end, int(in_place), _p(out), len(out), C.byref(no), _p(cow), len(cow),
                                          C.byref(nc)))
        return list(out[:no.value]), [tuple(x) for x in cow[:nc.value]]

    def new_blocks(self, parent, P, w0, end, in_place):
        pa = np.asarray(parent, dtype=np.int32)
        return self.lib.ref_target_new_blocks(self.h, _p(pa), len(pa), P, w0, end, int(in_place))

    def close(self):
        self.lib.ref_model_destroy(self.h)


def kv_row_table(entries, rows):
    entries = np.ascontiguousarray(entries)
    table = np.zeros(max(rows, 1) * 4, dtype=np.int32)
    _check(load().ref_kv_row_table(_p(entries), len(entries), rows, _p(table)))
    return table


def tree_rows(root, leaves, root_pos=None, noncausal=False, score_root=False, base=0, pnext=0):
    """run_forest's leaf hosting and row records for one tree. Returns dict(host, off, tok, pos, desc, readout, n_rows, next_root)."""
    root = np.ascontiguousarray(root, dtype=np.int32)
    offs = np.zeros(len(leaves) + 1, dtype=np.int32)
    for i, l in enumerate(leaves):
        offs[i + 1] = offs[i] + len(l)
    toks = np.ascontiguousarray([t for l in leaves for t in l] or [0], dtype=np.int32)
    rp = None if root_pos is None else np.ascontiguousarray(root_pos, dtype=np.int32)
    cap = len(root) + int(offs[-1]) + 1
    host, off = np.full(max(1, len(leaves)), -9, dtype=np.int32), np.full(max(1, len(leaves)), -9, dtype=np.int32)
    tok, pos, desc = np.zeros(cap, dtype=np.int32), np.zeros((cap, 4), dtype=np.int32), np.zeros((cap, 4), dtype=np.int32)
    readout = np.full(len(leaves) + 1, -1, dtype=np.int32)
    n_rows, next_root = C.c_int(), C.c_int()
    _check(load().ref_tree_rows(_p(root), len(root), _p(rp), len(leaves), _p(offs), _p(toks), int(noncausal), int(score_root), base, pnext, _p(host),
                                _p(off), _p(tok), _p(pos), _p(desc), _p(readout), C.byref(n_rows), C.byref(next_root)))
    n = n_rows.value
    return dict(host=host[:len(leaves)], off=off[:len(leaves)], tok=tok[:n], pos=pos[:n], desc=desc[:n],
                readout=readout[:len(leaves) + (1 if score_root else 0)], n_rows=n, next_root=next_root.value)


def block_tables(pool: Pool, parents, P, base, save_len, dst_same):
    """run_forest's block tables for targets that continue `parents` (lists of block ids). Returns (table, dst lists, cow pairs, saves)."""
    from espetero_b200.workloads import KVSAVE_DT
    n = len(parents)
    flat = np.ascontiguousarray([b for p in parents for b in p] or [0], dtype=np.int32)
    npar = np.ascontiguousarray([len(p) for p in parents], dtype=np.int32)
    P, base, save_len, dst_same = (np.ascontiguousarray(a, dtype=np.int32) for a in (P, base, save_len, dst_same))
    cap = int(sum(len(p) for p in parents) + sum((int(P[i]) + int(save_len[i])) // pool.bt + 2 for i in range(n)) + 8)
    table, dst, cow = np.zeros(cap, dtype=np.int32), np.zeros(cap, dtype=np.int32), np.zeros((cap, 2), dtype=np.int32)
    n_dst = np.zeros(max(1, n), dtype=np.int32)
    saves = np.zeros(int(save_len.sum()) + 1, dtype=KVSAVE_DT)
    nt, nc, ns = C.c_int(), C.c_int(), C.c_int()
    _check(pool.lib.ref_block_tables(pool.h, n, _p(flat), _p(npar), _p(P), _p(base), _p(save_len), _p(dst_same), _p(table), cap, C.byref(nt), _p(dst), cap,
                                     _p(n_dst), _p(cow), cap, C.byref(nc), _p(saves), len(saves), C.byref(ns)))
    lists, at = [], 0
    for i in range(n):
        lists.append(list(dst[at:at + n_dst[i]]))
        at += int(n_dst[i])
    return list(table[:nt.value]), lists, [tuple(x) for x in cow[:nc.value]], saves[:ns.value]


def round_e4m3(x: float) -> float:
    return float(load().ref_round_e4m3(C.c_float(x)))


def e4m3x2(w: int):
    lo, hi = C.c_float(), C.c_float()
    load().ref_e4m3x2(C.c_uint(w), C.byref(lo), C.byref(hi))
    return lo.value, hi.value


def attention(w, tiles, n_parts: int, which: str = "flash"):
    """The reference's flash_attention<G> ("flash") or attn_decode_gqa<G> ("decode") run by the SIMT emulator over
    `tiles` of a workload (256-dim fp16 heads with gate: the kernels' fixed shape). Returns (O bits, parts)."""
    assert w.HD == 256 and w.q_dtype == 0 and w.kv_dtype == 0 and w.X is not None and w.bt > 0
    from oracle import Params
    tiles = np.ascontiguousarray(tiles)
    O = np.zeros((w.n_rows, w.q_ld), dtype=np.uint16)
    parts = np.zeros(max(1, n_parts) * w.Hkv * 8 * w.G * 258, dtype=np.float32)
    p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    X = np.ascontiguousarray(w.X, dtype=np.float32)
    rc = load().ref_attention(0 if which == "flash" else 1, w.G, _p(w.Q), _p(w.Kb), _p(w.Vb), _p(w.kv), _p(w.blocks), _p(w.desc), _p(X), _p(O),
                              C.byref(p), _p(tiles), len(tiles), _p(w.trees), _p(parts))
    if rc != 0:
        raise RuntimeError(f"the reference does not instantiate G = {w.G}")
    return O, parts


class QsaParams(C.Structure):  # kernels/45_qsa.metal:36-46
    _fields_ = [("ld", C.c_int), ("bt", C.c_int), ("iblk", C.c_int), ("pool_off", C.c_int), ("pos_off", C.c_int), ("nbmax", C.c_int), ("nbw", C.c_int),
                ("eps", C.c_float), ("ibase", C.c_ulonglong)]


def qsa_plan(trees, desc, sparse=True):
    """The reference's qsa_plan: dict(rinfo [M, 4], srows, qtiles [n, 4], qt_of (flattened), counts = M, n_sparse, nbmax, nbb, ncb, n_tiles)."""
    trees = np.ascontiguousarray(trees)
    M = int(max(int(t["base"]) + int(t["M"]) for t in trees))
    groups = int(sum((int(t["M"]) + 7) // 8 for t in trees))
    rinfo, srows = np.zeros((M, 4), dtype=np.int32), np.zeros(max(1, M), dtype=np.int32)
    qtiles, qt_of, counts = np.zeros((max(1, groups), 4), dtype=np.int32), np.zeros(max(1, groups), dtype=np.int32), np.zeros(6, dtype=np.int32)
    d = None if desc is None else np.ascontiguousarray(desc, dtype=np.int32)
    _check(load().ref_qsa_plan(_p(trees), len(trees), _p(d), int(sparse), _p(rinfo), _p(srows), _p(qtiles), _p(qt_of), _p(counts)))
    return dict(rinfo=rinfo, srows=srows[:counts[1]], qtiles=qtiles[:counts[5]], qt_of=qt_of[:groups], counts=[int(x) for x in counts])


def qsa_select(scores, srows, rinfo, nbmax):
    nbw = (nbmax + 31) // 32
    sel = np.zeros((len(srows), nbw), dtype=np.uint32)
    p = QsaParams(0, 16, 0, 0, 0, nbmax, nbw, 1e-6, 0)
    load().ref_qsa_select(_p(np.ascontiguousarray(scores, dtype=np.float32)), _p(np.ascontiguousarray(srows, dtype=np.int32)), _p(rinfo), _p(sel),
                          C.byref(p), len(srows))
    return sel


def qsa_tiles(sel, trees, rinfo, qtiles, nbmax):
    nbw = (nbmax + 31) // 32
    tlist = np.zeros((max(1, len(qtiles)), 4112), dtype=np.uint32)
    tcount = np.zeros(max(1, len(qtiles)), dtype=np.uint32)
    p = QsaParams(0, 16, 0, 0, 0, nbmax, nbw, 1e-6, 0)
    load().ref_qsa_tiles(_p(sel), _p(np.ascontiguousarray(trees)), _p(rinfo), _p(np.ascontiguousarray(qtiles)), len(qtiles), _p(tlist), _p(tcount),
                         C.byref(p))
    return tlist, tcount


def attention_qsa(w, tiles, n_parts, tlist, tcount, rinfo, sel, nbmax):
    """The reference's flash_attention_qsa<G> (SIMT emulator) over `tiles`. Returns (O bits, parts)."""
    assert w.HD == 256 and w.q_dtype == 0 and w.kv_dtype == 0 and w.X is not None
    from oracle import Params
    tiles = np.ascontiguousarray(tiles)
    O = np.zeros((w.n_rows, w.q_ld), dtype=np.uint16)
    parts = np.zeros(max(1, n_parts) * w.Hkv * 8 * w.G * 258, dtype=np.float32)
    p = Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
    qp = QsaParams(0, w.bt, 0, 0, 0, nbmax, (nbmax + 31) // 32, 1e-6, 0)
    X = np.ascontiguousarray(w.X, dtype=np.float32)
    rc = load().ref_attention_qsa(w.G, _p(w.Q), _p(w.Kb), _p(w.Vb), _p(w.kv), _p(w.blocks), _p(w.desc), _p(X), _p(O), C.byref(p), _p(tiles), len(tiles),
                                  _p(w.trees), _p(parts), _p(tlist), _p(tcount), _p(rinfo), _p(sel), C.byref(qp))
    if rc != 0:
        raise RuntimeError(f"the reference does not instantiate G = {w.G}")
    return O, parts
