"""Host-side integer logic of the pass (KV block pool, target block lists, save entries, row
records) through the C ABI, bit for bit against the restatement of the reference's code in
oracle/forest_ref.py and against hand-derived cases. No GPU needed."""
import ctypes as C

import numpy as np
import pytest

from espetero_b200 import capi
from espetero_b200.workloads import KVSAVE_DT
from oracle import forest_ref as ref


class Pool:
    def __init__(self, n_blocks, bt):
        self.lib = capi.load()
        self.h = C.c_void_p()
        capi.check(self.lib.esp_kv_pool_create(C.byref(self.h), n_blocks, bt))
        self.n, self.bt = n_blocks, bt

    def alloc(self):
        b = C.c_int32()
        capi.check(self.lib.esp_kv_alloc(self.h, C.byref(b)))
        return b.value

    def retain(self, b):
        capi.check(self.lib.esp_kv_retain(self.h, b))

    def release(self, b):
        capi.check(self.lib.esp_kv_release(self.h, b))

    def refs(self):
        return [self.lib.esp_kv_refcount(self.h, b) for b in range(self.n)]

    def free(self):
        return self.lib.esp_kv_free_count(self.h)

    def target_blocks(self, parent, P, w0, end, in_place):
        pa = np.asarray(parent, dtype=np.int32)
        out = np.zeros(max(1, (end + self.bt - 1) // self.bt + len(parent) + 2), dtype=np.int32)
        cow = np.zeros((len(out), 2), dtype=np.int32)
        no, nc = C.c_int32(), C.c_int32()
        rc = self.lib.esp_kv_target_blocks(self.h, pa.ctypes.data if len(pa) else None, len(pa), P, w0, end, int(in_place), out.ctypes.data,
                                           len(out), C.byref(no), cow.ctypes.data, len(cow), C.byref(nc))
        capi.check(rc)
        return list(out[:no.value]), [tuple(x) for x in cow[:nc.value]]

    def new_blocks(self, parent, P, w0, end, in_place):
        pa = np.asarray(parent, dtype=np.int32)
        return self.lib.esp_kv_target_new_blocks(self.h, pa.ctypes.data if len(pa) else None, len(pa), P, w0, end, int(in_place))

    def close(self):
        self.lib.esp_kv_pool_destroy(self.h)


def test_pool_alloc_order_and_refcounts():
    p = Pool(4, 16)
    assert [p.alloc() for _ in range(4)] == [0, 1, 2, 3]          # block 0 is handed out first
    with pytest.raises(capi.EspError) as ei:
        p.alloc()
    assert ei.value.code == capi.ESP_ERR_CAPACITY and "KV cache full" in str(ei.value)
    p.retain(2)
    p.release(2)
    assert p.free() == 0
    p.release(2)
    p.release(0)
    assert p.free() == 2 and p.alloc() == 0 and p.alloc() == 2     # LIFO free list
    with pytest.raises(capi.EspError):
        p.release(1) or p.release(1)
    p.close()


def test_target_blocks_hand_derived():
    # bt 16, parent holds [0, 40) in blocks [0, 1, 2]; a decode step appends position 40 in place:
    # blocks 0, 1 shared, block 2 kept (owned alone) -> nothing allocated, no copy.
    p = Pool(8, 16)
    parent = [p.alloc() for _ in range(3)]
    assert p.new_blocks(parent, 40, 40, 41, True) == 0
    out, cow = p.target_blocks(parent, 40, 40, 41, True)
    assert out == [0, 1, 2] and cow == [] and p.refs()[:3] == [2, 2, 2]
    # the same append into another slot (not in place): block 2 is copied into a new block
    assert p.new_blocks(parent, 40, 40, 41, False) == 1
    out, cow = p.target_blocks(parent, 40, 40, 41, False)
    assert out == [0, 1, 3] and cow == [(2, 3)]
    # position 48 opens a new block: nothing to copy
    out, cow = p.target_blocks(parent, 48, 48, 49, True)
    assert out == [0, 1, 2, 4] and cow == []
    # a full cache leaves the pool untouched
    before, free = p.refs(), p.free()
    with pytest.raises(capi.EspError) as ei:
        p.target_blocks(parent, 40, 40, 40 + 16 * 5, False)
    assert ei.value.code == capi.ESP_ERR_CAPACITY and p.refs() == before and p.free() == free
    p.close()


def test_target_blocks_match_reference_restatement():
    rng = np.random.default_rng(21)
    for case in range(400):
        bt = int(rng.choice([16, 64]))
        n = 40
        a, b = Pool(n, bt), ref.KVPoolRef(n, bt)
        P = int(rng.integers(0, 6 * bt))
        parent = [a.alloc() for _ in range((P + bt - 1) // bt)]
        for _ in parent:
            b.alloc()
        # another slot may share some of the parent's blocks
        for blk in parent:
            if rng.random() < 0.3:
                a.retain(blk)
                b.retain(blk)
        w0 = int(rng.integers(max(0, P - 1), P + 1)) if P else 0
        end = w0 + int(rng.integers(1, 3 * bt))
        in_place = bool(rng.integers(0, 2))
        assert a.new_blocks(parent, P, w0, end, in_place) == ref.target_new_blocks(b, parent, P, w0, end, in_place)
        got = a.target_blocks(parent, P, w0, end, in_place)
        want = ref.target_blocks(b, parent, P, w0, end, in_place)
        assert got[0] == want[0] and got[1] == want[1], case
        assert a.refs() == b.ref and a.free() == len(b.free_list)
        # the blocks allocated are exactly what target_new_blocks promised
        a.close()


def test_save_entries_and_row_table():
    lib = capi.load()
    blocks = np.array([7, 3, 9], dtype=np.int32)
    out = np.zeros(20, dtype=KVSAVE_DT)
    capi.check(lib.esp_kv_save_entries(blocks.ctypes.data, 3, 16, 20, 100, 20, out.ctypes.data))
    want = ref.save_entries(list(blocks), 16, 20, 100, 20)
    assert [tuple(int(v) for v in e) for e in out] == want
    assert tuple(out[0]) == (100, 3, 4, 0) and tuple(out[12]) == (112, 9, 0, 0)
    rc = lib.esp_kv_save_entries(blocks.ctypes.data, 3, 16, 40, 0, 20, out.ctypes.data)
    assert rc == capi.ESP_ERR_INVALID
    # row table: a row saved into the save slot and the work slot has two entries
    ents = np.array([(0, 5, 1, 0), (1, 5, 2, 0), (0, 8, 1, 0)], dtype=KVSAVE_DT)
    table = np.zeros(3 * 4, dtype=np.int32)
    capi.check(lib.esp_kv_row_table(ents.ctypes.data, 3, 3, table.ctypes.data))
    assert list(table) == ref.row_table([tuple(int(v) for v in e) for e in ents], 3) == [5, 1, 8, 1, 5, 2, -1, -1, -1, -1, -1, -1]
    ents3 = np.array([(0, 5, 1, 0), (0, 6, 1, 0), (0, 7, 1, 0)], dtype=KVSAVE_DT)
    assert lib.esp_kv_row_table(ents3.ctypes.data, 3, 1, table.ctypes.data) == capi.ESP_ERR_INVALID


def _tree_rows(root, leaves, base, pnext, root_pos=None, noncausal=False, score_root=False):
    lib = capi.load()
    root_a = np.asarray(root, dtype=np.int32)
    offs = np.zeros(len(leaves) + 1, dtype=np.int32)
    offs[1:] = np.cumsum([len(x) for x in leaves])
    toks = np.asarray([t for x in leaves for t in x] or [0], dtype=np.int32)
    rp = None if root_pos is None else np.asarray(root_pos, dtype=np.int32).reshape(-1)
    i32p = C.POINTER(C.c_int32)
    spec = capi.TreeSpec(root_a.ctypes.data_as(i32p), len(root), len(leaves), None if rp is None else rp.ctypes.data_as(i32p),
                         offs.ctypes.data_as(i32p), toks.ctypes.data_as(i32p), int(noncausal), int(score_root))
    cap = len(root) + int(offs[-1]) + 1
    host = np.zeros(max(1, len(leaves)), np.int32)
    off = np.zeros(max(1, len(leaves)), np.int32)
    tok = np.zeros(cap, np.int32)
    pos = np.zeros((cap, 4), np.int32)
    desc = np.zeros((cap, 4), np.int32)
    read = np.zeros(len(leaves) + 1, np.int32)
    n, nr = C.c_int32(), C.c_int32()
    capi.check(lib.esp_forest_tree_rows(C.byref(spec), base, pnext, host.ctypes.data, off.ctypes.data, tok.ctypes.data, pos.ctypes.data,
                                        desc.ctypes.data, read.ctypes.data, cap, C.byref(n), C.byref(nr)))
    M = n.value
    nread = len(leaves) + (1 if (score_root or not leaves) else 0)
    return dict(host=list(host[:len(leaves)]), off=list(off[:len(leaves)]), tok=list(tok[:M]), pos=pos[:M].tolist(), desc=desc[:M].tolist(),
                readouts=list(read[:nread]), M=M, next_root=nr.value)


def test_tree_rows_hand_derived():
    # verify pass of the engine (src/engine/engine.cpp:3584-3598): a chain of 3 draft tokens given as
    # its three prefixes plus one sibling leaf: the prefixes are hosted by the longest chain.
    got = _tree_rows([11], [[5], [5, 6], [5, 6, 7], [9]], base=10, pnext=100)
    assert got["host"] == [2, 2, 2, 3] and got["off"] == [0, 0, 0, 3] and got["M"] == 1 + 3 + 1
    assert got["tok"] == [11, 5, 6, 7, 9]
    assert got["desc"] == [[0, 0, 0, 0], [1, 0, 1, 0], [1, 0, 1, 0], [1, 0, 1, 0], [4, 0, 1, 0]]
    assert [p[0] for p in got["pos"]] == [100, 101, 102, 103, 101]
    assert got["readouts"] == [10 + 1, 10 + 2, 10 + 3, 10 + 4]
    # plain decode row: the root alone, one readout at its last row
    got = _tree_rows([42], [], base=3, pnext=7)
    assert got["M"] == 1 and got["desc"] == [[0, 0, 0, 0]] and got["readouts"] == [3] and got["next_root"] == 8
    # noncausal root: every row sees the whole root
    got = _tree_rows([1, 2, 3], [], base=0, pnext=0, noncausal=True)
    assert [d[2] for d in got["desc"]] == [3, 3, 3]


def test_tree_rows_match_reference_restatement():
    rng = np.random.default_rng(22)
    for case in range(300):
        Tr = int(rng.integers(1, 6))
        root = [int(x) for x in rng.integers(0, 50, Tr)]
        NL = int(rng.integers(0, 7))
        leaves = []
        for _ in range(NL):
            if leaves and rng.random() < 0.5:   # make prefixes / duplicates likely
                src = leaves[int(rng.integers(0, len(leaves)))]
                k = int(rng.integers(1, len(src) + 1))
                leaf = src[:k] + [int(x) for x in rng.integers(0, 4, int(rng.integers(0, 3)))]
            else:
                leaf = [int(x) for x in rng.integers(0, 4, int(rng.integers(1, 5)))]
            leaves.append(leaf)
        root_pos = None
        if rng.random() < 0.3:
            root_pos = [[int(x) for x in rng.integers(0, 30, 3)] for _ in range(Tr)]
        base, pnext = int(rng.integers(0, 100)), int(rng.integers(0, 1000))
        sr = bool(rng.integers(0, 2))
        got = _tree_rows(root, leaves, base, pnext, root_pos, False, sr)
        want = ref.tree_rows(root, leaves, base, pnext, root_pos, False, sr)
        assert got == want, case


def test_anc_masks():
    lib = capi.load()
    parents = np.array([-1, 0, 0, 1, 3, 2, 5, 5], dtype=np.int32)
    masks = np.zeros(8, dtype=np.uint64)
    capi.check(lib.esp_forest_anc_masks(parents.ctypes.data, 8, masks.ctypes.data))
    assert [int(m) for m in masks] == ref.anc_masks(list(parents))
    assert int(masks[4]) == 0b11011 and int(masks[7]) == 0b10100101
    bad = np.array([-1, 1], dtype=np.int32)
    assert lib.esp_forest_anc_masks(bad.ctypes.data, 2, masks.ctypes.data) == capi.ESP_ERR_INVALID
