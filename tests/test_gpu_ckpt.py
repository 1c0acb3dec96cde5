"""Checkpoint files of a sequence's KV blocks (slot_save / slot_load, src/model/model.mm:604-740) through
the C ABI: byte layout of the file (header fields, blocks layer-major), round trip into another pool with a
different block list, and the reference's refusals (geometry, size, foreign sections, full cache)."""
import ctypes as C
import struct

import numpy as np
import pytest
import torch

from espetero_b200 import capi

pytestmark = pytest.mark.gpu

HEADER = struct.Struct("<II7i3i5Q2iQ2iQ")   # CkptHeader of the reference, 120 bytes
assert HEADER.size == 120


def _pool(n_layers, n_blocks, block_bytes, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, 256, size=n_layers * n_blocks * block_bytes, dtype=np.uint8)


def _save(path, kv_dev, blocks, length, next_pos, bt, n_layers, region_bytes, block_bytes):
    lib = capi.load()
    b = np.ascontiguousarray(blocks, dtype=np.int32)
    s = torch.cuda.current_stream().cuda_stream
    return lib.esp_kv_slot_save(str(path).encode(), C.c_void_p(s), C.c_void_p(kv_dev.data_ptr()), C.c_void_p(b.ctypes.data), length,
                                next_pos, bt, n_layers, region_bytes, block_bytes)


def _load(path, kv_dev, pool, cap, bt, n_layers, region_bytes, block_bytes):
    lib = capi.load()
    out = np.full(max(cap, 1), -1, dtype=np.int32)
    nb, ln, npos = C.c_int32(-1), C.c_int32(-1), C.c_int32(-1)
    s = torch.cuda.current_stream().cuda_stream
    rc = lib.esp_kv_slot_load(str(path).encode(), C.c_void_p(s), C.c_void_p(kv_dev.data_ptr()), pool, C.c_void_p(out.ctypes.data), cap,
                              C.byref(nb), C.byref(ln), C.byref(npos), bt, n_layers, region_bytes, block_bytes)
    return rc, out, nb.value, ln.value, npos.value


@pytest.mark.parametrize("length", [0, 1, 16, 37, 1000])
def test_checkpoint_layout_and_round_trip(tmp_path, length):
    lib = capi.load()
    bt, kv_ld, n_layers, n_blocks = 16, 512, 3, 80
    block_bytes = 2 * bt * kv_ld * 2                      # K rows + V rows, 16-bit
    region_bytes = n_blocks * block_bytes
    nb = (length + bt - 1) // bt
    host_pool = _pool(n_layers, n_blocks, block_bytes, 1)
    kv = torch.from_numpy(host_pool).cuda()
    blocks = np.random.default_rng(2).permutation(n_blocks)[:nb].astype(np.int32)
    path = tmp_path / "slot.ckpt"
    capi.check(_save(path, kv, blocks, length, length + 3, bt, n_layers, region_bytes, block_bytes))
    raw = path.read_bytes()
    h = HEADER.unpack(raw[:120])
    assert h[0] == 0x554B5043 and h[1] == 4 and h[2] == length and h[3] == length + 3
    assert h[9] == nb and h[10] == n_layers and h[11] == 0 and h[12] == block_bytes
    assert all(v == 0 for v in h[4:9]) and all(v == 0 for v in h[13:])
    assert len(raw) == 120 + nb * n_layers * block_bytes
    body = np.frombuffer(raw, dtype=np.uint8, offset=120).reshape(n_layers, nb, block_bytes) if nb else None
    pool3 = host_pool.reshape(n_layers, n_blocks, block_bytes)
    for l in range(n_layers):
        for i in range(nb):
            assert np.array_equal(body[l, i], pool3[l, blocks[i]])
    # load into an empty pool whose allocator hands out other blocks
    pool = C.c_void_p()
    capi.check(lib.esp_kv_pool_create(C.byref(pool), n_blocks, bt))
    try:
        for _ in range(5):                                 # shift the free list
            blk = C.c_int32()
            capi.check(lib.esp_kv_alloc(pool, C.byref(blk)))
        kv2 = torch.zeros_like(kv)
        free0 = lib.esp_kv_free_count(pool)
        rc, out, got_nb, ln, npos = _load(path, kv2, pool, nb, bt, n_layers, region_bytes, block_bytes)
        capi.check(rc)
        assert (got_nb, ln, npos) == (nb, length, length + 3)
        assert lib.esp_kv_free_count(pool) == free0 - nb
        assert len(set(out[:nb].tolist())) == nb
        got = kv2.cpu().numpy().reshape(n_layers, n_blocks, block_bytes)
        for l in range(n_layers):
            for i in range(nb):
                assert np.array_equal(got[l, out[i]], pool3[l, blocks[i]])
        untouched = np.ones(n_blocks, dtype=bool)
        untouched[out[:nb]] = False
        assert not got[:, untouched].any()
    finally:
        lib.esp_kv_pool_destroy(pool)


def test_checkpoint_refusals(tmp_path):
    lib = capi.load()
    bt, kv_ld, n_layers, n_blocks = 16, 256, 2, 12
    block_bytes = 2 * bt * kv_ld * 2
    region_bytes = n_blocks * block_bytes
    kv = torch.from_numpy(_pool(n_layers, n_blocks, block_bytes, 3)).cuda()
    blocks = np.arange(5, dtype=np.int32)
    good = tmp_path / "good.ckpt"
    capi.check(_save(good, kv, blocks, 70, 70, bt, n_layers, region_bytes, block_bytes))
    raw = bytearray(good.read_bytes())
    pool = C.c_void_p()
    capi.check(lib.esp_kv_pool_create(C.byref(pool), n_blocks, bt))
    try:
        def expect(data, code, **kw):
            p = tmp_path / "bad.ckpt"
            p.write_bytes(bytes(data))
            free0 = lib.esp_kv_free_count(pool)
            rc, *_ = _load(p, kv, pool, kw.get("cap", 16), bt, kw.get("n_layers", n_layers), region_bytes, kw.get("block_bytes", block_bytes))
            assert rc == code, lib.esp_attn_last_error()
            assert lib.esp_kv_free_count(pool) == free0          # nothing taken from the pool

        bad = bytearray(raw); bad[0] ^= 1
        expect(bad, capi.ESP_ERR_INVALID)                         # magic
        bad = bytearray(raw); bad[4] = 3
        expect(bad, capi.ESP_ERR_INVALID)                         # version
        expect(raw[:-16], capi.ESP_ERR_INVALID)                   # truncated
        expect(raw + b"\0" * 16, capi.ESP_ERR_INVALID)            # trailing bytes
        expect(raw, capi.ESP_ERR_INVALID, n_layers=3)             # another model's geometry
        expect(raw, capi.ESP_ERR_INVALID, block_bytes=block_bytes * 2)
        bad = bytearray(raw); struct.pack_into("<i", bad, 44, 2)  # n_linear = 2: linear-layer state present
        expect(bad, capi.ESP_ERR_UNSUPPORTED)
        bad = bytearray(raw); struct.pack_into("<i", bad, 8, 5 * bt + 1)   # len beyond its blocks
        expect(bad, capi.ESP_ERR_INVALID)
        expect(raw, capi.ESP_ERR_CAPACITY, cap=4)                 # caller's list too short
        taken = []
        while lib.esp_kv_free_count(pool) > 4:                    # cache nearly full
            blk = C.c_int32()
            capi.check(lib.esp_kv_alloc(pool, C.byref(blk)))
            taken.append(blk.value)
        expect(raw, capi.ESP_ERR_CAPACITY)
        assert b"KV cache full" in lib.esp_attn_last_error()
        # save-side validation: a block outside the region
        assert _save(tmp_path / "x.ckpt", kv, np.array([n_blocks], dtype=np.int32), 5, 5, bt, n_layers, region_bytes, block_bytes) == capi.ESP_ERR_INVALID
    finally:
        lib.esp_kv_pool_destroy(pool)
