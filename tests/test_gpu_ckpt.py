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


def _save(path, kv_dev, blocks, length, next_pos, bt, n_layers, region_bytes, block_bytes, scales=None, Hkv=0, scales_region=0):
    lib = capi.load()
    b = np.ascontiguousarray(blocks, dtype=np.int32)
    s = torch.cuda.current_stream().cuda_stream
    sp = None if scales is None else C.c_void_p(scales.data_ptr())
    return lib.esp_kv_slot_save(str(path).encode(), C.c_void_p(s), C.c_void_p(kv_dev.data_ptr()), C.c_void_p(b.ctypes.data), length,
                                next_pos, bt, n_layers, region_bytes, block_bytes, sp, Hkv, scales_region)


def _load(path, kv_dev, pool, cap, bt, n_layers, region_bytes, block_bytes, scales=None, Hkv=0, scales_region=0):
    lib = capi.load()
    out = np.full(max(cap, 1), -1, dtype=np.int32)
    nb, ln, npos = C.c_int32(-1), C.c_int32(-1), C.c_int32(-1)
    s = torch.cuda.current_stream().cuda_stream
    sp = None if scales is None else C.c_void_p(scales.data_ptr())
    rc = lib.esp_kv_slot_load(str(path).encode(), C.c_void_p(s), C.c_void_p(kv_dev.data_ptr()), pool, C.c_void_p(out.ctypes.data), cap,
                              C.byref(nb), C.byref(ln), C.byref(npos), bt, n_layers, region_bytes, block_bytes, sp, Hkv, scales_region)
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


def test_checkpoint_e4m3_pool_carries_its_block_scales(tmp_path):
    """An E4M3 pool's file holds the blocks' scale rows too: loaded into other block ids of a pool whose
    scale table is full of other values, the sequence's blocks get their own scales back; pools with and
    without scales refuse each other's files."""
    lib = capi.load()
    bt, Hkv, HD, n_layers, n_blocks, length = 16, 4, 128, 2, 40, 150
    kv_ld = Hkv * HD
    block_bytes = 2 * bt * kv_ld                           # one byte per element
    region_bytes = n_blocks * block_bytes
    srow = 2 * Hkv
    sregion = n_blocks * srow
    nb = (length + bt - 1) // bt
    host_pool = _pool(n_layers, n_blocks, block_bytes, 11)
    rng = np.random.default_rng(12)
    host_scales = rng.uniform(0.1, 4.0, size=(n_layers, n_blocks, srow)).astype(np.float32)
    kv, scales = torch.from_numpy(host_pool).cuda(), torch.from_numpy(host_scales).cuda()
    blocks = rng.permutation(n_blocks)[:nb].astype(np.int32)
    path = tmp_path / "fp8.ckpt"
    capi.check(_save(path, kv, blocks, length, length, bt, n_layers, region_bytes, block_bytes, scales, Hkv, sregion))
    raw = path.read_bytes()
    h = HEADER.unpack(raw[:120])
    assert h[18] == srow * 4                               # the word the reference leaves at zero
    assert len(raw) == 120 + nb * n_layers * (block_bytes + srow * 4)
    tail = np.frombuffer(raw, dtype=np.float32, offset=120 + nb * n_layers * block_bytes).reshape(n_layers, nb, srow)
    for l in range(n_layers):
        assert np.array_equal(tail[l], host_scales[l, blocks])
    pool = C.c_void_p()
    capi.check(lib.esp_kv_pool_create(C.byref(pool), n_blocks, bt))
    try:
        for _ in range(7):
            blk = C.c_int32()
            capi.check(lib.esp_kv_alloc(pool, C.byref(blk)))
        kv2 = torch.zeros_like(kv)
        scales2 = torch.full_like(scales, -7.0)            # what earlier users of the blocks left behind
        # a 16-bit pool (no scales) refuses the file, and a scaled pool refuses a file without them
        rc, *_ = _load(path, kv2, pool, nb, bt, n_layers, region_bytes, block_bytes)
        assert rc == capi.ESP_ERR_INVALID
        plain = tmp_path / "plain.ckpt"
        capi.check(_save(plain, kv, blocks, length, length, bt, n_layers, region_bytes, block_bytes))
        rc, *_ = _load(plain, kv2, pool, nb, bt, n_layers, region_bytes, block_bytes, scales2, Hkv, sregion)
        assert rc == capi.ESP_ERR_INVALID
        rc, out, got_nb, ln, _ = _load(path, kv2, pool, nb, bt, n_layers, region_bytes, block_bytes, scales2, Hkv, sregion)
        capi.check(rc)
        assert got_nb == nb and ln == length and not set(out[:nb].tolist()) & set(range(7))
        got_kv = kv2.cpu().numpy().reshape(n_layers, n_blocks, block_bytes)
        got_sc = scales2.cpu().numpy()
        pool3 = host_pool.reshape(n_layers, n_blocks, block_bytes)
        for l in range(n_layers):
            for i in range(nb):
                assert np.array_equal(got_kv[l, out[i]], pool3[l, blocks[i]])
                assert np.array_equal(got_sc[l, out[i]], host_scales[l, blocks[i]])
        untouched = np.ones(n_blocks, dtype=bool)
        untouched[out[:nb]] = False
        assert (got_sc[:, untouched] == -7.0).all()
    finally:
        lib.esp_kv_pool_destroy(pool)
