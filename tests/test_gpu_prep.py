"""attn_prep (kernels/40_attention.metal:23-102; generic kernels/82_qwen3_omni.metal:40-88) through the
C ABI against the double-precision restatement in oracle/: both layouts (gate-interleaved 256-dim heads
with 64 rotated dims; plain 128-dim heads with full rotary and the scale folded into the queries),
M-RoPE position components, the fused pool write (16-bit and E4M3 pools) and argument validation."""
import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl

pytestmark = pytest.mark.gpu


def _case(layout, rows, seed, q_dtype):
    rng = np.random.default_rng(seed)
    if layout == "gated256":
        H, Hkv, HD, rot_half = 16, 2, 256, 32
        q_stride, q_off, k_off = 2 * HD, 0, 2 * H * HD
        qscale = 1.0
    else:
        H, Hkv, HD, rot_half = 32, 4, 128, 64
        q_stride, q_off, k_off = HD, 0, H * HD
        qscale = float(HD) ** -0.5
    v_off = k_off + Hkv * HD
    ld = v_off + Hkv * HD + 8
    X = rng.standard_normal((rows, ld)).astype(np.float32) * rng.uniform(0.2, 3.0, size=(rows, 1)).astype(np.float32)
    qn_w = (1.0 + 0.2 * rng.standard_normal(HD)).astype(np.float32)
    kn_w = (1.0 + 0.2 * rng.standard_normal(HD)).astype(np.float32)
    inv_freq = (1e6 ** (-np.arange(rot_half) / rot_half)).astype(np.float32)
    sel = np.zeros(rot_half, dtype=np.int32)
    sel[rot_half // 4: rot_half // 2] = 1          # M-RoPE sections: temporal, height, width
    sel[rot_half // 2: 3 * rot_half // 4] = 2
    pos = np.zeros((rows, 4), dtype=np.int32)
    pos[:, 0] = rng.integers(0, 200000, size=rows)
    pos[:, 1] = rng.integers(0, 4096, size=rows)
    pos[:, 2] = rng.integers(0, 4096, size=rows)
    pp = capi.PrepParams(H, Hkv, ld, q_off, q_stride, k_off, v_off, H * HD, Hkv * HD, rot_half, 1e-6, qscale, 16, 0, 0)
    return dict(H=H, Hkv=Hkv, HD=HD, X=X, qn_w=qn_w, kn_w=kn_w, inv_freq=inv_freq, sel=sel, pos=pos, pp=pp, q_dtype=q_dtype, rows=rows)


def _ulp16(ref, dtype):
    mant = 10 if dtype == wl.F16 else 7
    mag = np.maximum(np.abs(ref), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(mag)) - mant)


def _run(c, ktab=None, pool=None, scales=None, kv_dtype=None):
    op = host.AttnOp(c["H"], c["Hkv"], c["HD"], 16, c["q_dtype"], c["q_dtype"] if kv_dtype is None else kv_dtype, 1.0)
    try:
        dev = op.device
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        rows, pp = c["rows"], c["pp"]
        Q = torch.zeros((rows, pp.q_ld), dtype=torch.int16, device=dev)
        Kb = torch.zeros((rows, pp.kv_ld), dtype=torch.int16, device=dev)
        Vb = torch.zeros((rows, pp.kv_ld), dtype=torch.int16, device=dev)
        kv = None if pool is None else t(pool)
        op.attn_prep(t(c["X"]), t(c["qn_w"]), t(c["kn_w"]), t(c["pos"]), t(c["inv_freq"]), t(c["sel"]), Q, Kb, Vb, pp,
                     ktab=None if ktab is None else t(ktab), kv=kv, kv_scales=None if scales is None else t(scales))
        op.check_status()
        torch.cuda.synchronize()
        out = [x.cpu().numpy().view(np.uint16) for x in (Q, Kb, Vb)]
        return out + [None if kv is None else kv.cpu().numpy()]
    finally:
        op.close()


@pytest.mark.parametrize("layout", ["gated256", "plain128"])
@pytest.mark.parametrize("q_dtype", [wl.F16, wl.BF16], ids=["f16", "bf16"])
def test_prep_matches_oracle(oracle_lib, layout, q_dtype):
    c = _case(layout, 37, 5, q_dtype)
    Q64, K64, V64 = oracle_lib.attn_prep_f64(c["X"], c["qn_w"], c["kn_w"], c["pos"], c["inv_freq"], c["sel"], c["rows"], c["HD"], c["pp"])
    Q, Kb, Vb, _ = _run(c)
    for got_bits, ref, name in ((Q, Q64, "Q"), (Kb, K64, "K")):
        got = wl.from_bits16(got_bits, q_dtype).astype(np.float64)
        # fp32 arithmetic, then one rounding to 16 bits: within 0.51 output ulp of the double result, plus the
        # fp32 error of the head's arithmetic, which is relative to the head's largest element (a rotation
        # can cancel two large terms into a small one)
        head_max = np.abs(ref).reshape(ref.shape[0], -1, c["HD"]).max(axis=2, keepdims=True)
        head_max = np.broadcast_to(head_max, (ref.shape[0], head_max.shape[1], c["HD"])).reshape(ref.shape)
        allow = 0.51 * _ulp16(ref, q_dtype) + 2e-6 * head_max + 1e-9
        err = np.abs(got - ref)
        assert (err <= allow).all(), f"{name}: {int((err > allow).sum())} elements off, worst {err.max():.3e}"
    # values are a plain cast: bit-exact
    pp = c["pp"]
    Vx = c["X"][:, pp.v_off: pp.v_off + pp.kv_ld]
    assert np.array_equal(Vb, wl.to_bits16(Vx, q_dtype))
    assert np.array_equal(wl.to_bits16(V64.astype(np.float32), q_dtype), Vb)


@pytest.mark.parametrize("layout", ["gated256", "plain128"])
def test_prep_writes_the_pool_rows(layout):
    """ktab: (block, pos, block2, pos2) per row; the pool entries must hold the Kb / Vb bits, rows
    without an entry leave the pool alone."""
    c = _case(layout, 9, 6, wl.BF16)
    pp = c["pp"]
    n_blocks, bt = 7, 16
    pp.bt, pp.kv_base = bt, 2 * n_blocks * bt * pp.kv_ld      # second layer region
    pool = np.full(2 * 2 * n_blocks * bt * pp.kv_ld, 0x7777, dtype=np.uint16)
    ktab = np.full((c["rows"], 4), -1, dtype=np.int32)
    ktab[0] = (3, 5, -1, -1)
    ktab[1] = (3, 6, 6, 0)         # saved into two slots
    ktab[4] = (0, 15, -1, -1)
    ktab[8] = (-1, -1, 2, 2)
    Q, Kb, Vb, kv = _run(c, ktab=ktab, pool=pool.view(np.int16))
    kv = kv.view(np.uint16)
    expect = pool.copy()
    blk = bt * pp.kv_ld
    for r in range(c["rows"]):
        for b, ps in ((ktab[r, 0], ktab[r, 1]), (ktab[r, 2], ktab[r, 3])):
            if b < 0:
                continue
            dst = pp.kv_base + b * 2 * blk + ps * pp.kv_ld
            expect[dst: dst + pp.kv_ld] = Kb[r]
            expect[dst + blk: dst + blk + pp.kv_ld] = Vb[r]
    assert np.array_equal(kv, expect)


def test_prep_e4m3_pool_matches_kv_save(oracle_lib):
    """With an E4M3 pool the fused write must give the codes esp_kv_save gives for the same rows."""
    c = _case("gated256", 6, 7, wl.BF16)
    pp = c["pp"]
    n_blocks, bt = 5, 16
    pp.bt, pp.kv_base = bt, 0
    rng = np.random.default_rng(1)
    scales = np.exp2(rng.uniform(-4, 2, size=(n_blocks, 2, c["Hkv"]))).astype(np.float32)
    pool = np.full(2 * n_blocks * bt * pp.kv_ld, 0x11, dtype=np.uint8)
    ktab = np.array([(1, 0, -1, -1), (1, 1, 4, 7), (-1, -1, -1, -1), (0, 3, -1, -1), (2, 15, -1, -1), (3, 8, 3, 9)], dtype=np.int32)
    Q, Kb, Vb, kv = _run(c, ktab=ktab, pool=pool, scales=scales, kv_dtype=wl.E4M3)
    expect = pool.copy()
    blk = bt * pp.kv_ld
    Kf, Vf = wl.from_bits16(Kb, wl.BF16), wl.from_bits16(Vb, wl.BF16)
    for r in range(c["rows"]):
        for b, ps in ((ktab[r, 0], ktab[r, 1]), (ktab[r, 2], ktab[r, 3])):
            if b < 0:
                continue
            dst = b * 2 * blk + ps * pp.kv_ld
            sk = np.repeat(scales[b, 0], c["HD"])
            sv = np.repeat(scales[b, 1], c["HD"])
            expect[dst: dst + pp.kv_ld] = wl.e4m3_encode((Kf[r] / sk).astype(np.float32))
            expect[dst + blk: dst + blk + pp.kv_ld] = wl.e4m3_encode((Vf[r] / sv).astype(np.float32))
    assert np.array_equal(kv, expect)


def test_prep_validation():
    c = _case("plain128", 2, 8, wl.BF16)
    c["pp"].rot_half = 48                      # not a power of two
    with pytest.raises(capi.EspError) as e:
        _run(c)
    assert e.value.code == capi.ESP_ERR_INVALID
    c = _case("plain128", 2, 8, wl.BF16)
    c["pp"].k_off += 2                         # not a multiple of 4 floats
    with pytest.raises(capi.EspError) as e:
        _run(c)
    assert e.value.code == capi.ESP_ERR_INVALID
