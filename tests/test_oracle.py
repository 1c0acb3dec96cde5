"""The oracle against itself: the fp32 restatements of the reference kernels
(flash_attention, attn_decode_gqa, attention_combine; kernels/40_attention.metal:156-343,
:598-781, :811-864) must agree with the float64 direct softmax within the stated
tolerance, and integer-exact identity probes must come out exact."""
import numpy as np
import pytest

from espetero_b200 import workloads as wl
from tests import util


def _decode_cases():
    return [
        dict(name="c1", trees=[(1024, 1)], H=8, Hkv=2, HD=128, dt=wl.F16, kvdt=None),
        dict(name="c2_small", trees=[(p, 1) for p in (512, 777, 16, 33, 2048)], H=32, Hkv=4, HD=128, dt=wl.BF16, kvdt=None),
        dict(name="c5_small", trees=[(4096, 1)], H=32, Hkv=8, HD=256, dt=wl.BF16, kvdt=wl.E4M3),
        dict(name="hd256_f16_gate", trees=[(300, 1), (0, 1)], H=16, Hkv=4, HD=256, dt=wl.F16, kvdt=None, gate=True),
    ]


@pytest.mark.parametrize("case", _decode_cases(), ids=lambda c: c["name"])
def test_decode_restatements_match_f64(oracle_lib, case):
    w = wl.make_pass(case["name"], 101, case["trees"], case["H"], case["Hkv"], case["HD"], 16, case["dt"], case["kvdt"],
                     gate=case.get("gate", False))
    ref, lse_ref = oracle_lib.attention_f64(w)
    tiles, jobs, nparts = oracle_lib.plan_tiles(w.trees, w.Hkv, split=512)
    for fn in (oracle_lib.decode_gqa_f32, oracle_lib.flash_f32):
        O, lse, parts = fn(w, tiles, 8, nparts)
        if len(jobs):
            oracle_lib.combine_f32(w, parts, jobs, O, lse, 8)
        util.check_output(O, ref, w, what=f"{fn.__name__}")
        fin = np.isfinite(lse_ref)
        assert np.abs(lse[fin] - lse_ref[fin]).max() < 2e-3


@pytest.mark.parametrize("mask", ["causal", "forest", "tree"])
def test_flash_restatement_masks(oracle_lib, mask):
    w = wl.make_pass("forest", 202, [(40, 20), (0, 9), (100, 16)], 8, 2, 128, 16, wl.BF16, mask=mask)
    ref, _, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    tiles, jobs, nparts = oracle_lib.plan_tiles(w.trees, w.Hkv, split=512)
    O, lse, parts = oracle_lib.flash_f32(w, tiles, 8, nparts)
    if len(jobs):
        oracle_lib.combine_f32(w, parts, jobs, O, lse, 8)
    util.check_output(O, ref, w, ref_abs=ref_abs)


def test_tree_mask_equals_path_flattening(oracle_lib):
    """A general draft tree through the ancestor bit mask gives, per node, the result of the
    reference's own form: the root-to-node path flattened into a causal chain
    (src/engine/engine.cpp:3584-3598 builds leaves as paths; duplicated ancestors carry the
    same K/V so the two forms are mathematically equal)."""
    P, M = 48, 12
    w = wl.make_pass("tree", 303, [(P, M)], 8, 2, 128, 16, wl.BF16, mask="tree")
    ref, _ = oracle_lib.attention_f64(w)
    par = w.extra["parents"][0]
    for node in range(M):
        path = []
        k = node
        while k >= 0:
            path.append(k)
            k = par[k]
        path = path[::-1]
        w2 = wl.make_pass("path", 303, [(P, len(path))], 8, 2, 128, 16, wl.BF16, mask="causal")
        w2.kv, w2.blocks = w.kv, w.blocks
        w2.Q, w2.Kb, w2.Vb = w.Q[path].copy(), w.Kb[path].copy(), w.Vb[path].copy()
        ref2, _ = oracle_lib.attention_f64(w2, rows=[len(path) - 1])
        assert np.abs(ref2[0] - ref[node]).max() < 1e-12


def test_identity_probe_exact(oracle_lib):
    """Q = 0 makes every visible key weigh exp(0) = 1, so the unnormalised record is the exact
    integer sum of the visible V rows: V carries the key index in base 16 over three dims plus a
    per-node indicator, all exactly representable in bf16, and any page-table or mask error
    changes an integer."""
    P, M, H, Hkv, HD, bt = 200, 7, 4, 2, 128, 16
    w = wl.make_pass("probe", 404, [(P, M)], H, Hkv, HD, bt, wl.BF16, mask="tree")
    w.Q[:] = 0
    pool = np.zeros((w.n_blocks, 2, bt, Hkv, HD), dtype=np.float32)
    for j in range(P):
        b = int(w.blocks[j // bt])
        for kvh in range(Hkv):
            pool[b, 1, j % bt, kvh, 0:3] = [j % 16, (j // 16) % 16, j // 256]
            pool[b, 1, j % bt, kvh, 3] = kvh + 1
    w.kv = wl.f32_to_bf16_bits(pool.reshape(-1))
    vb = np.zeros((M, Hkv, HD), dtype=np.float32)
    for n in range(M):
        vb[n, :, 8 + n] = 1.0
    w.Vb = wl.f32_to_bf16_bits(vb.reshape(M, -1))
    tiles, jobs, nparts = oracle_lib.plan_tiles(w.trees, w.Hkv, split=0)
    tiles = tiles.copy()
    tiles["part"] = np.arange(len(tiles))
    O, lse, parts = oracle_lib.flash_f32(w, tiles, 8, len(tiles))
    rec = parts.reshape(-1, HD + 2)
    par = w.extra["parents"][0]
    for node in range(M):
        anc = set()
        k = node
        while k >= 0:
            anc.add(k)
            k = par[k]
        for h in range(H):
            kvh, hg = h // (H // Hkv), h % (H // Hkv)
            r = rec[(0 * Hkv + kvh) * 8 * (H // Hkv) + node * (H // Hkv) + hg]
            assert r[HD] == 0.0 and r[HD + 1] == P + len(anc)
            assert r[0] == sum(j % 16 for j in range(P)) and r[1] == sum((j // 16) % 16 for j in range(P))
            assert r[2] == sum(j // 256 for j in range(P)) and r[3] == (kvh + 1) * P
            assert [int(r[8 + n]) for n in range(M)] == [1 if n in anc else 0 for n in range(M)]


def test_kv_save_and_copy(oracle_lib):
    w = wl.make_pass("save", 505, [(0, 40)], 8, 2, 128, 16, wl.BF16, spare_blocks=6)
    kv = w.kv.copy()
    entries = np.zeros(40, dtype=wl.KVSAVE_DT)
    for i in range(40):
        entries[i] = (i, 5 - i // 16, i % 16, 0)
    oracle_lib.kv_save(w, kv, entries)
    pool = kv.reshape(w.n_blocks, 2, 16, w.kv_ld)
    for i in range(40):
        assert np.array_equal(pool[5 - i // 16, 0, i % 16], w.Kb[i]) and np.array_equal(pool[5 - i // 16, 1, i % 16], w.Vb[i])
    oracle_lib.kv_copy_blocks(w, kv, np.array([[5, 0], [4, 1]], dtype=np.int32), kv.size, 1)
    assert np.array_equal(pool[0], pool[5]) and np.array_equal(pool[1], pool[4])
    # E4M3 pool: the saved codes are e4m3(x / scale of the destination block)
    w8 = wl.make_pass("save8", 506, [(0, 16)], 8, 2, 128, 16, wl.BF16, kv_dtype=wl.E4M3, spare_blocks=2)
    kv8 = w8.kv.copy()
    e8 = np.zeros(16, dtype=wl.KVSAVE_DT)
    for i in range(16):
        e8[i] = (i, 1, i, 0)
    oracle_lib.kv_save(w8, kv8, e8)
    pool8 = kv8.reshape(w8.n_blocks, 2, 16, 2, 128)
    x = wl.bf16_bits_to_f32(w8.Kb).reshape(16, 2, 128)
    want = wl.e4m3_encode(x / w8.kv_scales[1, 0][None, :, None])
    assert np.array_equal(pool8[1, 0] & 0x7F, want & 0x7F)


def test_attn_prep_oracle_against_numpy(oracle_lib):
    """The C restatement of attn_prep (40_attention.metal:23-102) against the same formulas written
    with numpy arrays: RMSNorm, rotary pairs (d, d + rot_half) with the M-RoPE component per frequency."""
    import oracle
    rng = np.random.default_rng(3)
    H, Hkv, HD, rot_half, rows = 4, 2, 128, 32, 5
    q_stride, k_off = 2 * HD, 2 * H * HD
    v_off = k_off + Hkv * HD
    ld = v_off + Hkv * HD
    X = rng.standard_normal((rows, ld)).astype(np.float32)
    qn, kn = rng.uniform(0.5, 1.5, HD).astype(np.float32), rng.uniform(0.5, 1.5, HD).astype(np.float32)
    inv_freq = (10000.0 ** (-np.arange(rot_half) / rot_half)).astype(np.float32)
    sel = (np.arange(rot_half) % 3).astype(np.int32)
    pos = rng.integers(0, 5000, size=(rows, 4)).astype(np.int32)
    pp = oracle.PrepParams(H, Hkv, ld, 0, q_stride, k_off, v_off, H * HD, Hkv * HD, rot_half, 1e-5, 0.25, 16, 0, 0)
    Q, K, V = oracle.attn_prep_f64(X, qn, kn, pos, inv_freq, sel, rows, HD, pp)

    def head(x, w, r):
        x = x.astype(np.float64)
        y = x / np.sqrt((x * x).mean() + np.float64(np.float32(1e-5))) * w
        ang = (pos[r, sel].astype(np.float32) * inv_freq).astype(np.float64)   # fp32 product, as the kernels form it
        lo, hi = y[:rot_half].copy(), y[rot_half:2 * rot_half].copy()
        y[:rot_half] = lo * np.cos(ang) - hi * np.sin(ang)
        y[rot_half:2 * rot_half] = hi * np.cos(ang) + lo * np.sin(ang)
        return y

    for r in range(rows):
        for h in range(H):
            np.testing.assert_allclose(Q[r, h * HD:(h + 1) * HD], 0.25 * head(X[r, h * q_stride: h * q_stride + HD], qn, r), rtol=1e-12, atol=1e-12)
        for h in range(Hkv):
            np.testing.assert_allclose(K[r, h * HD:(h + 1) * HD], head(X[r, k_off + h * HD: k_off + (h + 1) * HD], kn, r), rtol=1e-12, atol=1e-12)
    np.testing.assert_array_equal(V, X[:, v_off: v_off + Hkv * HD].astype(np.float64))
