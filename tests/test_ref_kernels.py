"""The floating-point side pinned to the reference's OWN kernels. oracle/_ref/libplan_ref.so also holds
attn_prep, flash_attention<G> and attn_decode_gqa<G> of kernels/40_attention.metal, cut from the reference
tree and compiled as C++ over a small SIMT emulator (oracle/ref_simt.h: every GPU thread a fiber;
threadgroup barriers, simdgroup shuffles and 8 x 8 matrix products as rendezvous points). They are the
256-dim, fp16, gated originals. Checked here, on the CPU:
  - the float64 oracle agrees with what those kernels compute, within the stated tolerance, over decode,
    prefill, forest masks, noncausal roots, split tiles merged by the reference's own attention_combine,
    short tails, several block sizes and every instantiated G;
  - the oracle's fp32 restatements follow them: flash to the last fp16 bit (records: every fp32 bit) but for
    isolated rounding ties, decode to a few fp32 ulps (its dims are permuted inside the products, which
    changes the order of additions);
  - attn_prep's restatement in double agrees with the emulated kernel to half an fp16 ulp.
tests/golden/ref_kernels.npz holds outputs of these runs for machines without the reference tree and for
the GPU tests (tests/test_gpu_ref_kernels.py)."""
import ctypes as C

import numpy as np
import pytest

from espetero_b200 import workloads as wl
from oracle import ref

pytestmark = pytest.mark.skipif(ref.load() is None, reason="oracle/_ref/libplan_ref.so was not built (no reference tree on this machine)")

TOL = 2e-3


def half_ulp16(x):
    return np.exp2(np.floor(np.log2(np.maximum(np.abs(x), 2.0 ** -14))) - 11)


def ref_forward(w, split=512, groups=256, which=None):
    """The pass as the reference runs it: plan_tiles, the attention kernel its dispatch would pick
    (src/model/impl/forest.h:2864-2868), attention_combine. Returns (O bits, plan)."""
    tiles, jobs, n_parts = ref.plan_tiles(w.trees, w.Hkv, split, groups)
    single = all(int(t["M"]) == 1 for t in w.trees)
    O, parts = ref.attention(w, tiles, n_parts, which or ("decode" if single else "flash"))
    if len(jobs):
        import oracle
        p = oracle.Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)
        X = np.ascontiguousarray(w.X, dtype=np.float32)
        ref.load().ref_attention_combine(C.c_void_p(parts.ctypes.data), C.c_void_p(X.ctypes.data), C.c_void_p(O.ctypes.data), C.byref(p),
                                         C.c_void_p(np.ascontiguousarray(jobs).ctypes.data), len(jobs))
    return O, (tiles, jobs, n_parts), parts


CASES = {
    # name: (trees [(P, M)], H, Hkv, bt, mask, planner split, planner groups)
    "decode_g4": ([(1024, 1)], 8, 2, 16, "causal", 512, 256),
    "decode_g8_batch": ([(300, 1), (17, 1), (0, 1), (1000, 1), (64, 1)], 16, 2, 16, "causal", 512, 256),
    "decode_g1_bt64": ([(130, 1), (63, 1)], 2, 2, 64, "causal", 512, 256),
    "decode_g6_unsplit": ([(77, 1), (8, 1), (1, 1)], 6, 1, 16, "causal", 0, 256),
    "decode_g3": ([(200, 1)], 3, 1, 32, "causal", 512, 64),
    "prefill_g2": ([(0, 37), (0, 8)], 4, 2, 16, "causal", 512, 256),
    "chunked_g4": ([(90, 20), (16, 9)], 8, 2, 16, "causal", 512, 256),
    "forest_g8": ([(40, 12), (0, 9), (100, 16), (33, 1)], 8, 1, 16, "forest", 512, 256),
    "verify_split_g4": ([(700, 12)], 4, 1, 16, "forest", 128, 1024),
}


def make_case(name):
    trees, H, Hkv, bt, mask, split, groups = CASES[name]
    seed = 7000 + sorted(CASES).index(name)
    return wl.make_pass(name, seed, trees, H, Hkv, 256, bt, wl.F16, gate=True, scale=1.0 / 16.0, mask=mask), split, groups


@pytest.mark.parametrize("name", sorted(CASES))
def test_float64_oracle_agrees_with_the_reference_kernels(oracle_lib, name):
    w, split, groups = make_case(name)
    O, (tiles, jobs, n_parts), _ = ref_forward(w, split, groups)
    if name in ("decode_g4", "verify_split_g4"):
        assert n_parts > 0                                  # split tiles, merged by the reference's attention_combine
    want, _ = oracle_lib.attention_f64(w)
    got = wl.f16_bits_to_f32(O).astype(np.float64)
    err = np.abs(got - want)
    assert (err <= TOL + half_ulp16(want)).all(), f"{name}: max abs err {err.max():.3e}"
    assert err.max() < 1.5e-3                               # in fact well inside: the two compute the same thing


def test_noncausal_root_and_all_rows_of_a_tile(oracle_lib):
    """A noncausal root (desc.z = Tr: every row sees the whole root) and a tree whose rows end inside a tile."""
    w = wl.make_pass("noncausal", 7100, [(20, 11)], 4, 2, 256, 16, wl.F16, gate=True, scale=1.0 / 16.0)
    w.desc[:, 2] = 11
    O, _, _ = ref_forward(w)
    want, _ = oracle_lib.attention_f64(w)
    assert np.abs(wl.f16_bits_to_f32(O) - want).max() < 1.5e-3
    causal = wl.make_pass("noncausal", 7100, [(20, 11)], 4, 2, 256, 16, wl.F16, gate=True, scale=1.0 / 16.0)
    O2, _, _ = ref_forward(causal)
    assert not np.array_equal(O, O2)


@pytest.mark.parametrize("name", ["prefill_g2", "chunked_g4", "forest_g8", "verify_split_g4"])
def test_flash_restatement_reproduces_the_kernel(oracle_lib, name):
    w, split, groups = make_case(name)
    tiles, jobs, n_parts = ref.plan_tiles(w.trees, w.Hkv, split, groups)
    O, parts = ref.attention(w, tiles, n_parts, "flash")
    O2, _, parts2 = oracle_lib.flash_f32(w, tiles, 8, n_parts)
    written = np.zeros(w.n_rows, dtype=bool)
    for t in tiles:
        if t["part"] < 0:
            tr = w.trees[int(t["tree"])]
            written[int(t["r0"]):min(int(t["r0"]) + 8, int(tr["base"]) + int(tr["M"]))] = True
    if written.any():
        a, b = wl.f16_bits_to_f32(O[written]), wl.f16_bits_to_f32(O2[written])
        assert (O[written] != O2[written]).mean() < 1e-4 and (np.abs(a - b) <= 2 * half_ulp16(a)).all()   # the same bits but for isolated last-bit ties
    if n_parts:
        n = n_parts * w.Hkv * 8 * w.G * 258
        a, b = parts[:n].reshape(-1, 258), parts2[:n].reshape(-1, 258)
        live = np.isfinite(a[:, 256]) | (a[:, 257] != 0)
        a, b = a[live], b[live]
        # m and l to fp32 rounding (the emulator and the restatement add the terms of a product in different orders);
        # the unnormalised O to what one fp16 ulp of a p adds where such a rounding falls the other way
        assert np.abs(a[:, 256] - b[:, 256]).max() <= 1e-5 and np.allclose(a[:, 257], b[:, 257], rtol=1e-5)
        assert (np.abs(a[:, :256] - b[:, :256]) <= 1e-3 * a[:, 257:258]).all()


@pytest.mark.parametrize("name", ["decode_g4", "decode_g8_batch", "decode_g1_bt64", "decode_g6_unsplit", "decode_g3"])
def test_decode_restatement_follows_the_kernel(oracle_lib, name):
    w, split, groups = make_case(name)
    tiles, jobs, n_parts = ref.plan_tiles(w.trees, w.Hkv, split, groups)
    O, parts = ref.attention(w, tiles, n_parts, "decode")
    O2, _, parts2 = oracle_lib.decode_gqa_f32(w, tiles, 8, n_parts)
    a, b = wl.f16_bits_to_f32(O), wl.f16_bits_to_f32(O2)
    assert np.abs(a - b).max() <= 2.0 ** -10 * max(1.0, np.abs(a).max()) and (O != O2).mean() < 0.02
    if n_parts:
        n = n_parts * w.Hkv * 8 * w.G
        ra = parts[:n * 258].reshape(-1, 8, w.G, 258)[:, 0]
        rb = parts2[:n * 258].reshape(-1, 8, w.G, 258)[:, 0]
        assert np.abs(ra - rb).max() <= 1e-4 * np.abs(ra[..., :256]).max()
        assert np.array_equal(np.isfinite(ra[..., 256]), np.isfinite(rb[..., 256]))


def test_flash_and_decode_kernels_agree_on_single_rows(oracle_lib):
    """The reference's own cross-check (src/model/impl/bench.h:712-721): attn_decode_gqa against flash_attention."""
    w, split, groups = make_case("decode_g8_batch")
    Od, _, _ = ref_forward(w, split, groups, which="decode")
    Of, _, _ = ref_forward(w, split, groups, which="flash")
    assert np.abs(wl.f16_bits_to_f32(Od) - wl.f16_bits_to_f32(Of)).max() < 1e-3


def test_attn_prep_restatement_agrees_with_the_reference_kernel(oracle_lib):
    rng = np.random.default_rng(7200)
    rows, H, Hkv, HD, bt, n_blocks = 9, 4, 2, 256, 16, 6
    q_ld, kv_ld = H * HD, Hkv * HD
    ld = 2 * q_ld + 2 * kv_ld
    X = rng.standard_normal((rows, ld)).astype(np.float32)
    qn, kn = rng.uniform(0.5, 1.5, HD).astype(np.float32), rng.uniform(0.5, 1.5, HD).astype(np.float32)
    pos = np.zeros((rows, 4), dtype=np.int32)
    pos[:, 0], pos[:, 1], pos[:, 2] = np.arange(rows) + 3, rng.integers(0, 50, rows), rng.integers(0, 50, rows)
    inv_freq = (10000.0 ** (-np.arange(32) / 32.0)).astype(np.float32)
    sel = rng.integers(0, 3, 32).astype(np.int32)
    ktab = np.full((rows, 4), -1, dtype=np.int32)
    for r in range(rows):
        ktab[r, 0], ktab[r, 1] = r % n_blocks, r % bt
        if r % 3 == 0:
            ktab[r, 2], ktab[r, 3] = (r + 1) % n_blocks, (r + 5) % bt
    Q, Kb, Vb = (np.zeros((rows, n), dtype=np.uint16) for n in (q_ld, kv_ld, kv_ld))
    kv = np.zeros(n_blocks * 2 * bt * kv_ld, dtype=np.uint16)

    class P(C.Structure):  # AttnPrepParams of the kernel (kernels/40_attention.metal:12-21)
        _fields_ = [("H", C.c_int), ("Hkv", C.c_int), ("ld", C.c_int), ("k_off", C.c_int), ("q_ld", C.c_int), ("kv_ld", C.c_int), ("eps", C.c_float),
                    ("bt", C.c_int), ("save", C.c_int), ("pad", C.c_int), ("kv_base", C.c_ulonglong)]
    p = P(H, Hkv, ld, 2 * q_ld, q_ld, kv_ld, 1e-6, bt, 1, 0, 0)
    ref.load().ref_attn_prep(*(C.c_void_p(a.ctypes.data) for a in (X, qn, kn, pos, inv_freq, Q, Kb, Vb)), C.byref(p), C.c_void_p(sel.ctypes.data),
                             C.c_void_p(ktab.ctypes.data), C.c_void_p(kv.ctypes.data), rows)
    pp = oracle_lib.PrepParams(H, Hkv, ld, 0, 2 * HD, 2 * q_ld, 2 * q_ld + kv_ld, q_ld, kv_ld, 32, 1e-6, 1.0, bt, 0, 0)
    Q64, K64, V64 = oracle_lib.attn_prep_f64(X, qn, kn, pos, inv_freq, sel, rows, HD, pp)
    for got, want in ((Q, Q64), (Kb, K64), (Vb, V64)):
        g = wl.f16_bits_to_f32(got).astype(np.float64)
        assert (np.abs(g - want) <= 0.51 * 2 * half_ulp16(want) + 2e-6 * np.abs(want).max()).all()
    # the pool rows are the rounded K / V rows (kv_save folded in)
    pool = kv.reshape(n_blocks, 2, bt, kv_ld)
    for r in range(rows):
        for b, ps in ((ktab[r, 0], ktab[r, 1]), (ktab[r, 2], ktab[r, 3])):
            if b >= 0:
                assert np.array_equal(pool[b, 0, ps], Kb[r]) and np.array_equal(pool[b, 1, ps], Vb[r])
