"""Parity of multi-row passes (prefill, tree verify, forest masks) with the oracle, through the
C ABI. Rows with only a handful of visible keys (the first rows of a prefill) are checked with
the rigorous bound on rounding P to 16 bits added to the stated tolerance (see util.check_output)."""
import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mask", ["causal", "forest", "tree"])
@pytest.mark.parametrize("dt,kvdt,HD", [(wl.BF16, None, 128), (wl.F16, None, 256), (wl.BF16, wl.E4M3, 128)], ids=["bf16", "f16hd256", "fp8"])
def test_general_kernel_masks(oracle_lib, mask, dt, kvdt, HD):
    w = wl.make_pass("forest", 202, [(40, 20), (0, 9), (100, 16), (33, 1)], 8, 2, HD, 16, dt, kvdt, mask=mask, gate=(mask == "forest"))
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    O, lse, parts, plan, kernel = host.run_pass(w, options={"attn_umma": 0})
    assert kernel == "flash_general"
    util.check_output(O, ref, w, ref_abs=ref_abs)
    assert np.abs(lse - lse_ref).max() < 2e-3


@pytest.mark.parametrize("M", [1, 7, 8, 9, 16])
def test_row_count_edges(oracle_lib, M):
    w = wl.make_pass("rows", 300 + M, [(17, M), (0, M)], 8, 4, 128, 16, wl.BF16)
    ref, _, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    O, lse, parts, plan, kernel = host.run_pass(w, options={"attn_gqa": 0, "attn_umma": 0})
    util.check_output(O, ref, w, ref_abs=ref_abs)


def test_verify_small_split_and_combine(oracle_lib):
    """A verify pass (prefix + 16-node tree) split over the prefix: records + combine."""
    w = wl.config_c4(n_seqs=3, prefix=1024)
    ref, lse_ref = oracle_lib.attention_f64(w)
    O, lse, parts, plan, kernel = host.run_pass(w, options={"attn_umma": 0})
    assert plan.n_parts > 0
    util.check_output(O, ref, w)
    assert np.abs(lse - lse_ref).max() < 2e-3


def test_tree_mask_probe_is_exact():
    """Q = 0 and Vb = one-hot per node: the record of node n holds exactly its ancestor set."""
    P, M, H, Hkv, HD = 64, 16, 8, 2, 128
    w = wl.make_pass("treeprobe", 9, [(P, M), (0, M)], H, Hkv, HD, 16, wl.BF16, mask="tree")
    w.Q[:] = 0
    w.kv[:] = 0
    vb = np.zeros((w.n_rows, Hkv, HD), dtype=np.float32)
    for r in range(w.n_rows):
        vb[r, :, r % M] = 1.0
    w.Vb = wl.f32_to_bf16_bits(vb.reshape(w.n_rows, -1))
    O, lse, parts, plan, kernel = host.run_pass(w, force_parts=True, split=0, options={"attn_umma": 0})
    rec = parts[: plan.n_parts * Hkv * 8 * w.G * (HD + 2)].reshape(plan.n_parts, Hkv, 8, w.G, HD + 2)
    for t in plan.tiles:
        ti, r0, part = int(t["tree"]), int(t["r0"]), int(t["part"])
        par = w.extra["parents"][ti]
        base = int(w.trees[ti]["base"])
        for fm in range(min(8, base + M - r0)):
            node = r0 + fm - base
            anc, k = set(), node
            while k >= 0:
                anc.add(k)
                k = par[k]
            r = rec[part, :, fm]
            assert np.all(r[..., HD] == 0.0)
            assert np.all(r[..., HD + 1] == int(w.trees[ti]["P"]) + len(anc))
            got = r[..., :M]
            want = np.array([1.0 if n in anc else 0.0 for n in range(M)], dtype=np.float32)
            assert np.all(got == want)


def test_prefill_small(oracle_lib):
    w = wl.config_c3(n_seqs=2, rows=200)
    ref, lse_ref, ref_abs = oracle_lib.attention_f64(w, with_abs=True)
    O, lse, parts, plan, kernel = host.run_pass(w, options={"attn_umma": 0})
    util.check_output(O, ref, w, ref_abs=ref_abs)
    assert np.abs(lse - lse_ref).max() < 2e-3
