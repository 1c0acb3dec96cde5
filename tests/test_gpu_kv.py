"""kv_save and kv_copy_blocks on the GPU: bit-exact against the oracle's restatement
(kernels/40_attention.metal:875-905), then attention over the saved rows."""
import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kvdt", [None, wl.E4M3], ids=["bf16", "fp8"])
def test_kv_save_matches_oracle(oracle_lib, kvdt):
    rows = 70
    w = wl.make_pass("save", 505, [(0, rows)], 8, 2, 128, 16, wl.BF16, kvdt, spare_blocks=8)
    entries = np.zeros(rows, dtype=wl.KVSAVE_DT)
    order = np.random.default_rng(1).permutation(8)
    for i in range(rows):
        entries[i] = (i, int(order[i // 16]), i % 16, 0)
    want = w.kv.copy()
    oracle_lib.kv_save(w, want, entries)
    op = host.AttnOp.for_workload(w)
    try:
        dp = op.upload(w)
        keep = op.kv_save(dp, entries)
        torch.cuda.synchronize()
        got = dp.kv.cpu().numpy().view(w.kv.dtype)
        if kvdt is None:
            assert np.array_equal(got, want)
        else:
            assert np.array_equal(got & 0x7F, want & 0x7F)       # +-0 may differ in sign only
            nz = (want & 0x7F) != 0
            assert np.array_equal(got[nz], want[nz])
    finally:
        op.close()


def test_kv_copy_blocks_matches_oracle(oracle_lib):
    w = wl.make_pass("cow", 506, [(64, 1)], 8, 2, 128, 16, wl.BF16, spare_blocks=12)
    n_layers = 2
    region = w.kv.size // n_layers // (2 * 16 * w.kv_ld) * (2 * 16 * w.kv_ld)
    pairs = np.array([[0, 5], [3, 1], [2, 6]], dtype=np.int32)
    want = w.kv.copy()
    oracle_lib.kv_copy_blocks(w, want, pairs, region, n_layers)
    op = host.AttnOp.for_workload(w)
    try:
        dp = op.upload(w)
        keep = op.kv_copy_blocks(dp, pairs, region, n_layers)
        torch.cuda.synchronize()
        assert np.array_equal(dp.kv.cpu().numpy().view(np.uint16), want)
    finally:
        op.close()


def test_prefill_then_decode_reads_saved_rows(oracle_lib):
    """kv_save a prefill's rows into fresh pages, then decode against them: equals attention over
    the same rows as batch keys."""
    rows = 48
    w = wl.make_pass("chain", 507, [(0, rows)], 8, 2, 128, 16, wl.BF16, spare_blocks=4)
    blocks = np.array([2, 0, 3], dtype=np.int32)
    entries = np.zeros(rows, dtype=wl.KVSAVE_DT)
    for i in range(rows):
        entries[i] = (i, int(blocks[i // 16]), i % 16, 0)
    op = host.AttnOp.for_workload(w)
    try:
        dp = op.upload(w)
        op.kv_save(dp, entries)
        torch.cuda.synchronize()
        kv_after = dp.kv.cpu().numpy().view(np.uint16)
    finally:
        op.close()
    # decode row = the last prefill row, cached keys = rows 0..rows-2
    w2 = wl.make_pass("chain2", 508, [(rows - 1, 1)], 8, 2, 128, 16, wl.BF16, spare_blocks=2)
    w2.kv, w2.n_blocks = kv_after, w.n_blocks
    w2.blocks = blocks
    w2.Q, w2.Kb, w2.Vb = w.Q[rows - 1:rows].copy(), w.Kb[rows - 1:rows].copy(), w.Vb[rows - 1:rows].copy()
    O, lse, _, _, kernel = host.run_pass(w2)
    assert kernel == "decode_gqa"
    ref, _ = oracle_lib.attention_f64(w, rows=[rows - 1])
    util.check_output(O, ref, w2)
