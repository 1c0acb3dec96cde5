"""Parity at the full sizes of the benchmark configurations, through exactly the plan the bench runs
(ESP_PLAN_B200, the bench's CTA targets, default options - so the in-kernel merges, the one-wave plans
and the inline-plan paths that only full-size passes reach are the ones checked): batched decode over
32 sequences up to 32768 keys, tree verify over 16 x 4096-key prefixes, the 131072-key E4M3 decode in
full, and the 4 x 8192-row causal prefill on a sample of rows (first and last 16 rows of every
sequence + 256 seeded rows, all heads: the full float64 result would be ~1e13 flop).
Tolerance: 2e-3 (1e-2 over the E4M3 pool) against the float64 oracle + half an ulp of the 16-bit
output; the prefill rows, which may have a handful of keys, also get the bound on rounding P to 16
bits before P.V."""
import numpy as np
import pytest
import torch

import bench
from espetero_b200 import host, workloads as wl

pytestmark = pytest.mark.gpu


def _forward(name, w):
    op = host.AttnOp.for_workload(w, bench.TILE_ROWS[name])
    try:
        plan = bench.bench_plan(name, w)
        dp = op.upload(w, plan)
        op.forward(dp)
        op.check_status()
        torch.cuda.synchronize()
        return dp.O.cpu().numpy().view(np.uint16), dp.lse.cpu().numpy(), plan, op.last_kernel
    finally:
        op.close()


@pytest.mark.parametrize("name,kernel", [("c2", "decode_gqa"), ("c4", "flash_umma"), ("c5", "decode_gqa"), ("c3", "flash_umma_duo")])
def test_bench_configuration_at_full_size_matches_oracle(oracle_lib, name, kernel):
    w = bench.build_workload(name, rank=0)
    if name == "c2":
        assert len(w.trees) == 32 and int(w.trees["P"].max()) > 30000
    O, lse, plan, ran = _forward(name, w)
    assert ran == kernel
    rep = bench.parity_report(name, w, O, lse)
    print(name, rep)
    if name == "c3":
        assert rep["rows_checked"] >= 4 * 32 + 200
    else:
        assert rep["rows_checked"] == w.n_rows
    assert rep["beyond_allowance"] == 0 and rep["ok"], rep
    if name != "c3":
        # decode and verify rows have hundreds of keys or more: no element needs the P-rounding term
        ref, _ = oracle_lib.attention_f64(w)
        got = wl.from_bits16(O, w.q_dtype).astype(np.float64)
        mant = 7
        half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -14))) - mant - 1)
        assert (np.abs(got - ref) <= rep["tol"] + half_ulp).all()
