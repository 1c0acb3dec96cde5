"""The CUDA path against outputs of the reference's OWN attention kernels (tests/golden/ref_kernels.npz:
flash_attention / attn_decode_gqa / attention_combine of kernels/40_attention.metal, run by the SIMT emulator
of oracle/ref_simt.h where the reference tree was present) on the same seeded inputs, through the C ABI the
way a drop-in caller drives it: a context with the reference's tile height, plan_tiles' plan, 256-dim fp16
heads with the output gate. Tolerance: 2e-3 on the fp16 outputs (both sides round P to fp16 and accumulate in
fp32; they differ in block sizes and summation order only)."""
import os

import numpy as np
import pytest

from espetero_b200 import capi, host, workloads as wl
from tests.test_ref_kernels import CASES, make_case

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz"))


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("route", ["default", "general"])
def test_cuda_path_matches_the_reference_kernels(name, route):
    w, split, groups = make_case(name)
    want = wl.f16_bits_to_f32(G[name + "_O"]).astype(np.float64)
    options = {"attn_gqa": 0, "attn_umma": 0} if route == "general" else None
    O, lse, parts, plan, kernel = host.run_pass(w, mode=capi.ESP_PLAN_REFERENCE, tile_rows=8, split=split, groups=groups, options=options)
    assert [len(plan.tiles), len(plan.jobs), plan.n_parts] == list(G[name + "_plan"])     # the reference planner's plan, bit for bit
    single = all(int(t["M"]) == 1 for t in w.trees)
    if route == "general":
        assert kernel == "flash_general"
    elif single and w.G in (1, 2, 4, 8):
        assert kernel == "decode_gqa"
    got = wl.f16_bits_to_f32(O).astype(np.float64)
    err = np.abs(got - want)
    half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 2.0 ** -14))) - 11)
    assert (err <= 2e-3 + half_ulp).all(), f"{name}/{kernel}: max abs err {err.max():.3e}"
