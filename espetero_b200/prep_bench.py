"""Timing of esp_attn_prep alone (it is not part of bench.py's metric, which is the attention pass):

    python -m espetero_b200.prep_bench [--rows N] [--layout plain128|gated256] [--steps K]

Prints the CUDA-event time per launch and the algorithmic bandwidth: per row the kernel reads
(H + 2 Hkv) * HD floats of the fused projection and writes as many 16-bit elements."""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import capi, host, workloads as wl

LAYOUTS = {
    # name: H, Hkv, HD, rot_half, gate interleaved with the query heads
    "plain128": (64, 8, 128, 64, False),    # the causal-prefill shape of the bench (C3) with full rotary
    "gated256": (32, 8, 256, 32, True),     # kernels/40_attention.metal:23-102
}


def run(layout: str, rows: int, steps: int, device: int = 0) -> dict:
    H, Hkv, HD, rot_half, gated = LAYOUTS[layout]
    q_stride = 2 * HD if gated else HD
    k_off = H * q_stride
    v_off = k_off + Hkv * HD
    ld = v_off + Hkv * HD
    op = host.AttnOp(H, Hkv, HD, 16, wl.BF16, wl.BF16, 1.0, device=device)
    try:
        dev = op.device
        X = torch.randn(rows, ld, device=dev)
        qn, kn = torch.ones(HD, device=dev), torch.ones(HD, device=dev)
        pos = torch.randint(0, 100000, (rows, 4), dtype=torch.int32, device=dev)
        inv = torch.tensor((1e6 ** (-np.arange(rot_half) / rot_half)).astype(np.float32), device=dev)
        sel = torch.zeros(rot_half, dtype=torch.int32, device=dev)
        Q = torch.zeros(rows, H * HD, dtype=torch.int16, device=dev)
        Kb = torch.zeros(rows, Hkv * HD, dtype=torch.int16, device=dev)
        Vb = torch.zeros_like(Kb)
        pp = capi.PrepParams(H, Hkv, ld, 0, q_stride, k_off, v_off, H * HD, Hkv * HD, rot_half, 1e-6, 1.0, 16, 0, 0)
        for _ in range(3):
            op.attn_prep(X, qn, kn, pos, inv, sel, Q, Kb, Vb, pp)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            op.attn_prep(X, qn, kn, pos, inv, sel, Q, Kb, Vb, pp)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        nbytes = rows * (H + 2 * Hkv) * HD * (4 + 2)
        return {"layout": layout, "rows": rows, "us_per_launch": 1e3 * ms, "algorithmic_bytes": nbytes, "GB_per_s": nbytes / ms / 1e6}
    finally:
        op.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=0, help="0: 32768 rows for plain128, 8192 for gated256")
    ap.add_argument("--layout", default="all", choices=["all"] + sorted(LAYOUTS))
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    for layout in (sorted(LAYOUTS) if args.layout == "all" else [args.layout]):
        rows = args.rows or (32768 if layout == "plain128" else 8192)
        print(run(layout, rows, args.steps))


if __name__ == "__main__":
    main()
