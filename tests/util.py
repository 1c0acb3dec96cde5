"""Helpers shared by the tests: tolerances and comparisons against the oracle."""
import numpy as np

from espetero_b200 import workloads as wl

# Stated tolerances (max abs error against the float64 oracle).
TOL_16 = 2e-3      # fp16 / bf16 pools
TOL_FP8 = 1e-2     # E4M3 pools


def tol_for(w) -> float:
    return TOL_FP8 if w.kv_dtype == wl.E4M3 else TOL_16


def out_ulp_half(ref: np.ndarray, dtype: int) -> np.ndarray:
    """Half a unit in the last place of the output type at |ref|: what rounding the final
    value to fp16 / bf16 alone may add on top of the arithmetic error."""
    mant = 10 if dtype == wl.F16 else 7
    e = np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -14)))
    return np.exp2(e - mant - 1)


def p_rounding_unit(w) -> float:
    """Relative half-ulp of the 16-bit type P is rounded to before P.V (the reference rounds P
    to its 16-bit type too, kernels/40_attention.metal:297): 2^-12 for fp16, 2^-9 for bf16;
    E4M3 pools run their MMAs in fp16."""
    return 2.0 ** -12 if (w.q_dtype == wl.F16 or w.kv_dtype == wl.E4M3) else 2.0 ** -9


def check_output(O_bits: np.ndarray, ref64: np.ndarray, w, rows=None, tol=None, what="O", ref_abs=None):
    """max |O - oracle| <= tol + half an output ulp [+ u_P * sum_j p_j |v_j| when ref_abs is given].

    tol is the stated arithmetic tolerance (2e-3; 1e-2 with an E4M3 pool). The output-ulp term is
    what storing the result in fp16 / bf16 adds. ref_abs (the oracle's sum_j softmax_j |v_j|) adds
    the rigorous bound on rounding P to 16 bits, which matters only for rows with a handful of
    visible keys (first rows of a prefill); decode / verify cases are checked without it."""
    tol = tol_for(w) if tol is None else tol
    got = wl.from_bits16(O_bits if rows is None else O_bits[rows], w.q_dtype).astype(np.float64)
    err = np.abs(got - ref64)
    allow = tol + out_ulp_half(ref64, w.q_dtype)
    if ref_abs is not None:
        allow = allow + p_rounding_unit(w) * ref_abs
    bad = err > allow
    assert not bad.any(), f"{what}: max abs err {err.max():.3e} (tol {tol:g} + rounding), {bad.sum()} elements off, first at {np.argwhere(bad)[0]}"
    return float(err.max())


def records_to_output(parts: np.ndarray, w, plan_tiles, jobs, tile_rows: int):
    """Merge fp32 records on the host in float64 (for strict checks of the unrounded result).
    Returns (O [rows, H*HD] float64, lse [rows, H]); rows not covered by a job are NaN."""
    HD, G, Hkv = w.HD, w.G, w.Hkv
    rec = parts[: (parts.size // (HD + 2)) * (HD + 2)].reshape(-1, HD + 2).astype(np.float64)
    O = np.full((w.n_rows, w.H * HD), np.nan)
    lse = np.full((w.n_rows, w.H), np.nan)
    for job in jobs:
        for r in range(int(job["rows"])):
            for h in range(w.H):
                kvh, hg = h // G, h % G
                idx = [((int(job["part0"]) + s) * Hkv + kvh) * tile_rows * G + r * G + hg for s in range(int(job["nparts"]))]
                m = rec[idx, HD]
                l = rec[idx, HD + 1]
                M = m.max()
                if not np.isfinite(M):
                    O[int(job["r0"]) + r, h * HD:(h + 1) * HD] = 0
                    lse[int(job["r0"]) + r, h] = -np.inf
                    continue
                wgt = np.where(np.isfinite(m), np.exp(m - M), 0.0)
                L = (wgt * l).sum()
                acc = (wgt[:, None] * rec[idx, :HD]).sum(axis=0)
                O[int(job["r0"]) + r, h * HD:(h + 1) * HD] = acc / L
                lse[int(job["r0"]) + r, h] = M + np.log(L)
    return O, lse
