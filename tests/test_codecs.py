"""Storage-type codecs: the numpy encoders of the workload generator, the oracle's C++
codecs and torch's own conversions must agree bit for bit (E4M3 semantics follow
ds4_round_e4m3 / ds4_e4m3x2, kernels/80_dsv4.metal:22-33, :58-60 of the reference)."""
import numpy as np
import torch

from espetero_b200 import workloads as wl


def _samples():
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.exp2(rng.integers(-12, 10, 20000)).astype(np.float32),
        np.array([0.0, -0.0, 448.0, -448.0, 500.0, -1e9, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 2.0 ** -6, 0.0175, 464.0, 447.9, 1e-8],
                 dtype=np.float32),
        # exact ties on the e4m3 grid: between 1.0 (mantissa 0) and 1.125, etc.
        np.array([1.0625, 1.1875, 1.3125, 17.0, 19.0, 2.0 ** -9 * 1.5, 2.0 ** -9 * 2.5], dtype=np.float32),
    ])
    return x


def test_e4m3_numpy_matches_oracle(oracle_lib):
    lib = oracle_lib.load()
    x = _samples()
    codes = wl.e4m3_encode(x)
    want = np.array([lib.orc_e4m3_encode(float(v)) for v in x], dtype=np.uint8)
    # -0 and +0 differ only in the sign bit
    assert np.array_equal(codes & 0x7F, want & 0x7F)
    nz = (codes & 0x7F) != 0
    assert np.array_equal(codes[nz], want[nz])
    dec = wl.e4m3_decode(codes)
    want_dec = np.array([lib.orc_e4m3_decode(int(c)) for c in codes], dtype=np.float32)
    assert np.array_equal(dec, want_dec)
    rounded = np.array([lib.orc_round_e4m3(float(v)) for v in x], dtype=np.float32)
    assert np.array_equal(np.abs(dec), np.abs(rounded))


def test_e4m3_known_values():
    # grid facts of e4m3fn: max 448, smallest subnormal 2^-9, ties to even
    assert wl.e4m3_decode(wl.e4m3_encode(np.array([1e6], np.float32)))[0] == 448.0
    assert wl.e4m3_decode(wl.e4m3_encode(np.array([2.0 ** -10], np.float32)))[0] == 0.0          # tie -> even (0)
    assert wl.e4m3_decode(wl.e4m3_encode(np.array([3 * 2.0 ** -10], np.float32)))[0] == 2.0 ** -8  # tie -> even (2 * 2^-9)
    assert wl.e4m3_decode(wl.e4m3_encode(np.array([1.0625], np.float32)))[0] == 1.0               # tie -> even mantissa
    assert wl.e4m3_decode(wl.e4m3_encode(np.array([1.1875], np.float32)))[0] == 1.25
    allc = np.arange(256, dtype=np.uint8)
    vals = wl.e4m3_decode(allc)
    ok = ~np.isnan(vals)
    assert ok.sum() == 254
    assert np.array_equal(wl.e4m3_encode(vals[ok]) & 0x7F, allc[ok] & 0x7F)  # round trip on the grid


def test_e4m3_matches_torch():
    x = _samples()
    x = np.clip(x, -448, 448)  # torch does not saturate out-of-range inputs the same way
    t = torch.from_numpy(x).to(torch.float8_e4m3fn)
    want = t.view(torch.uint8).numpy()
    got = wl.e4m3_encode(x)
    nz = (got & 0x7F) != 0
    assert np.array_equal(got[nz], want[nz])
    assert np.array_equal(got & 0x7F, want & 0x7F)
    assert np.array_equal(wl.e4m3_decode(got), t.to(torch.float32).numpy())


def test_bf16_f16_match_torch_and_oracle(oracle_lib):
    lib = oracle_lib.load()
    x = _samples()
    bf = wl.f32_to_bf16_bits(x)
    assert np.array_equal(bf, torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    h = wl.f32_to_f16_bits(x)
    assert np.array_equal(h, torch.from_numpy(x).to(torch.float16).view(torch.int16).numpy().view(np.uint16))
    for v, b, hh in zip(x[:3000], bf[:3000], h[:3000]):
        assert lib.orc_bf16_encode(float(v)) == b
        assert lib.orc_f16_encode(float(v)) == hh
    assert np.array_equal(wl.bf16_bits_to_f32(bf[:3000]), np.array([lib.orc_bf16_decode(int(b)) for b in bf[:3000]], np.float32))
    f = np.array([lib.orc_f16_decode(int(b)) for b in h[:3000]], np.float32)
    assert np.array_equal(wl.f16_bits_to_f32(h[:3000]), f)
