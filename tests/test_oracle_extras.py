"""CPU checks of the oracle functions that have no known-answer test in the reference's suite:
quantize_output_fp8 (api.rs:1951-2011), transform_sf_batched (api.rs:1263-1311) and the spelled-out
exponential of the SwiGLU step.  The round-to-nearest quantiser is pinned to quant_mx_host, which the
reference's own tests pin; the stochastic mode and the exponential are checked through their defining
properties."""
import math

import numpy as np

import oracle as o


def rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def test_quantize_output_rne_is_quant_mx_g32_on_a_pitched_input():
    m, n, pitch = 37, 160, 200
    x = rand((m, pitch), 1) * 3.0
    x[3, :5] = [0.0, -0.0, 1e-35, 448.0, -1e30]
    data, sf = o.quantize_output_fp8(x, n)
    wd, ws = o.quant_mx_host(np.ascontiguousarray(x[:, :n]), o.FP8, 32)
    assert np.array_equal(data, wd) and np.array_equal(sf, ws)


def test_quantize_output_stochastic_picks_a_neighbour_and_is_unbiased():
    m, n = 64, 256
    x = rand((m, n), 2)
    rne, sf = o.quantize_output_fp8(x, n)
    table = o.e4m3_table()
    scale = o.dequant_mx_host(np.full((m, n), 0x38, np.uint8), sf, m, n, o.FP8, 32)      # code 0x38 = 1.0 -> the scales
    v = x / scale                                                                         # exact: powers of two
    grid = np.sort(np.unique(table[np.isfinite(table)]))
    acc = np.zeros((m, n), dtype=np.float64)
    trials = 64
    for seed in range(trials):
        st, sf2 = o.quantize_output_fp8(x, n, stochastic=True, seed=seed)
        assert np.array_equal(sf2, sf)                       # the scale does not depend on the mode
        q = table[st]
        lo = grid[np.searchsorted(grid, v, side="right") - 1]
        hi = grid[np.minimum(np.searchsorted(grid, v, side="left"), grid.size - 1)]
        assert np.all((q == lo) | (q == hi)), "a stochastic code is not one of the two neighbours"
        acc += q
    # same seed, same codes; the mean over seeds approaches the value (RNE alone is biased per element)
    again, _ = o.quantize_output_fp8(x, n, stochastic=True, seed=5)
    five, _ = o.quantize_output_fp8(x, n, stochastic=True, seed=5)
    assert np.array_equal(again, five)
    err_st = np.abs(acc / trials - v).mean()
    err_rne = np.abs(table[rne] - v).mean()
    assert err_st < 0.5 * err_rne


def test_hash_is_the_documented_mix():
    def ref(idx, seed):
        x = ((idx & 0xffffffff) * 0x9E3779B9 + (idx >> 32) * 0x7F4A7C15 + seed) & 0xffffffff
        x ^= x >> 16
        x = (x * 0x85EBCA6B) & 0xffffffff
        x ^= x >> 13
        x = (x * 0xC2B2AE35) & 0xffffffff
        x ^= x >> 16
        return x
    for idx, seed in ((0, 0), (1, 0), (12345678901, 7), (2 ** 40 + 3, 0xdeadbeef)):
        assert o.hash_u32(idx, seed) == ref(idx, seed)


def test_transform_sf_batched_is_per_batch_transform():
    batch, mn, sf_k = 3, 33, 7
    e = np.random.default_rng(3).integers(100, 140, size=(batch, mn, sf_k))
    sf = np.ldexp(1.0, e - 127).astype(np.float32)
    out = o.transform_sf_batched_host(sf, batch, mn)
    rows = (sf_k + 3) // 4
    assert out.shape == (batch * rows, 36)
    for b in range(batch):
        assert np.array_equal(out[b * rows:(b + 1) * rows], o.transform_sf_host(sf[b], mn))


def test_spelled_out_exponential_tracks_expf():
    xs = np.concatenate([np.linspace(-87, 87, 20001), rand(5000, 4) * 4]).astype(np.float32)
    worst = 0.0
    for x in xs:
        got, want = o.exp_taylor6(float(x)), math.exp(float(x))
        worst = max(worst, abs(got - want) / want)
    assert worst < 2.5e-7          # about two units in the last place of f32
    assert o.exp_taylor6(0.0) == 1.0
    assert o.exp_taylor6(-1000.0) == o.exp_taylor6(-87.0) and o.exp_taylor6(1000.0) == o.exp_taylor6(87.0)
