"""Pins the CPU oracle (oracle/golden.c) against the known-answer tests that the
reference's own test-suite holds for this path: deepgemm/tests/golden_tests.rs,
deepgemm/tests/cpu_tests.rs:109-132 and deepgemm/tests/parity_tests.rs:55-63,503-593."""
import math

import numpy as np
import pytest

import oracle as o


class Lcg:
    """The reference tests' generator (golden_tests.rs:12-24,123-131)."""

    def __init__(self, seed):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next_u32(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return self.s >> 33

    def next_f32(self, lo, hi):
        lo, hi = np.float32(lo), np.float32(hi)
        return np.float32(lo + (np.float32(self.next_u32()) / np.float32(4294967295)) * (hi - lo))

    def next_i32_bounded(self, n):
        return 0 if n <= 0 else int(self.next_u32() % n)

    def vec(self, n, lo, hi):
        return np.array([self.next_f32(lo, hi) for _ in range(n)], dtype=np.float32)


def max_rel_err(a, b):
    a, b = a.ravel().astype(np.float32), b.ravel().astype(np.float32)
    den = np.maximum(np.maximum(np.abs(a), np.abs(b)), np.float32(1e-6))
    return float(np.max(np.abs((a - b) / den)))


# golden_tests.rs:30-43
def test_e4m3_roundtrip_covers_full_grid():
    for code in range(256):
        if code & 0x7F == 0x7F:
            assert math.isnan(o.e4m3_decode(code))
            continue
        v = o.e4m3_decode(code)
        assert math.isfinite(v)
        assert o.quant_e4m3(v) == code


# golden_tests.rs:45-63
def test_e2m1_roundtrip_and_ties():
    for code in range(16):
        assert o.quant_e2m1(o.e2m1_decode(code)) == code
    assert o.e2m1_decode(0x6) == 4.0 and o.e2m1_decode(0x7) == 6.0
    assert o.e2m1_decode(0x8) == 0.0 and math.copysign(1.0, o.e2m1_decode(0x8)) == -1.0
    assert o.e2m1_decode(0x9) == -0.5
    assert o.quant_e2m1(3.5) == 0x6
    assert o.quant_e2m1(2.5) == 0x4
    assert o.quant_e2m1(0.25) == 0x0
    assert o.quant_e2m1(100.0) == 0x7
    assert o.quant_e2m1(-100.0) == 0xF


# golden_tests.rs:65-79
def test_ue8m0_is_the_ieee_exponent_byte():
    for e in range(-40, 41):
        v = 2.0 ** e
        assert o.f32_to_ue8m0(v) == e + 127
        assert abs(o.ue8m0_decode(o.f32_to_ue8m0(v)) - v) <= abs(v) * 1e-6


# golden_tests.rs:85-120
def test_transform_sf_host_layout():
    mn, sf_k = 33, 7
    rng = Lcg(0xDEADBEEF)
    sf = np.array([2.0 ** (rng.next_i32_bounded(14) - 7) for _ in range(mn * sf_k)], dtype=np.float32)
    packed = o.transform_sf_host(sf, mn)
    assert packed.shape == (2, 36)
    for m in range(mn):
        for k in range(sf_k):
            byte = (int(packed[k // 4, m]) >> (8 * (k % 4))) & 0xFF
            assert byte == o.f32_to_ue8m0(sf[m * sf_k + k])
    assert not packed[:, mn:].any()
    # missing k bytes (k = 7 of the second word) are zero too
    assert not ((packed[1, :mn] >> 24) & 0xFF).any()


# golden_tests.rs:149-173
def test_quant_dequant_fp8_round_trip_error():
    m, k = 16, 256
    x = Lcg(12345).vec(m * k, -4.0, 4.0).reshape(m, k)
    data, sf = o.quant_mx_host(x, o.FP8, 32)
    assert data.shape == (m, k)
    back = o.dequant_mx_host(data, sf, m, k, o.FP8, 32)
    assert max_rel_err(x, back) < 0.08


# golden_tests.rs:175-215
def test_quant_dequant_fp4_round_trip_error():
    m, k = 16, 256
    x = Lcg(54321).vec(m * k, -6.0, 6.0).reshape(m, k)
    data, sf = o.quant_mx_host(x, o.FP4, 32)
    assert data.shape == (m, k // 2)
    back = o.dequant_mx_host(data, sf, m, k, o.FP4, 32)
    agg = 0.0
    for r in range(m):
        for c in range(k):
            slot = c // 32
            s = o.ue8m0_decode((int(sf[slot // 4, r]) >> (8 * (slot % 4))) & 0xFF)
            assert abs(x[r, c] - back[r, c]) <= 0.35 * max(abs(x[r, c]), s)
            agg += abs(x[r, c] - back[r, c]) / (abs(x[r, c]) + s)
    assert agg / (m * k) < 0.25


# golden_tests.rs:217-243
def test_scale_selection_kats():
    assert o.ue8m0_exp_fp4(6.0) == 127
    assert o.ue8m0_exp_fp4(7.0) == 128
    assert o.ue8m0_exp_fp4(8.0) == 128
    assert o.ue8m0_exp_fp8(448.0) == 127
    assert o.ue8m0_exp_fp8(500.0) == 128
    assert o.ue8m0_exp_fp8(512.0) == 128
    assert o.ue8m0_exp_fp8(1e-30) == 105
    assert o.ue8m0_exp_fp8(0.0) == 105
    assert o.ue8m0_exp_fp4(0.0) == 1
    assert 1 <= o.ue8m0_exp_fp4(1e-30) <= 30


# golden_tests.rs:249-298
def test_golden_gemm_matches_direct_fp32_matmul():
    m, n, k = 32, 48, 256
    rng = Lcg(999)
    xa = rng.vec(m * k, -4.0, 4.0).reshape(m, k)
    xb = rng.vec(n * k, -4.0, 4.0).reshape(n, k)
    qa, sa = o.quant_mx_host(xa, o.FP8, 32)
    qb, sb = o.quant_mx_host(xb, o.FP8, 32)
    da = o.dequant_mx_host(qa, sa, m, k, o.FP8, 32)
    db = o.dequant_mx_host(qb, sb, n, k, o.FP8, 32)
    a = o.GoldenOperand(qa, sa, o.FP8, 32, k)
    b = o.GoldenOperand(qb, sb, o.FP8, 32, k)
    got = o.gemm_ref(a, b, m=m, n=n)
    want = np.zeros((m, n), dtype=np.float32)
    for kk in range(k):  # f32 accumulation in k order, as the reference test does
        want += np.outer(da[:, kk], db[:, kk]).astype(np.float32)
    assert max_rel_err(got, want) < 1e-4
    # hoisting the decode out of the MAC loop changes no bit
    assert np.array_equal(got, o.gemm_ref_naive(a, b, m, n))


# golden_tests.rs:300-346
def test_golden_gemm_fp4_and_bf16_pack():
    m, n, k = 24, 32, 128
    rng = Lcg(0xC0FFEE)
    xa = rng.vec(m * k, -6.0, 6.0).reshape(m, k)
    xb = rng.vec(n * k, -6.0, 6.0).reshape(n, k)
    qa, sa = o.quant_mx_host(xa, o.FP4, 32)
    qb, sb = o.quant_mx_host(xb, o.FP4, 32)
    a = o.GoldenOperand(qa, sa, o.FP4, 32, k)
    b = o.GoldenOperand(qb, sb, o.FP4, 32, k)
    got = o.gemm_ref(a, b, m=m, n=n)
    assert (np.abs(got) > 1e-3).any()
    assert np.array_equal(got, o.gemm_ref_naive(a, b, m, n))
    assert o.f32_to_bf16_bits(1.0) == 0x3F80
    assert o.f32_to_bf16_bits(0.5) == 0x3F00
    assert o.f32_to_bf16_bits(1.0 + 2.0 ** -8) == 0x3F80
    assert o.f32_to_bf16_bits(1.0 + 3 * 2.0 ** -8) == 0x3F82
    assert o.f32_to_bf16_bits(1.0 + 6 * 2.0 ** -8) == 0x3F83
    xs = np.array([1.0, 0.5, 1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8, -2.71, 1e-20, -65504.0], dtype=np.float32)
    assert [int(v) for v in o.f32_to_bf16_bits_np(xs)] == [o.f32_to_bf16_bits(v) for v in xs]


# golden_tests.rs:352-401
def test_mqa_logits_ref_matches_naive():
    T, H, D, S = 8, 4, 64, 32
    rng = Lcg(31337)
    q = rng.vec(T * H * D, -1.0, 1.0).reshape(T, H, D)
    kv = rng.vec(S * D, -1.0, 1.0).reshape(S, D)
    w = rng.vec(T * H, 0.1, 0.9).reshape(T, H)
    ks = np.array([t % 4 for t in range(T)], dtype=np.uint32)
    ke = np.array([32 - t % 3 for t in range(T)], dtype=np.uint32)
    got = o.mqa_logits_ref(q, kv, w, ks, ke)
    dots = np.einsum("thd,sd->ths", q.astype(np.float64), kv.astype(np.float64))
    want = np.einsum("th,ths->ts", w.astype(np.float64), np.maximum(dots, 0.0))
    for t in range(T):
        for s in range(S):
            if ks[t] <= s < ke[t]:
                assert abs(got[t, s] - want[t, s]) <= 1e-4 * (1 + abs(want[t, s]))
            else:
                assert got[t, s] == 0.0
    # k_end beyond num_kv is clamped (golden.rs:483)
    got2 = o.mqa_logits_ref(q, kv, w, ks, ke + 100)
    assert got2.shape == (T, S)


# golden_tests.rs:403-431
def test_quantize_rne_matches_formula():
    vals = np.array([(i * 0.03125 - 8.0) * (0.001 if i % 7 == 0 else 1.0) for i in range(512)], dtype=np.float32)
    for g in range(16):
        grp = vals[g * 32:(g + 1) * 32]
        e = o.ue8m0_exp_fp8(float(np.abs(grp).max()))
        inv = np.float32(2.0 ** -(e - 127))
        for v in grp:
            dec = o.e4m3_decode(o.quant_e4m3(float(np.float32(v * inv)))) * 2.0 ** (e - 127)
            assert abs(dec - v) <= abs(v) * 0.12 + 2e-3


# cpu_tests.rs:109-132
def test_sf_packing_layout_and_bit_trick():
    assert o.sf_shape(1, 7168, 32)[0] == 56
    assert o.sf_shape(1, 7168, 128)[0] == 14
    assert o.tma_aligned(100, 4) == 100
    assert o.tma_aligned(101, 4) == 104
    exps = [130, 131, 129, 128]
    floats = np.array([np.uint32(e << 23) for e in exps], dtype=np.uint32).view(np.float32)
    packed = o.transform_sf_host(floats.reshape(1, 4), 1)
    assert int(packed[0, 0]) == exps[0] | exps[1] << 8 | exps[2] << 16 | exps[3] << 24


class XorShift:
    """parity_tests.rs:492-501"""

    def __init__(self, seed):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def vec(self, n):
        out = np.empty(n, dtype=np.float32)
        s = self.s
        M = 0xFFFFFFFFFFFFFFFF
        for i in range(n):
            s ^= (s << 13) & M
            s ^= s >> 7
            s ^= (s << 17) & M
            out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 24)) - np.float32(8.0)
        self.s = s
        return out


# parity_tests.rs:503-593 : quantise -> gemm_ref -> calc_diff against the unquantised product.
@pytest.mark.parametrize("recipe,mnk", [
    (("fp8", 128, 128), (64, 128, 512)),
    (("fp8", 32, 32), (64, 128, 512)),
    (("fp8", 128, 128), (128, 256, 1024)),
    (("fp4", 32, 32), (64, 128, 512)),
])
def test_parity_quant_tolerance_model(recipe, mnk):
    kind, ga, gb = recipe
    m, n, k = mnk
    dt = o.FP4 if kind == "fp4" else o.FP8
    x = XorShift(0x9E3779B97F4A7C15 ^ m ^ (n << 32)).vec(m * k).reshape(m, k)
    w = XorShift(0xBF58476D1CE4E5B9 ^ n ^ (k << 32)).vec(n * k).reshape(n, k)
    qa, sa = o.quant_mx_host(x, dt, ga)
    qb, sb = o.quant_mx_host(w, dt, gb)
    got = o.gemm_ref(o.GoldenOperand(qa, sa, dt, ga, k), o.GoldenOperand(qb, sb, dt, gb, k), m=m, n=n)
    ref = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    assert o.calc_diff(got, ref) < (0.02 if kind == "fp4" else 0.001)


def test_block128_generator_replicates_block_scale():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((256, 512)).astype(np.float32)
    data, sf = o.quant_fp8_block128_host(x)
    for rb in range(2):
        for g in range(4):
            blk = x[rb * 128:(rb + 1) * 128, g * 128:(g + 1) * 128]
            e = o.ue8m0_exp_fp8(float(np.abs(blk).max()))
            bytes_ = (sf[g // 4, rb * 128:(rb + 1) * 128] >> (8 * (g % 4))) & 0xFF
            assert (bytes_ == e).all()
    back = o.dequant_mx_host(data, sf, 256, 512, o.FP8, 128)
    assert max_rel_err(x, back) < 0.6  # coarse: block scale, small values flush
    assert o.calc_diff(x, back) < 1e-3
