"""Writes tests/golden/fixtures.npz: small inputs together with the outputs of the CPU oracle
(oracle/golden.c, the C restatement of deepgemm/src/golden.rs:56-510 that tests/test_oracle_kat.py
pins against the reference's known-answer tests).  The reference itself is Rust and cannot run
where these tests run, so the vectors come from the pinned oracle; they freeze its behaviour, so
that a later change of the oracle or of a kernel shows up against bytes that are under version
control.  Run from the repository root:  python tests/golden/make_fixtures.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as o  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures.npz")


def randn(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def main():
    f = {}
    # quant_mx: ragged m, edge values (zeros, signed zero, saturation, tiny blocks, NaN of both signs)
    x = randn((37, 512), 11)
    x[0, :8] = [0.0, -0.0, 448.0, -448.0, 1e30, -1e30, np.nan, -np.nan]
    x[1, :] = 0.0
    x[2, :256] *= 1e-20
    x[3, :4] = [6.0, -6.0, 2.5, 3.5]
    f["quant_x"] = x
    for name, dt, gran in (("fp8_g128", o.FP8, 128), ("fp8_g32", o.FP8, 32), ("fp4_g32", o.FP4, 32)):
        data, sf = o.quant_mx_host(x, dt, gran)
        f[f"quant_{name}_data"], f[f"quant_{name}_sf"] = data, sf
        f[f"dequant_{name}"] = o.dequant_mx_host(data, sf, x.shape[0], x.shape[1], dt, gran)
    # transform_sf: power-of-two scales [mn, sf_k] -> packed words
    sf_in = np.exp2(np.random.default_rng(12).integers(-20, 20, size=(70, 7))).astype(np.float32)
    f["transform_in"] = sf_in
    f["transform_out"] = o.transform_sf_host(sf_in, 70)
    # dense GEMMs on the reference's own CPU-runnable shape (M 128, N 256, K 512)
    # (FP8 with one scale per 128; smaller FP8 G32 and FP4 cases)
    for name, dt, gran, (m, n, k) in (("fp8_g128", o.FP8, 128, (128, 256, 512)), ("fp8_g32", o.FP8, 32, (128, 64, 256)),
                                      ("fp4_g32", o.FP4, 32, (128, 128, 256))):
        a, b = randn((m, k), 13), randn((n, k), 14)
        ad, asf = o.quant_mx_host(a, dt, gran)
        bd, bsf = o.quant_mx_host(b, dt, gran)
        ga, gb = o.GoldenOperand(ad, asf, dt, gran, k), o.GoldenOperand(bd, bsf, dt, gran, k)
        f[f"gemm_{name}_a"], f[f"gemm_{name}_asf"], f[f"gemm_{name}_b"], f[f"gemm_{name}_bsf"] = ad, asf, bd, bsf
        f[f"gemm_{name}_d_bf16"] = o.f32_to_bf16_bits_np(o.gemm_ref(ga, gb, m=m, n=n))
    # grouped contiguous: 3 experts of N 128, blocks [1, -1, 0, 2, 0]
    blocks = np.array([1, -1, 0, 2, 0], dtype=np.int32)
    ga_x, gb_x = randn((128 * len(blocks), 128), 15), randn((3 * 128, 128), 16)
    ad, asf = o.quant_mx_host(ga_x, o.FP8, 128)
    bd, bsf = o.quant_fp8_block128_host(gb_x)
    ga, gb = o.GoldenOperand(ad, asf, o.FP8, 128, 128), o.GoldenOperand(bd, bsf, o.FP8, 128, 128)
    d = np.zeros((ga_x.shape[0], 128), dtype=np.uint16)
    for i, e in enumerate(blocks):
        if e >= 0:
            rows = np.arange(128 * i, 128 * (i + 1))
            d[rows] = o.f32_to_bf16_bits_np(o.gemm_ref(ga, gb, rows=rows, n=128, b_row0=int(e) * 128))
    f.update(grouped_blocks=blocks, grouped_a=ad, grouped_asf=asf, grouped_b=bd, grouped_bsf=bsf, grouped_d_bf16=d)
    # mqa_logits (fp32 contract): 8 queries, 32 heads, D 128, 256 kv tokens, causal windows
    q = o.quant_e4m3_array(randn((8, 32, 128), 17))
    kv = o.quant_e4m3_array(randn((256, 128), 18))
    kv_scale = np.exp2(np.random.default_rng(19).integers(-3, 3, size=256)).astype(np.float32)
    w = randn((8, 32), 20)
    ks = np.zeros(8, dtype=np.uint32)
    ke = (256 - 8 + np.arange(8) + 1).astype(np.uint32)
    table = o.e4m3_table()
    logits = o.mqa_logits_ref(table[q], table[kv] * kv_scale[:, None], w, ks, ke)
    f.update(mqa_q=q, mqa_kv=kv, mqa_kv_scale=kv_scale, mqa_w=w, mqa_ks=ks, mqa_ke=ke, mqa_logits=logits)
    np.savez_compressed(OUT, **f)
    print(OUT, os.path.getsize(OUT), "bytes,", len(f), "arrays")


if __name__ == "__main__":
    main()
