"""Committed golden vectors (tests/golden/fixtures.npz, written by tests/golden/make_fixtures.py from
the pinned oracle).  Without a GPU: the oracle still reproduces them bit for bit.  With a GPU: the
CUDA path, called through the C ABI, reproduces the quantisation vectors bit for bit and the GEMM /
mqa_logits vectors within the contract's tolerance (calc_diff <= 1e-3 FP8, 2e-3 FP4)."""
import os

import numpy as np
import pytest

import oracle as o

FX = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixtures.npz"))
QUANT = (("fp8_g128", "fp8", 128), ("fp8_g32", "fp8", 32), ("fp4_g32", "fp4", 32))
GEMM = (("fp8_g128", "fp8", 128, (128, 256, 512)), ("fp8_g32", "fp8", 32, (128, 64, 256)), ("fp4_g32", "fp4", 32, (128, 128, 256)))


def _odt(kind):
    return o.FP4 if kind == "fp4" else o.FP8


def _bf16(bits):
    return o.bf16_bits_to_f32(bits)


# ------------------------------------------------------------------ oracle against the vectors
@pytest.mark.parametrize("name,kind,gran", QUANT)
def test_oracle_reproduces_quant_vectors(name, kind, gran):
    x = FX["quant_x"]
    data, sf = o.quant_mx_host(x, _odt(kind), gran)
    assert np.array_equal(data, FX[f"quant_{name}_data"]) and np.array_equal(sf, FX[f"quant_{name}_sf"])
    back = o.dequant_mx_host(data, sf, x.shape[0], x.shape[1], _odt(kind), gran)
    assert np.array_equal(back.view(np.uint32), FX[f"dequant_{name}"].view(np.uint32))


def test_oracle_reproduces_transform_and_gemm_vectors():
    assert np.array_equal(o.transform_sf_host(FX["transform_in"], 70), FX["transform_out"])
    for name, kind, gran, (m, n, k) in GEMM:
        ga = o.GoldenOperand(FX[f"gemm_{name}_a"], FX[f"gemm_{name}_asf"], _odt(kind), gran, k)
        gb = o.GoldenOperand(FX[f"gemm_{name}_b"], FX[f"gemm_{name}_bsf"], _odt(kind), gran, k)
        assert np.array_equal(o.f32_to_bf16_bits_np(o.gemm_ref(ga, gb, m=m, n=n)), FX[f"gemm_{name}_d_bf16"])
        assert np.array_equal(o.f32_to_bf16_bits_np(o.gemm_ref_naive(ga, gb, m, n)), FX[f"gemm_{name}_d_bf16"])
    table = o.e4m3_table()
    logits = o.mqa_logits_ref(table[FX["mqa_q"]], table[FX["mqa_kv"]] * FX["mqa_kv_scale"][:, None], FX["mqa_w"], FX["mqa_ks"],
                              FX["mqa_ke"])
    assert np.array_equal(logits.view(np.uint32), FX["mqa_logits"].view(np.uint32))


# ------------------------------------------------------------------ CUDA path against the vectors
@pytest.mark.gpu
@pytest.mark.parametrize("name,kind,gran", QUANT)
def test_gpu_quant_reproduces_vectors(name, kind, gran):
    import torch
    from deepgemm import Dtype, dequant_mx, quant_mx
    from helpers import dev
    x = FX["quant_x"]
    dt = Dtype.Fp4 if kind == "fp4" else Dtype.Fp8
    data, sf = quant_mx(dev(x), x.shape[0], x.shape[1], dt, gran)
    torch.cuda.synchronize()
    assert np.array_equal(data.cpu().numpy(), FX[f"quant_{name}_data"])
    assert np.array_equal(sf.buf.cpu().numpy().view(np.uint32), FX[f"quant_{name}_sf"])
    back = dequant_mx(data, sf, x.shape[0], x.shape[1], dt)
    assert np.array_equal(back.cpu().numpy().view(np.uint32), FX[f"dequant_{name}"].view(np.uint32))


@pytest.mark.gpu
def test_gpu_transform_sf_reproduces_vector():
    from deepgemm import transform_sf
    from helpers import dev
    got = transform_sf(dev(FX["transform_in"]), 70, 128)
    assert np.array_equal(got.buf.cpu().numpy().view(np.uint32), FX["transform_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("name,kind,gran,shape", GEMM)
def test_gpu_gemm_reproduces_vectors(name, kind, gran, shape):
    from deepgemm import Dtype, Operand, gemm_nt, poll_device_status
    from helpers import assert_close_to_oracle, dev, new_output, sf_tensor, to_f32
    m, n, k = shape
    dt = Dtype.Fp4 if kind == "fp4" else Dtype.Fp8
    a = Operand.k_major(dt, m, k, k, sf_tensor(FX[f"gemm_{name}_asf"], gran), dev(FX[f"gemm_{name}_a"]))
    b = Operand.k_major(dt, n, k, k, sf_tensor(FX[f"gemm_{name}_bsf"], gran), dev(FX[f"gemm_{name}_b"]))
    out = new_output(m, n)
    gemm_nt(a, b, out)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), _bf16(FX[f"gemm_{name}_d_bf16"]), kind, name)


@pytest.mark.gpu
def test_gpu_grouped_gemm_reproduces_vector():
    from deepgemm import Dtype, Operand, m_grouped_gemm_nt_contiguous, poll_device_status
    from helpers import assert_close_to_oracle, dev, new_output, sf_tensor, to_f32
    blocks = FX["grouped_blocks"]
    m, k, n, groups = 128 * len(blocks), 128, 128, 3
    a = Operand.k_major(Dtype.Fp8, m, k, k, sf_tensor(FX["grouped_asf"], 128), dev(FX["grouped_a"]))
    b = Operand.k_major(Dtype.Fp8, n, k, k, sf_tensor(FX["grouped_bsf"], 128), dev(FX["grouped_b"]))
    out = new_output(m, n, fill=0.0)
    m_grouped_gemm_nt_contiguous(a, b, out, dev(blocks), groups)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), _bf16(FX["grouped_d_bf16"]), "fp8", "grouped")


@pytest.mark.gpu
def test_gpu_mqa_logits_reproduces_vector():
    import torch
    from deepgemm import mqa_logits_f32, poll_device_status
    from helpers import dev
    q, kv = FX["mqa_q"], FX["mqa_kv"]
    T, H, D = q.shape
    S = kv.shape[0]
    ks, ke = FX["mqa_ks"], FX["mqa_ke"]
    logits = torch.zeros((T, S), dtype=torch.float32, device="cuda")
    mqa_logits_f32(dev(q), dev(kv), dev(FX["mqa_kv_scale"]), dev(FX["mqa_w"]), dev(ks.view(np.int32)), dev(ke.view(np.int32)),
                   T, S, H, D, logits, S)
    poll_device_status()
    got, ref = logits.cpu().numpy(), FX["mqa_logits"]
    gv = np.concatenate([got[t, :ke[t] - ks[t]] for t in range(T)])
    rv = np.concatenate([ref[t, ks[t]:ke[t]] for t in range(T)])
    assert o.calc_diff(gv, rv) <= 1e-3
    assert np.abs(gv - rv).max() <= 0.05 * (np.sqrt(np.mean(rv.astype(np.float64) ** 2)) + 1e-30)
