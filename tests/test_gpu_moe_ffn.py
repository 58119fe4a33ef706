"""The MoE feed-forward layer beyond the reference's moe_grouped_layer (which stops after the gate/up
GEMM, deepgemm/src/api_serving.rs:371-375): SwiGLU + FP8 re-quantisation (dg_swiglu_quant) against the
oracle's swiglu_f32 + quant_mx_host, and the whole layer (two grouped GEMMs) against the oracle
composed copy by copy.  dg_swiglu_quant is held to the oracle byte for byte: both evaluate the same
operation-by-operation exponential (the platform expf differs between machines in its last bit; the
oracle's own test bounds the distance of the spelled-out exponential from expf).  The layer output is
held to the FP8 GEMM contract, calc_diff <= 1e-3."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import Dtype, Operand, SfGran, SfTensor, moe, poll_device_status, quant_mx, swiglu_quant
from helpers import dev, randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,inter,gran,pad", [(200, 512, 128, 0), (37, 256, 32, 64), (129, 384, 128, 8), (5, 128, 32, 0),
                                              (1000, 2048, 128, 0)])
def test_swiglu_quant_matches_oracle(m, inter, gran, pad):
    x = randn((m, 2 * inter + pad), m + inter) * 2.0
    x[0, :8] = [0.0, -0.0, 30.0, -30.0, 88.0, -88.0, 100.0, -100.0]
    bits = o.f32_to_bf16_bits_np(x)
    want_f32 = o.swiglu_f32(bits[:, :2 * inter], inter)
    want_data, want_sf = o.quant_mx_host(want_f32, o.FP8, gran)
    gate_up = dev(bits.view(np.int16), torch.bfloat16)
    data, sf = swiglu_quant(gate_up, m, inter, gran)
    poll_device_status()
    got_data, got_sf = data.cpu().numpy(), sf.buf.cpu().numpy().view(np.uint32)
    assert got_sf.shape == want_sf.shape
    assert np.array_equal(got_sf, want_sf), f"SF words differ at {np.argwhere(got_sf != want_sf)[:4]}"
    bad = np.argwhere(got_data != want_data)
    assert bad.size == 0, f"{len(bad)} code bytes differ, first {bad[:4]}"


def test_swiglu_quant_argument_checks():
    from deepgemm import InvalidArg
    g = torch.zeros((8, 512), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(InvalidArg):
        swiglu_quant(g, 8, 192, 128)          # width not a multiple of the granularity
    with pytest.raises(InvalidArg):
        swiglu_quant(g, 8, 512, 128)          # the rows hold 512 columns, not 2 x 512


def test_moe_ffn_layer_matches_oracle():
    E, topk, T, H, I = 4, 2, 96, 512, 256
    rng = np.random.default_rng(5)
    x = randn((T, H), 1)
    w13 = randn((E * 2 * I, H), 2) * 0.05
    w2 = randn((E * H, I), 3) * 0.05
    idx = np.stack([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.int32)
    tw = rng.random((T, topk)).astype(np.float32) + 0.1
    tw /= tw.sum(1, keepdims=True)
    xd, xsf = o.quant_mx_host(x, o.FP8, 128)
    w13d, w13sf = o.quant_mx_host(w13, o.FP8, 128)
    w2d, w2sf = o.quant_mx_host(w2, o.FP8, 128)
    gx = o.GoldenOperand(xd, xsf, o.FP8, 128, H)
    g13 = o.GoldenOperand(w13d, w13sf, o.FP8, 128, H)
    g2 = o.GoldenOperand(w2d, w2sf, o.FP8, 128, I)
    want = np.zeros((T, H), dtype=np.float32)
    for e in range(E):
        rows = np.nonzero((idx == e).any(1))[0]
        if rows.size == 0:
            continue
        up = o.f32_to_bf16_bits_np(o.gemm_ref(gx, g13, rows=rows, n=2 * I, b_row0=e * 2 * I))
        hd, hsf = o.quant_mx_host(o.swiglu_f32(up, I), o.FP8, 128)
        y = o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(o.gemm_ref(o.GoldenOperand(hd, hsf, o.FP8, 128, I), g2, m=rows.size, n=H, b_row0=e * H)))
        for i, t in enumerate(rows):
            want[t] += tw[t, list(idx[t]).index(e)] * y[i]
    sft = lambda words: SfTensor(words.shape[0], words.shape[1], SfGran.G128, dev(words.view(np.int32)))
    layer = moe.GroupedMoEFfn(Operand.k_major(Dtype.Fp8, 2 * I, H, H, sft(w13sf), dev(w13d)),
                              Operand.k_major(Dtype.Fp8, H, I, I, sft(w2sf), dev(w2d)), E)
    got = layer.forward(dev(xd), sft(xsf), dev(idx), dev(tw)).float().cpu().numpy()
    poll_device_status()
    assert np.isfinite(got).all()
    assert o.calc_diff(got, want) <= 1e-3
    rms = np.sqrt((want.astype(np.float64) ** 2).mean())
    assert np.abs(got - want).max() <= 0.05 * rms
