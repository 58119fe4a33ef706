"""GPU parity of the layout and batch variants of the dense GEMM, through the C ABI: MN-major operand
views (api::gemm_nn / gemm_tn / gemm_tt, deepgemm/src/api.rs:720-759), fp8_bmm over transform_sf_batched
arenas (api.rs:966-993, 1263-1311), gemm_nt_alpha (api.rs:663-673), mixed FP8 x FP4 operands (api.rs:264-265;
the reference's tolerance row "mixed 0.01", deepgemm-bench/src/main.rs:2045-2051 -- held here to the FP4
bound of 2e-3 against the oracle on identical codes), quantize_output_fp8 (api.rs:1951-2011, bytes) and a
contiguous grouped GEMM recorded into a CUDA graph."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import (Dtype, InvalidArg, Operand, Output, SfGran, SfTensor, bmm, fp8_bmm, gemm_nn, gemm_nt, gemm_nt_alpha, gemm_tn,
                      gemm_tt, m_grouped_fp8_gemm_nt_contiguous, poll_device_status, quantize_output_fp8, transform_sf_batched)
from helpers import assert_close_to_oracle, bf16_round, dev, new_output, quantised_operand, randn, sf_tensor, to_f32

pytestmark = pytest.mark.gpu


def mn_view(op, pad=0):
    """The same operand as an MN-major view: a [K, rows + pad] buffer holding the transpose (pitch kept a
    multiple of 16 bytes, as every tensor map needs)."""
    pad += (-(op.rows + pad)) % 16
    t = op.data
    if op.dtype == Dtype.Bf16:
        buf = torch.zeros((op.k, op.rows + pad), dtype=torch.bfloat16, device="cuda")
    else:
        buf = torch.zeros((op.k, op.rows + pad), dtype=torch.uint8, device="cuda")
    buf[:, :op.rows] = t.t()
    return Operand.mn_major(op.dtype, op.rows, op.k, op.rows + pad, op.sf, buf)


@pytest.mark.parametrize("layout", ["nn", "tn", "tt"])
@pytest.mark.parametrize("kind,m,n,k,pad", [("fp8", 256, 384, 1024, 0), ("fp8", 100, 200, 256, 56), ("fp8", 300, 144, 640, 16),
                                            ("bf16", 256, 320, 512, 0), ("bf16", 70, 136, 192, 8)])
def test_mn_major_views(layout, kind, m, n, k, pad):
    xa, xb = randn((m, k), m + n), randn((n, k), m + n + 1)
    if kind == "bf16":
        from helpers import bf16_operand
        a, fa = bf16_operand(xa)
        b, fb = bf16_operand(xb)
        ref = o.gemm_f32_ref(fa, fb)
    else:
        a, ga = quantised_operand(xa, "fp8", 128)
        b, gb = quantised_operand(xb, "fp8", 32)
        ref = o.gemm_ref(ga, gb, m=m, n=n)
    out = new_output(m, n)
    if layout == "nn":
        gemm_nn(a, mn_view(b, pad), out)
    elif layout == "tn":
        gemm_tn(mn_view(a, pad), b, out)
    else:
        gemm_tt(mn_view(a, pad), mn_view(b, pad), out)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), bf16_round(ref), kind, f"{kind} {layout} {m}x{n}x{k}")


def test_blas_entries_insist_on_the_view_they_need():
    a, _ = quantised_operand(randn((128, 256), 1), "fp8", 128)
    b, _ = quantised_operand(randn((128, 256), 2), "fp8", 128)
    out = new_output(128, 128)
    for fn in (gemm_nn, gemm_tn, gemm_tt):
        with pytest.raises(InvalidArg):
            fn(a, b, out)
    a4, _ = quantised_operand(randn((128, 256), 3), "fp4", 32)
    with pytest.raises(InvalidArg):
        gemm_nt(Operand.mn_major(Dtype.Fp4, 128, 256, 128, a4.sf, a4.data), a4, out)


@pytest.mark.parametrize("alpha,f32,accumulate", [(0.5, False, False), (-3.0, True, False), (2.0, True, True), (None, False, False)])
def test_gemm_nt_alpha(alpha, f32, accumulate):
    m, n, k = 200, 264, 512
    a, ga = quantised_operand(randn((m, k), 5), "fp8", 128)
    b, gb = quantised_operand(randn((n, k), 6), "fp8", 128)
    ref = o.gemm_ref(ga, gb, m=m, n=n) * (1.0 if alpha is None else alpha)
    d0 = randn((m, n), 7)
    out = new_output(m, n, f32=f32, fill=0.0)
    if accumulate:
        out.data.copy_(torch.from_numpy(d0))
        ref = ref + d0
    gemm_nt_alpha(a, b, out, accumulate, alpha)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), ref if f32 else bf16_round(ref), "fp8", f"alpha {alpha}")


@pytest.mark.parametrize("fp4_side", ["a", "b"])
@pytest.mark.parametrize("m,n,k,gran8", [(256, 384, 1024, 128), (100, 200, 512, 32), (300, 1000, 768, 128)])
def test_mixed_fp8_fp4_operands(fp4_side, m, n, k, gran8):
    xa, xb = randn((m, k), k + 1), randn((n, k), k + 2)
    a, ga = quantised_operand(xa, "fp4" if fp4_side == "a" else "fp8", 32 if fp4_side == "a" else gran8)
    b, gb = quantised_operand(xb, "fp4" if fp4_side == "b" else "fp8", 32 if fp4_side == "b" else gran8)
    out = new_output(m, n)
    gemm_nt(a, b, out)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), bf16_round(o.gemm_ref(ga, gb, m=m, n=n)), "fp4", f"mixed fp4 on {fp4_side} {m}x{n}x{k}")


@pytest.mark.parametrize("kind,batch,m,n,k,gran", [("fp8", 3, 128, 256, 512, 128), ("fp8", 4, 100, 136, 256, 32), ("fp8", 2, 300, 520, 1024, 128),
                                                    ("fp4", 2, 128, 128, 512, 32), ("bf16", 3, 130, 72, 192, 0)])
def test_bmm_over_batched_sf_arenas(kind, batch, m, n, k, gran):
    xa, xb = randn((batch, m, k), batch + m), randn((batch, n, k), batch + n)
    refs = []
    if kind == "bf16":
        ta, tb = torch.from_numpy(xa).to(torch.bfloat16), torch.from_numpy(xb).to(torch.bfloat16)
        a = Operand.k_major(Dtype.Bf16, m, k, k, None, ta.reshape(batch * m, k).cuda())
        b = Operand.k_major(Dtype.Bf16, n, k, k, None, tb.reshape(batch * n, k).cuda())
        refs = [o.gemm_f32_ref(ta[i].float().numpy(), tb[i].float().numpy()) for i in range(batch)]
    else:
        odt, dt = (o.FP8, Dtype.Fp8) if kind == "fp8" else (o.FP4, Dtype.Fp4)
        qa = [o.quant_mx_host(xa[i], odt, gran) for i in range(batch)]
        qb = [o.quant_mx_host(xb[i], odt, gran) for i in range(batch)]
        refs = [o.gemm_ref(o.GoldenOperand(qa[i][0], qa[i][1], odt, gran, k), o.GoldenOperand(qb[i][0], qb[i][1], odt, gran, k), m=m, n=n)
                for i in range(batch)]
        # scale-factor arenas through transform_sf_batched: decode the oracle's exponent bytes to f32 scales first
        def arena(q, rows):
            groups = k // gran
            words = np.stack([w for _, w in q])                                      # [batch, sf_rows, align4(rows)]
            bytes_ = np.stack([(words >> (8 * j)) & 0xff for j in range(4)], axis=2)  # [batch, sf_rows, 4, cols]
            e = bytes_.reshape(batch, -1, words.shape[2])[:, :groups, :rows]          # [batch, groups, rows]
            sf = np.ldexp(1.0, e.astype(np.int32) - 127).astype(np.float32).transpose(0, 2, 1)   # [batch, rows, groups]
            t = transform_sf_batched(dev(np.ascontiguousarray(sf)), batch, rows, gran)
            assert np.array_equal(t.buf.cpu().numpy().view(np.uint32), o.transform_sf_batched_host(sf, batch, rows))
            return t
        a = Operand.k_major(dt, m, k, k, arena(qa, m), dev(np.concatenate([c for c, _ in qa])))
        b = Operand.k_major(dt, n, k, k, arena(qb, n), dev(np.concatenate([c for c, _ in qb])))
    out = Output(Dtype.Bf16, m, n, n, torch.full((batch * m, n), float("nan"), dtype=torch.bfloat16, device="cuda"))
    (fp8_bmm if kind == "fp8" else bmm)(a, b, out, batch)
    poll_device_status()
    got = out.data.float().cpu().numpy().reshape(batch, m, n)
    for i in range(batch):
        assert_close_to_oracle(got[i], bf16_round(refs[i]), kind, f"{kind} bmm batch {i}")


def test_bmm_with_an_mn_major_operand():
    batch, m, n, k = 2, 128, 256, 512
    xa, xb = randn((batch, m, k), 1), randn((batch, n, k), 2)
    qa = [o.quant_mx_host(xa[i], o.FP8, 128) for i in range(batch)]
    qb = [o.quant_mx_host(xb[i], o.FP8, 128) for i in range(batch)]
    sfa = np.concatenate([w for _, w in qa])          # [batch * sf_rows, cols]: the arena layout
    sfb = np.concatenate([w for _, w in qb])
    a = Operand.k_major(Dtype.Fp8, m, k, k, sf_tensor(sfa, 128), dev(np.concatenate([c for c, _ in qa])))
    bt = np.concatenate([c.T for c, _ in qb])         # [batch * K, N]
    b = Operand.mn_major(Dtype.Fp8, n, k, n, sf_tensor(sfb, 128), dev(np.ascontiguousarray(bt)))
    out = Output(Dtype.Bf16, m, n, n, torch.zeros((batch * m, n), dtype=torch.bfloat16, device="cuda"))
    fp8_bmm(a, b, out, batch)
    poll_device_status()
    got = out.data.float().cpu().numpy().reshape(batch, m, n)
    for i in range(batch):
        ref = o.gemm_ref(o.GoldenOperand(*qa[i], o.FP8, 128, k), o.GoldenOperand(*qb[i], o.FP8, 128, k), m=m, n=n)
        assert_close_to_oracle(got[i], bf16_round(ref), "fp8", f"bmm nn batch {i}")


@pytest.mark.parametrize("m,n,pitch", [(128, 256, 256), (33, 96, 128), (257, 7168, 7168), (5, 32, 36)])
def test_quantize_output_fp8_bytes(m, n, pitch):
    x = randn((m, pitch), m + n) * 5.0
    x[0, :6] = [0.0, -0.0, 448.0, -500.0, 1e-35, np.nan]
    for stochastic, seed in ((False, 0), (True, 0), (True, 12345)):
        want_data, want_sf = o.quantize_output_fp8(x, n, stochastic, seed)
        data, sf = quantize_output_fp8(dev(x), m, n, pitch, stochastic, seed)
        torch.cuda.synchronize()
        assert np.array_equal(sf.cpu().numpy().view(np.uint32), want_sf)
        bad = np.argwhere(data.cpu().numpy() != want_data)
        assert bad.size == 0, f"stochastic={stochastic}: {len(bad)} code bytes differ, first {bad[:4]}"
    with pytest.raises(InvalidArg):
        quantize_output_fp8(dev(x), m, n + 8, pitch + 8)


def test_contiguous_gemm_recorded_into_a_cuda_graph():
    """A captured launch uses the static tile schedule (the counter pairs of the dynamic one are shared
    between launches); replays and eager launches in between give the same bits."""
    E, n, k = 3, 256, 512
    blocks = [0, 0, 2, -1, 1, 1, 1]
    m = 128 * len(blocks)
    a, ga = quantised_operand(randn((m, k), 1), "fp8", 128)
    w, gw = quantised_operand(randn((E * n, k), 2), "fp8", 128)
    w = Operand.k_major(Dtype.Fp8, n, k, k, w.sf, w.data)
    mi = torch.tensor(blocks, dtype=torch.int32, device="cuda")
    eager = new_output(m, n, fill=0.0)
    m_grouped_fp8_gemm_nt_contiguous(a, w, eager, mi, E)          # warm-up outside the capture, and the eager result
    torch.cuda.synchronize()
    captured = new_output(m, n, fill=0.0)
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            m_grouped_fp8_gemm_nt_contiguous(a, w, captured, mi, E)
    for _ in range(3):
        captured.data.zero_()
        g.replay()
        for _ in range(4):
            m_grouped_fp8_gemm_nt_contiguous(a, w, eager, mi, E)
        torch.cuda.synchronize()
        assert torch.equal(captured.data, eager.data)
    poll_device_status()
    got = to_f32(captured)
    for blk, e in enumerate(blocks):
        rows = np.arange(blk * 128, blk * 128 + 128)
        if e < 0:
            assert not got[rows].any()
        else:
            assert_close_to_oracle(got[rows], bf16_round(o.gemm_ref(ga, gw, rows=rows, n=n, b_row0=e * n)), "fp8", f"block {blk}")
