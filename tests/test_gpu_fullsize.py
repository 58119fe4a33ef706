"""Parity at the sizes the benchmark times.  Every configuration of the benchmark runs once at full size
with the library's own tile choice; the oracle recomputes a sample of the outputs over the full K
(128 rows x 256 columns per dense shape, rows from several experts / groups for the grouped ones, sampled
queries and kv tokens for mqa_logits) from the very codes and scale factors the kernel read.
Bounds: calc_diff <= 1e-3 (FP8) / 2e-3 (FP4) as stated in the contract, and no element further than 5 % of
the sample's RMS from the oracle (a wrong tile shows there long before it moves calc_diff).
Gate modelled on the reference's verify (deepgemm-bench/src/main.rs:2029-2202)."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import sampled
from deepgemm import (Dtype, Operand, Output, SfGran, SfTensor, get_gemm_config, gemm_nt, m_grouped_fp8_gemm_nt_contiguous,
                      m_grouped_fp8_gemm_nt_masked, moe, mqa_logits_f32, poll_device_status, quant_mx, synth)

pytestmark = pytest.mark.gpu
MAX_ERR = 0.05


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _assert(par, tol, what):
    assert par["calc_diff"] <= tol, f"{what}: calc_diff {par['calc_diff']:.3e} > {tol}"
    assert par["max_err"] <= MAX_ERR, f"{what}: element error {par['max_err']:.3e} of rms"


@pytest.mark.parametrize("m", [128, 4096])
@pytest.mark.parametrize("n,k", [(24576, 1536), (7168, 16384), (4096, 7168)])
def test_dense_fp8_benchmark_shapes(m, n, k):
    g = _gen(m + n)
    a_codes, a_sf = quant_mx(torch.randn((m, k), device="cuda", generator=g), m, k, Dtype.Fp8, 128)
    b_codes, b_words = synth.block128_quant_fp8(torch.randn((n, k), device="cuda", generator=g))
    a = Operand.k_major(Dtype.Fp8, m, k, k, a_sf, a_codes)
    b = Operand.k_major(Dtype.Fp8, n, k, k, SfTensor(k // 512, n, SfGran.G128, b_words), b_codes)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm_nt(a, b, Output(Dtype.Bf16, m, n, n, out))
    poll_device_status()
    cfg = get_gemm_config(Dtype.Fp8, 0, m, n, k)
    rows = sampled.pick(m, 128, 1, sampled.edges(m, cfg["block_m"]))
    cols = sampled.pick(n, 256, 2, sampled.edges(n, cfg["block_n"]))
    _assert(sampled.check_gemm_sample(a_codes, a_sf.buf, b_codes, b_words, out, rows, cols, o.FP8, 128, o.FP8, 128, k), 1e-3,
            f"fp8 {m}x{n}x{k} tile {cfg['block_m']}x{cfg['block_n']}")
    assert not torch.isnan(out[::97, ::89].float()).any()          # every tile was written


@pytest.mark.parametrize("m,n,k", [(8192, 8192, 8192), (4096, 7168, 7168)])
def test_dense_fp4_benchmark_shapes(m, n, k):
    g = _gen(m + k)
    a_codes, a_sf = quant_mx(torch.randn((m, k), device="cuda", generator=g), m, k, Dtype.Fp4, 32)
    b_codes, b_sf = quant_mx(torch.randn((n, k), device="cuda", generator=g), n, k, Dtype.Fp4, 32)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm_nt(Operand.k_major(Dtype.Fp4, m, k, k, a_sf, a_codes), Operand.k_major(Dtype.Fp4, n, k, k, b_sf, b_codes),
            Output(Dtype.Bf16, m, n, n, out))
    poll_device_status()
    cfg = get_gemm_config(Dtype.Fp4, 0, m, n, k)
    rows = sampled.pick(m, 128, 3, sampled.edges(m, cfg["block_m"]))
    cols = sampled.pick(n, 256, 4, sampled.edges(n, cfg["block_n"]))
    _assert(sampled.check_gemm_sample(a_codes, a_sf.buf, b_codes, b_sf.buf, out, rows, cols, o.FP4, 32, o.FP4, 32, k), 2e-3,
            f"fp4 {m}x{n}x{k}")
    assert not torch.isnan(out[::101, ::103].float()).any()


def test_grouped_contiguous_benchmark_size():
    """256 experts, top-8, 16384 tokens, K 7168, N 4096: the layout of the benchmark step (experts in order, each
    padded to 128 rows, an unused tail), rows sampled from the first, a middle and the last expert, from a
    partially filled block, and an unused block that must stay untouched."""
    E, topk, T, K, N = 256, 8, 16384, 7168, 4096
    w = synth.random_expert_weights(E, N, K, seed=1000, device="cuda")
    x8, x_sf = synth.quantised_tokens(torch.randn((T, K), device="cuda", generator=_gen(0)))
    idx, _ = synth.random_topk_routing(T, E, topk, seed=7, device="cuda")
    p = moe.device_plan(idx, E, 128, div=topk)
    a = moe.gather_rows(x8, p.slot_src)
    a_sf = moe.sf_permute(x_sf, p.slot_src)
    d = torch.full((p.capacity, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    m_grouped_fp8_gemm_nt_contiguous(Operand.k_major(Dtype.Fp8, p.capacity, K, K, a_sf, a), w, Output(Dtype.Bf16, p.capacity, N, N, d),
                                     p.block_expert, E)
    poll_device_status()
    blocks = p.block_expert.cpu().numpy()
    offsets = p.offsets.cpu().numpy()
    counts = p.counts.cpu().numpy()
    assert (blocks >= 0).sum() >= 1024 and (blocks < 0).any()
    cfg = get_gemm_config(Dtype.Fp8, 1, p.capacity, N, K, E)
    cols = sampled.pick(N, 256, 5, sampled.edges(N, cfg["block_n"]))
    for e in (0, 1, E // 2, E - 2, E - 1):
        first, cnt = int(offsets[e]), int(counts[e])
        rows = first + sampled.pick(cnt, 32, e, [0, 1, 127, 128, cnt - 1, cnt - 2])
        par = sampled.check_gemm_sample(a, a_sf.buf, w.data, w.sf.buf, d, rows, cols, o.FP8, 128, o.FP8, 128, K, b_row_offset=e * N)
        _assert(par, 1e-3, f"expert {e}")
    unused = np.nonzero(blocks < 0)[0]
    assert torch.isnan(d[int(unused[0]) * 128:int(unused[0]) * 128 + 128].float()).all(), "an unused block was written"
    assert torch.isnan(d[int(unused[-1]) * 128:].float()).all()
    used_rows = torch.as_tensor(np.nonzero(blocks >= 0)[0][::7] * 128 + 5, device="cuda")
    assert not torch.isnan(d[used_rows][:, ::61].float()).any(), "a used block was left unwritten"


def test_grouped_masked_benchmark_size():
    """32 groups, max_m 256, expected_m 128, masked_m uniform in [0, 256] (incl. 0 and 256), K 7168, N 4096."""
    G, max_m, N, K = 32, 256, 4096, 7168
    w = synth.random_expert_weights(G, N, K, seed=5, device="cuda")
    g = _gen(9)
    a_codes, a_sf = quant_mx(torch.randn((G * max_m, K), device="cuda", generator=g), G * max_m, K, Dtype.Fp8, 128)
    masked = torch.randint(0, 257, (G,), device="cuda", generator=g, dtype=torch.int32)
    masked[3], masked[4], masked[5] = 0, 256, 1
    d = torch.full((G * max_m, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    m_grouped_fp8_gemm_nt_masked(Operand.k_major(Dtype.Fp8, max_m, K, K, a_sf, a_codes), w, Output(Dtype.Bf16, max_m, N, N, d), masked, G, 128)
    poll_device_status()
    mm = masked.cpu().numpy()
    cols = sampled.pick(N, 256, 6, sampled.edges(N, get_gemm_config(Dtype.Fp8, 2, max_m, N, K, G)["block_n"]))
    for gi in (0, 4, 5, 17, G - 1):
        if mm[gi] == 0:
            continue
        rows = gi * max_m + sampled.pick(int(mm[gi]), 24, gi, [0, int(mm[gi]) - 1, 127, 128])
        _assert(sampled.check_gemm_sample(a_codes, a_sf.buf, w.data, w.sf.buf, d, rows, cols, o.FP8, 128, o.FP8, 128, K, b_row_offset=gi * N),
                1e-3, f"group {gi}")
    for gi in range(G):                                            # rows beyond masked_m stay untouched
        if mm[gi] < max_m:
            assert torch.isnan(d[gi * max_m + int(mm[gi]):(gi + 1) * max_m, ::257].float()).all(), f"group {gi} wrote beyond masked_m"


def test_mqa_logits_benchmark_size():
    """4096 queries x 64 heads x 128, 32768 kv tokens, causal ends ke = S - T + i + 1: sampled queries (first, last,
    block edges) against sampled kv tokens including each query's last valid column and the first invalid one."""
    T, S, H, D = 4096, 32768, 64, 128
    g = _gen(11)
    q = torch.randn((T, H, D), device="cuda", generator=g).to(torch.float8_e4m3fn)
    kvf = torch.randn((S, D), device="cuda", generator=g)
    scale = kvf.abs().amax(dim=1) / 448.0
    kv = (kvf / scale[:, None]).to(torch.float8_e4m3fn)
    wq = torch.randn((T, H), device="cuda", generator=g)
    ks = torch.zeros(T, dtype=torch.int32, device="cuda")
    ke = (S - T + torch.arange(T, device="cuda") + 1).to(torch.int32)
    logits = torch.full((T, S), float("nan"), dtype=torch.float32, device="cuda")
    mqa_logits_f32(q.view(torch.uint8), kv.view(torch.uint8), scale, wq, ks, ke, T, S, H, D, logits, S)
    poll_device_status()
    qs = sampled.pick(T, 64, 12, [0, 1, 2, 3, 4, T - 1, T - 2, T - 4, T - 5, 2047, 2048])
    ends = (S - T + qs + 1)
    js = sampled.pick(S, 4096, 13, [0, 127, 128, S - 1] + [int(e) - 1 for e in ends] + [int(e) for e in ends if e < S])
    qi, ji = torch.as_tensor(qs, device="cuda"), torch.as_tensor(js, device="cuda")
    kv_dec = kv[ji].float() * scale[ji][:, None]
    ref = o.mqa_logits_ref(q[qi].float().cpu().numpy(), kv_dec.cpu().numpy(), wq[qi].cpu().numpy(),
                           np.zeros(len(qs), np.uint32), np.full(len(qs), len(js), np.uint32))
    got = logits[qi][:, ji].cpu().numpy()
    valid = js[None, :] < ends[:, None]
    assert np.isnan(got[~valid]).all(), "a column outside [ks, ke) was written"
    assert np.isfinite(got[valid]).all()
    d = o.calc_diff(got[valid], ref[valid])
    assert d <= 1e-3, d
    rms = np.sqrt((ref[valid].astype(np.float64) ** 2).mean())
    assert np.abs(got[valid] - ref[valid]).max() <= MAX_ERR * rms
