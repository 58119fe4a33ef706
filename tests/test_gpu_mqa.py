"""GPU parity of mqa_logits against the oracle's mqa_logits_ref (deepgemm/src/golden.rs:469-501),
through the C ABI.  Tolerance: calc_diff <= 1e-3 (the FP8 bound of the stated contract) plus an
element-wise bound; columns outside [ks, ke) must stay untouched."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import Dtype, Operand, mqa_logits, mqa_logits_f32, poll_device_status
from helpers import dev, randn, sf_tensor

pytestmark = pytest.mark.gpu
E4M3 = o.e4m3_table()


def _inputs_f32(T, S, H, D, seed):
    q8 = o.quant_e4m3_array(randn((T, H, D), seed))
    kvf = randn((S, D), seed + 1)
    scale = (np.abs(kvf).max(axis=1) / 448.0).astype(np.float32)
    kv8 = o.quant_e4m3_array(kvf / scale[:, None])
    w = randn((T, H), seed + 2)
    return q8, kv8, scale, w


def _check(got, ref, ks, ke, S, fill):
    T = got.shape[0]
    for t in range(T):
        n = max(0, min(int(ke[t]), S) - int(ks[t]))
        assert (got[t, n:] == fill).all(), f"row {t}: columns beyond the span were written"
        if n:
            want = ref[t, ks[t]:ks[t] + n]
            assert np.isfinite(got[t, :n]).all()
    gv = np.concatenate([got[t, :max(0, min(int(ke[t]), S) - int(ks[t]))] for t in range(T)])
    rv = np.concatenate([ref[t, ks[t]:min(int(ke[t]), S)] if ke[t] > ks[t] else ref[t, :0] for t in range(T)])
    assert o.calc_diff(gv, rv) <= 1e-3
    rms = np.sqrt(np.mean(rv.astype(np.float64) ** 2)) + 1e-30
    assert np.abs(gv - rv).max() / rms <= 0.05


@pytest.mark.parametrize("T,S,H,D,mode", [
    (8, 256, 64, 128, "full"), (64, 1024, 64, 128, "causal"), (37, 700, 64, 128, "ragged"),
    (16, 384, 32, 128, "ragged"), (10, 300, 128, 128, "ragged"), (12, 512, 64, 64, "causal"),
    (12, 512, 64, 32, "ragged"), (600, 2048, 64, 128, "causal"),
])
def test_mqa_logits_f32_contract(T, S, H, D, mode):
    q8, kv8, scale, w = _inputs_f32(T, S, H, D, T + S)
    rng = np.random.default_rng(T * S)
    if mode == "full":
        ks, ke = np.zeros(T, np.uint32), np.full(T, S, np.uint32)
    elif mode == "causal":                       # ke_i = S - T + i + 1, ks = 0
        ks, ke = np.zeros(T, np.uint32), (S - T + np.arange(T) + 1).astype(np.uint32)
    else:                                        # arbitrary windows, some empty, some past the end
        ks = rng.integers(0, S, T).astype(np.uint32)
        ke = (ks + rng.integers(0, S, T)).astype(np.uint32)
        ke[::5] = ks[::5]
        ke[1::7] = S + 50
    ref = o.mqa_logits_ref(E4M3[q8], E4M3[kv8] * scale[:, None], w, ks, ke)
    stride = S + 3
    fill = -777.0
    logits = torch.full((T, stride), fill, dtype=torch.float32, device="cuda")
    mqa_logits_f32(dev(q8), dev(kv8), dev(scale), dev(w), dev(ks.view(np.int32)), dev(ke.view(np.int32)),
                   T, S, H, D, logits, stride)
    poll_device_status()
    _check(logits.cpu().numpy(), ref, ks, ke, S, fill)


@pytest.mark.parametrize("T,S,H,D", [(8, 256, 64, 128), (50, 900, 64, 128), (24, 512, 32, 128), (12, 384, 64, 64)])
def test_mqa_logits_ue8m0_contract(T, S, H, D):
    """The reference SM100 flavour: UE8M0 per-32 scales on q and kv, bf16 weights and output."""
    qf, kvf = randn((T * H, D), 3), randn((S, D), 4) * 3.0
    q8, qsf = o.quant_mx_host(qf, o.FP8, 32)
    kv8, kvsf = o.quant_mx_host(kvf, o.FP8, 32)
    wb = torch.from_numpy(randn((T, H), 5)).to(torch.bfloat16)
    rng = np.random.default_rng(T)
    ks = rng.integers(0, S // 2, T).astype(np.uint32)
    ke = (ks + rng.integers(1, S, T)).astype(np.uint32)
    qd = o.dequant_mx_host(q8, qsf, T * H, D, o.FP8, 32).reshape(T, H, D)
    kvd = o.dequant_mx_host(kv8, kvsf, S, D, o.FP8, 32)
    ref = o.mqa_logits_ref(qd, kvd, wb.float().numpy(), ks, ke)
    qop = Operand.k_major(Dtype.Fp8, T * H, D, D, sf_tensor(qsf, 32), dev(q8))
    kvop = Operand.k_major(Dtype.Fp8, S, D, D, sf_tensor(kvsf, 32), dev(kv8))
    fill = -9.0
    logits = torch.full((T, S), fill, dtype=torch.bfloat16, device="cuda")
    mqa_logits(qop, kvop, wb.cuda(), dev(ks.view(np.int32)), dev(ke.view(np.int32)), T, S, H, D, logits, S)
    poll_device_status()
    got = logits.float().cpu().numpy()
    _check(got, o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(ref)), ks, ke, S, fill)


@pytest.mark.parametrize("H,D", [(16, 128), (36, 128), (100, 64), (128, 128), (256, 128), (4, 32), (96, 128)])
def test_mqa_logits_f32_head_counts(H, D):
    """Any multiple of 4 up to 256 (deepgemm/src/api.rs:1639-1650)."""
    T, S = 21, 640
    q8, kv8, scale, w = _inputs_f32(T, S, H, D, H + D)
    rng = np.random.default_rng(H)
    ks = rng.integers(0, S // 2, T).astype(np.uint32)
    ke = (ks + rng.integers(0, S, T)).astype(np.uint32)
    ref = o.mqa_logits_ref(E4M3[q8], E4M3[kv8] * scale[:, None], w, ks, ke)
    fill = -3.0
    logits = torch.full((T, S), fill, dtype=torch.float32, device="cuda")
    mqa_logits_f32(dev(q8), dev(kv8), dev(scale), dev(w), dev(ks.view(np.int32)), dev(ke.view(np.int32)), T, S, H, D, logits, S)
    poll_device_status()
    _check(logits.cpu().numpy(), ref, ks, ke, S, fill)


@pytest.mark.parametrize("T,S,H,D", [(8, 256, 64, 128), (40, 700, 64, 128), (24, 512, 32, 64), (10, 300, 96, 128)])
def test_mqa_logits_mxfp4(T, S, H, D):
    """The reference accepts packed FP4 q / kv with head_dim 64 / 128 (deepgemm/src/api.rs:1639-1650)."""
    qf, kvf = randn((T * H, D), 13), randn((S, D), 14) * 2.0
    q4, qsf = o.quant_mx_host(qf, o.FP4, 32)
    kv4, kvsf = o.quant_mx_host(kvf, o.FP4, 32)
    wb = torch.from_numpy(randn((T, H), 15)).to(torch.bfloat16)
    rng = np.random.default_rng(T + 1)
    ks = rng.integers(0, S // 2, T).astype(np.uint32)
    ke = (ks + rng.integers(1, S, T)).astype(np.uint32)
    qd = o.dequant_mx_host(q4, qsf, T * H, D, o.FP4, 32).reshape(T, H, D)
    kvd = o.dequant_mx_host(kv4, kvsf, S, D, o.FP4, 32)
    ref = o.mqa_logits_ref(qd, kvd, wb.float().numpy(), ks, ke)
    qop = Operand.k_major(Dtype.Fp4, T * H, D, D, sf_tensor(qsf, 32), dev(q4))
    kvop = Operand.k_major(Dtype.Fp4, S, D, D, sf_tensor(kvsf, 32), dev(kv4))
    fill = -9.0
    logits = torch.full((T, S), fill, dtype=torch.bfloat16, device="cuda")
    mqa_logits(qop, kvop, wb.cuda(), dev(ks.view(np.int32)), dev(ke.view(np.int32)), T, S, H, D, logits, S)
    poll_device_status()
    _check(logits.float().cpu().numpy(), o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(ref)), ks, ke, S, fill)


@pytest.mark.parametrize("kind,H,D,page_kv", [("fp8", 64, 128, 64), ("fp8", 64, 128, 4), ("fp8", 32, 64, 16), ("fp8", 64, 128, 256),
                                              ("fp8", 36, 128, 32), ("fp4", 64, 128, 64), ("fp4", 32, 64, 8), ("fp8", 64, 128, 128)])
def test_mqa_logits_paged(kind, H, D, page_kv):
    """Decode over a paged cache (deepgemm/src/api.rs:1752-1941): requests of 1..5 query tokens with growing
    context lengths, pages scattered over the cache, every request checked against the oracle on its own
    gathered kv tokens; columns at and beyond a token's context length stay untouched."""
    from deepgemm import mqa_logits_paged
    rng = np.random.default_rng(H + page_kv)
    odt, dt = (o.FP8, Dtype.Fp8) if kind == "fp8" else (o.FP4, Dtype.Fp4)
    reqs = [(1, 700), (3, 1300), (5, 260), (2, 1), (4, 2049), (1, 128), (2, 0)]        # (query tokens, context of the last token)
    T = sum(n for n, _ in reqs)
    indices, ctx = [], []
    for r, (n, c) in enumerate(reqs):
        indices += [7 * r + 3] * n
        ctx += [max(0, c - (n - 1 - i)) for i in range(n)]
    max_ctx = max(c for _, c in reqs)
    stride = -(-max_ctx // page_kv) + 2
    num_pages = sum(-(-c // page_kv) for _, c in reqs) + 5
    perm = rng.permutation(num_pages)
    table = np.zeros((T, stride), dtype=np.int32)
    table[:] = 10 ** 6          # entries nobody may follow: beyond a request's context, or rows of non-first tokens
    bytes_per = D if kind == "fp8" else D // 2
    kv_pages = np.zeros((num_pages * page_kv, bytes_per), dtype=np.uint8)
    kv_sf_pages = np.zeros(num_pages * page_kv, dtype=np.uint32)
    per_req, used, t0 = [], 0, 0
    for n, c in reqs:
        kvf = randn((max(c, 1), D), 100 + t0) * 2.0
        codes, words = o.quant_mx_host(kvf, odt, 32)
        pages = perm[used:used + -(-c // page_kv)]
        used += len(pages)
        table[t0, :len(pages)] = pages
        for i, pgid in enumerate(pages):
            lo, hi = i * page_kv, min(c, (i + 1) * page_kv)
            kv_pages[pgid * page_kv:pgid * page_kv + hi - lo] = codes[lo:hi]
            kv_sf_pages[pgid * page_kv:pgid * page_kv + hi - lo] = words[0, lo:hi]
        per_req.append((t0, n, c, o.dequant_mx_host(codes, words, max(c, 1), D, odt, 32)))
        t0 += n
    qf = randn((T * H, D), 5)
    qc, qsf = o.quant_mx_host(qf, odt, 32)
    qd = o.dequant_mx_host(qc, qsf, T * H, D, odt, 32).reshape(T, H, D)
    wb = torch.from_numpy(randn((T, H), 6)).to(torch.bfloat16)
    fill = -5.0
    width = max_ctx + 8
    logits = torch.full((T, width), fill, dtype=torch.bfloat16, device="cuda")
    qop = Operand.k_major(dt, T * H, D, D, sf_tensor(qsf, 32), dev(qc))
    mqa_logits_paged(qop, dev(kv_pages), dev(kv_sf_pages.view(np.int32)), wb.cuda(), page_kv, num_pages,
                     dev(np.array(ctx, dtype=np.int32)), dev(np.array(indices, dtype=np.int32)), dev(table), stride, T, H, D,
                     logits, width)
    poll_device_status()
    got = logits.float().cpu().numpy()
    for t0, n, c, kvd in per_req:
        ke = np.array(ctx[t0:t0 + n], dtype=np.uint32)
        ks = np.zeros(n, np.uint32)
        ref = o.mqa_logits_ref(qd[t0:t0 + n], kvd[:max(c, 1)], wb.float().numpy()[t0:t0 + n], ks, ke)
        ref = np.pad(ref, ((0, 0), (0, width - ref.shape[1])))
        if ke.max() == 0:
            assert (got[t0:t0 + n] == fill).all()
            continue
        _check(got[t0:t0 + n], o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(ref)), ks, ke, width, fill)
