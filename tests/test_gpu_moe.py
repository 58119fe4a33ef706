"""GPU checks of the MoE step around the grouped GEMM (single rank) against the oracle, of the
row-movement kernels, and of the benchmark's device-side weight quantiser against the oracle's."""
import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import Dtype, Operand, SfGran, SfTensor, moe, synth
from deepgemm.api import poll_device_status, quant_mx
from helpers import bf16_round, dev, randn

pytestmark = pytest.mark.gpu


def test_block128_quantiser_matches_oracle():
    x = randn((256, 1024), 5)
    x[3, 100] = 300.0
    codes, sf = synth.block128_quant_fp8(dev(x))
    wc, ws = o.quant_fp8_block128_host(x)
    assert np.array_equal(sf.cpu().numpy().view(np.uint32), ws)
    assert np.array_equal(codes.cpu().numpy(), wc)


def test_gather_rows_sf_and_combine():
    rng = np.random.default_rng(0)
    src = torch.from_numpy(rng.integers(0, 256, (50, 256), dtype=np.uint8)).cuda()
    idx = torch.tensor([3, -1, 49, 0, 3, -1, 7], dtype=torch.int32, device="cuda")
    got = moe.gather_rows(src, idx).cpu().numpy()
    s = src.cpu().numpy()
    for i, j in enumerate(idx.tolist()):
        assert np.array_equal(got[i], s[j] if j >= 0 else np.zeros(256, np.uint8))
    words = torch.from_numpy(rng.integers(0, 2 ** 31, (3, 52), dtype=np.int32)).cuda()
    sf = SfTensor(3, 52, SfGran.G128, words)
    perm = moe.sf_permute(sf, idx).buf.cpu().numpy()
    wire = moe.sf_to_wire(sf, idx)
    back = moe.sf_from_wire(wire, torch.arange(7, dtype=torch.int32, device="cuda"), 128).buf.cpu().numpy()
    w = words.cpu().numpy()
    for i, j in enumerate(idx.tolist()):
        want = w[:, j] if j >= 0 else np.zeros(3, np.int32)
        assert np.array_equal(perm[:, i], want) and np.array_equal(back[:, i], want)
    rows = torch.from_numpy(randn((20, 64), 1)).to(torch.bfloat16).cuda()
    pos = torch.tensor([[0, 5, -1], [19, 19, 2]], dtype=torch.int32, device="cuda")
    wt = torch.tensor([[0.5, 0.25, 9.0], [1.0, -1.0, 2.0]], dtype=torch.float32, device="cuda")
    got = moe.combine(rows, pos, wt).float().cpu().numpy()
    r = rows.float().cpu().numpy()
    want = np.stack([0.5 * r[0] + 0.25 * r[5], r[19] - r[19] + 2.0 * r[2]])
    assert np.array_equal(got, bf16_round(want.astype(np.float32)))


def test_moe_forward_single_rank_matches_oracle():
    E, topk, T, K, N = 8, 2, 300, 512, 256
    w = synth.random_expert_weights(E, N, K, seed=3, device=torch.device("cuda"))
    x = randn((T, K), 9)
    x8, x_sf = quant_mx(dev(x), T, K, Dtype.Fp8, 128)
    idx, tw = synth.random_topk_routing(T, E, topk, seed=1, device=torch.device("cuda"))
    layer = moe.ExpertParallelMoE(w, E)
    out = layer.forward(x8, x_sf, idx, tw)
    poll_device_status()
    got = out.float().cpu().numpy()
    ga = o.GoldenOperand(x8.cpu().numpy(), x_sf.buf.cpu().numpy().view(np.uint32), o.FP8, 128, K)
    gb = o.GoldenOperand(w.data.cpu().numpy(), w.sf.buf.cpu().numpy().view(np.uint32), o.FP8, 128, K)
    idx_h, tw_h = idx.cpu().numpy(), tw.cpu().numpy()
    ref = np.zeros((T, N), dtype=np.float32)
    for j in range(topk):
        for e in range(E):
            rows = np.nonzero(idx_h[:, j] == e)[0]
            if rows.size:
                d = bf16_round(o.gemm_ref(ga, gb, rows=rows, n=N, b_row0=e * N))   # GEMM output is bf16
                ref[rows] += tw_h[rows, j:j + 1] * d
    assert o.calc_diff(got, ref) <= 1e-3
    assert np.abs(got - ref).max() <= 0.05 * np.sqrt((ref ** 2).mean())
    # padding blocks of the layout were skipped, real blocks carry their expert
    mi = layer.last_m_indices
    assert (mi >= -1).all() and int((mi >= 0).sum()) >= E


def test_device_plan_matches_torch_plan_contract():
    """dg_moe_plan against build_contiguous_layout: same counts, block owners and padding; the
    same set of rows in every group (the order inside a group is free)."""
    E, rows = 16, 5000
    g = torch.Generator(device="cuda").manual_seed(4)
    e = torch.randint(0, E, (rows,), device="cuda", generator=g, dtype=torch.int32)
    e[::50] = 3                                  # a heavy expert
    e[e == 7] = 8                                # an empty expert
    ref = moe.build_contiguous_layout(e, E)
    p = moe.device_plan(e, E, 128, div=1, capacity=ref.m_cap)
    torch.cuda.synchronize()
    assert torch.equal(p.counts.long(), ref.counts)
    assert torch.equal(p.block_expert, ref.m_indices)
    assert torch.equal(p.slot_src >= 0, ref.src_row >= 0)
    src, slot = p.slot_src.cpu().numpy(), p.slot_of_row.cpu().numpy()
    assert (src[slot] == np.arange(rows)).all()
    eh, be = e.cpu().numpy(), p.block_expert.cpu().numpy()
    assert (be[slot // 128] == eh).all()
    # sort-only form (align 1, div = top-k): slots are exactly the rows, ordered by expert
    q = moe.device_plan(e, E, 1, div=4, capacity=rows)
    torch.cuda.synchronize()
    order = q.slot_src.cpu().numpy()
    assert sorted(order.tolist()) == sorted((np.arange(rows) // 4).tolist())
    es = eh[np.argsort(q.slot_of_row.cpu().numpy(), kind="stable")]
    assert (np.diff(es) >= 0).all()
