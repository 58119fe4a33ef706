"""GPU parity of the dense and grouped GEMMs against the oracle's gemm_ref, through the C ABI.
Tolerance: calc_diff = 1 - 2*sum(xy)/sum(x^2+y^2) <= 1e-3 (FP8) / 2e-3 (FP4), the stated
contract, on identical oracle-quantised inputs (helpers.TOL), plus an element-wise bound."""
import os

import numpy as np
import pytest
import torch

import oracle as o
from deepgemm import (Dtype, Operand, Output, m_grouped_gemm_nt_contiguous_gather, m_grouped_gemm_nt_contiguous_scatter, bf16_gemm_nt, fp4_gemm_nt, fp8_gemm_nt, gemm_nt, get_gemm_config,
                      m_grouped_fp8_gemm_nt_contiguous, m_grouped_fp8_gemm_nt_masked, m_grouped_gemm_nt_contiguous,
                      m_grouped_gemm_nt_masked, poll_device_status, SfGran, SfTensor)
from helpers import (assert_close_to_oracle, bf16_operand, bf16_round, dev, new_output, quantised_operand, randn,
                     to_f32)

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_env():
    yield
    for v in ("DG_BLOCK_N", "DG_NUM_STAGES", "DG_BAND", "DG_CLUSTER", "DG_SPLIT_K"):
        os.environ.pop(v, None)


def run_dense(kind, m, n, k, gran_a=32, gran_b=32, block128_b=False, f32=False, seed=0, block_n=None, stages=None,
              cluster=None):
    if cluster:
        os.environ["DG_CLUSTER"] = str(cluster)
    if block_n:
        os.environ["DG_BLOCK_N"] = str(block_n)
    if stages:
        os.environ["DG_NUM_STAGES"] = str(stages)
    xa, xb = randn((m, k), seed), randn((n, k), seed + 1)
    if kind == "bf16":
        a, fa = bf16_operand(xa)
        b, fb = bf16_operand(xb)
        ref = o.gemm_f32_ref(fa, fb)
        fn = bf16_gemm_nt
    else:
        a, ga = quantised_operand(xa, kind, gran_a)
        b, gb = quantised_operand(xb, kind, gran_b, block128=block128_b)
        ref = o.gemm_ref(ga, gb, m=m, n=n)
        fn = fp8_gemm_nt if kind == "fp8" else fp4_gemm_nt
    out = new_output(m, n, f32=f32)
    fn(a, b, out)
    poll_device_status()
    got = to_f32(out)
    assert_close_to_oracle(got, ref if f32 else bf16_round(ref), kind, f"{kind} {m}x{n}x{k}")
    return got, ref


# ---- the reference's own CPU-runnable configuration: FP8 M128 N256 K512, 1x128 / 128x128 scales
def test_fp8_config_golden_case():
    run_dense("fp8", 128, 256, 512, gran_a=128, gran_b=128, block128_b=True, seed=0)


@pytest.mark.parametrize("kind", ["bf16", "fp8", "fp4"])
def test_single_tile(kind):
    run_dense(kind, 128, 128, 512, seed=3, block_n=128)


@pytest.mark.parametrize("gran_a,gran_b", [(32, 32), (128, 128), (128, 32), (32, 128)])
def test_fp8_granularities(gran_a, gran_b):
    run_dense("fp8", 256, 384, 1536, gran_a=gran_a, gran_b=gran_b, seed=5)


@pytest.mark.parametrize("block_n", [32, 64, 96, 128, 160, 192, 224])
def test_fp8_every_block_n(block_n):
    run_dense("fp8", 256, 512, 1024, gran_a=128, gran_b=128, seed=block_n, block_n=block_n)


@pytest.mark.parametrize("kind,cluster,block_n,n", [
    ("fp8", 1, 48, 520), ("fp8", 1, 176, 1000), ("fp8", 1, 208, 1040), ("fp8", 2, 208, 1344), ("fp8", 2, 80, 400),
    ("fp4", 1, 208, 624), ("bf16", 1, 144, 440), ("bf16", 2, 240, 720),
])
def test_tile_widths_that_are_multiples_of_16(kind, cluster, block_n, n):
    """Tile widths need not be multiples of 32: the last 32-column chunk of a tile is then half used and the
    epilogue must stop at the tile's end, not at the chunk's (the columns behind it belong to the next tile)."""
    run_dense(kind, 300, n, 1024, gran_a=128 if kind == "fp8" else 32, gran_b=128 if kind == "fp8" else 32, seed=block_n,
              block_n=block_n, cluster=cluster)


def test_tile_width_208_with_f32_output():
    run_dense("fp8", 260, 1040, 512, gran_a=128, gran_b=128, seed=9, block_n=208, f32=True)


@pytest.mark.parametrize("block_n", [32, 128, 224])
def test_fp4_block_n(block_n):
    run_dense("fp4", 256, 512, 1024, seed=block_n, block_n=block_n)


@pytest.mark.parametrize("block_n", [64, 256])
def test_bf16_block_n(block_n):
    run_dense("bf16", 256, 512, 512, seed=block_n, block_n=block_n)


@pytest.mark.parametrize("kind,m,n,k", [
    ("fp8", 100, 200, 256),     # ragged M and N (N % 8 == 0)
    ("fp8", 1, 8, 128),         # smallest
    ("fp8", 300, 1000, 640),
    ("fp8", 129, 260, 128),     # N % 8 != 0: scalar store path
    ("fp4", 100, 200, 512),
    ("bf16", 70, 136, 192),
])
def test_ragged_shapes(kind, m, n, k):
    run_dense(kind, m, n, k, seed=m + n)


@pytest.mark.parametrize("cluster", [1, 2])
@pytest.mark.parametrize("kind,m,n,k", [
    ("fp8", 512, 896, 1024), ("fp8", 100, 200, 256), ("fp8", 300, 1000, 640), ("fp8", 1, 8, 128),
    ("fp4", 384, 448, 1024), ("bf16", 384, 512, 512), ("bf16", 130, 72, 192),
])
def test_single_cta_and_cta_pair_tiles(cluster, kind, m, n, k):
    """Both tilings on the same shapes: one CTA per 128-row tile, and a CTA pair per 256-row tile
    (including shapes where the second CTA of the last pair has no valid row)."""
    run_dense(kind, m, n, k, gran_a=128 if kind == "fp8" else 32, gran_b=32, seed=m + cluster, cluster=cluster)


@pytest.mark.parametrize("cluster,block_n", [(2, 32), (2, 96), (2, 224), (1, 224)])
def test_cta_pair_block_n(cluster, block_n):
    run_dense("fp8", 512, 1344, 2048, gran_a=128, gran_b=128, seed=block_n, block_n=block_n, cluster=cluster)


@pytest.mark.parametrize("stages", [2, 3])
def test_pipeline_wraps_with_few_stages(stages):
    run_dense("fp8", 384, 640, 4096, gran_a=128, gran_b=128, seed=11, stages=stages)


def test_many_tiles_per_cta_and_long_k():
    """More tiles than CTAs (persistent loop, both accumulator stages) and a deep K loop."""
    run_dense("fp8", 2048, 4096, 2048, gran_a=128, gran_b=128, block128_b=True, seed=21)
    run_dense("fp8", 128, 256, 16384, gran_a=128, gran_b=128, seed=22)


@pytest.mark.parametrize("kind,m,n,k,splits", [
    ("fp8", 128, 512, 4096, 0), ("fp8", 128, 512, 4096, 4), ("fp8", 77, 200, 8192, 8), ("fp8", 128, 260, 2048, 2),
    ("fp4", 100, 384, 8192, 4), ("bf16", 128, 256, 2048, 4),
])
def test_split_k_for_single_row_block(kind, m, n, k, splits):
    """Weight-streaming shapes (one row block, long K) run split over K ranges with a fixed-order
    reduction; splits = 0 lets the library choose."""
    if splits:
        os.environ["DG_SPLIT_K"] = str(splits)
    run_dense(kind, m, n, k, gran_a=128 if kind == "fp8" else 32, gran_b=128 if kind == "fp8" else 32, seed=k + splits)


def test_split_k_accumulate_f32_and_determinism():
    os.environ["DG_SPLIT_K"] = "4"
    m, n, k = 128, 384, 4096
    a, ga = quantised_operand(randn((m, k), 1), "fp8", 128)
    b, gb = quantised_operand(randn((n, k), 2), "fp8", 128)
    o1, o2 = new_output(m, n), new_output(m, n)
    fp8_gemm_nt(a, b, o1)
    fp8_gemm_nt(a, b, o2)
    assert torch.equal(o1.data, o2.data)
    of = new_output(m, n, f32=True, fill=2.0)
    pf = new_output(m, n, f32=True)
    gemm_nt(a, b, pf)
    gemm_nt(a, b, of, accumulate=True)
    poll_device_status()
    assert np.array_equal(to_f32(of), to_f32(pf) + np.float32(2.0))
    assert_close_to_oracle(to_f32(pf), o.gemm_ref(ga, gb, m=m, n=n), "fp8", "split-K f32")
    os.environ["DG_SPLIT_K"] = "0"      # switched off: same contract
    p1 = new_output(m, n, f32=True)
    gemm_nt(a, b, p1)
    assert_close_to_oracle(to_f32(p1), o.gemm_ref(ga, gb, m=m, n=n), "fp8", "no split")


def test_f32_output_and_strided_output():
    got, ref = run_dense("fp8", 256, 256, 512, f32=True, seed=31)
    xa, xb = randn((200, 256), 32), randn((96, 256), 33)
    a, ga = quantised_operand(xa, "fp8", 32)
    b, gb = quantised_operand(xb, "fp8", 32)
    out = new_output(200, 96, stride=136, fill=7.0)
    gemm_nt(a, b, out)
    poll_device_status()
    assert_close_to_oracle(to_f32(out), bf16_round(o.gemm_ref(ga, gb, m=200, n=96)), "fp8", "strided D")
    assert bool((out.data[:, 96:] == 7.0).all()), "columns beyond N were touched"


def test_accumulate_adds_the_rounded_tile():
    """D0 + bf16(acc), rounded to bf16 (the oracle has no accumulate model; the reference adds
    the cast tile in D's dtype, deepgemm/kernels/gemm_sm100.cu:309-315)."""
    m, n, k = 256, 256, 512
    xa, xb = randn((m, k), 41), randn((n, k), 42)
    a, ga = quantised_operand(xa, "fp8", 128)
    b, gb = quantised_operand(xb, "fp8", 128)
    d0 = bf16_round(randn((m, n), 43) * 10)
    out = new_output(m, n)
    out.data.copy_(torch.from_numpy(d0))
    plain = new_output(m, n)
    gemm_nt(a, b, plain)
    gemm_nt(a, b, out, accumulate=True)
    poll_device_status()
    want = bf16_round(d0 + to_f32(plain))
    assert np.array_equal(to_f32(out), want)
    outf = new_output(m, n, f32=True, fill=1.5)
    plainf = new_output(m, n, f32=True)
    gemm_nt(a, b, plainf)
    gemm_nt(a, b, outf, accumulate=True)
    assert np.array_equal(to_f32(outf), to_f32(plainf) + np.float32(1.5))


def test_bitwise_determinism():
    xa, xb = randn((512, 1024), 51), randn((768, 1024), 52)
    a, _ = quantised_operand(xa, "fp8", 128)
    b, _ = quantised_operand(xb, "fp8", 128)
    o1, o2 = new_output(512, 768), new_output(512, 768)
    fp8_gemm_nt(a, b, o1)
    fp8_gemm_nt(a, b, o2)
    poll_device_status()
    assert torch.equal(o1.data, o2.data)


# ---- grouped --------------------------------------------------------------------------------
def _stacked_b(kind, groups, n, k, seed, gran=32):
    xb = randn((groups * n, k), seed)
    if kind == "bf16":
        op, f = bf16_operand(xb)
        op.rows = n
        return op, f
    op, g = quantised_operand(xb, kind, gran)
    op.rows = n
    return op, g


@pytest.mark.parametrize("cluster", [1, 2])
@pytest.mark.parametrize("kind", ["fp8", "fp4", "bf16"])
def test_m_grouped_contiguous(kind, cluster):
    os.environ["DG_CLUSTER"] = str(cluster)
    groups, n, k = 4, 256, 512
    # expert of each 128-row block, -1 = padding: pairs, odd runs, a run of 3, a trailing single
    blocks = [0, 0, 2, -1, 3, 1, 1, -1, 2, 2, 2, 0, 3, 3, 3, 3, 1]
    m = 128 * len(blocks)
    xa = randn((m, k), 61)
    xa[128 * 5 + 70: 128 * 6] = 0.0                   # zero padding rows inside a block
    b, gb = _stacked_b(kind, groups, n, k, 62)
    if kind == "bf16":
        a, fa = bf16_operand(xa)
    else:
        a, ga = quantised_operand(xa, kind, 32)
    out = new_output(m, n, fill=3.0)
    m_indices = dev(np.array(blocks, dtype=np.int32))
    m_grouped_gemm_nt_contiguous(a, b, out, m_indices, groups)
    poll_device_status()
    got = to_f32(out)
    for i, e in enumerate(blocks):
        rows = np.arange(128 * i, 128 * (i + 1))
        if e < 0:
            assert (got[rows] == 3.0).all(), "a padding block was written"
            continue
        if kind == "bf16":
            ref = o.gemm_f32_ref(fa[rows], gb[e * n:(e + 1) * n])
        else:
            ref = o.gemm_ref(ga, gb, rows=rows, n=n, b_row0=e * n)
        assert_close_to_oracle(got[rows], bf16_round(ref), kind, f"block {i} expert {e}")


def test_m_grouped_contiguous_many_blocks_random_runs():
    """A long random m_indices (runs of 1..5 blocks, padding blocks in between) on CTA pairs:
    exercises the in-kernel tile list over several 32-block chunks."""
    rng = np.random.default_rng(5)
    groups, n, k = 8, 128, 256
    blocks = []
    while len(blocks) < 90:
        blocks += [int(rng.integers(0, groups))] * int(rng.integers(1, 6))
        if rng.random() < 0.3:
            blocks.append(-1)
    m = 128 * len(blocks)
    a, ga = quantised_operand(randn((m, k), 1), "fp8", 128)
    b, gb = _stacked_b("fp8", groups, n, k, 2, gran=128)
    out = new_output(m, n, fill=3.0)
    m_grouped_gemm_nt_contiguous(a, b, out, dev(np.array(blocks, dtype=np.int32)), groups)
    poll_device_status()
    got = to_f32(out)
    for i, e in enumerate(blocks):
        rows = np.arange(128 * i, 128 * (i + 1))
        if e < 0:
            assert (got[rows] == 3.0).all()
        else:
            assert_close_to_oracle(got[rows], bf16_round(o.gemm_ref(ga, gb, rows=rows, n=n, b_row0=e * n)), "fp8", f"block {i}")


@pytest.mark.parametrize("groups,n,k,tokens,blocks", [
    (3, 384, 512, 200, [2, 0, 0, -1, 1]),
    (4, 416, 1024, 77, [3, 3, 1, 0, 2, 2]),          # 416 = two 208-wide tiles; sources repeat (fewer tokens than rows)
    (2, 4096, 7168, 300, [1, 0, 1]),                  # the shape of the MoE step: K = 7168, twenty column tiles
])
def test_m_grouped_contiguous_gather_equals_the_permuted_copy(groups, n, k, tokens, blocks):
    """Extension entry: the producer gathers the rows of A from an un-permuted matrix through a row list
    (tile::gather4).  Every non-padding row must equal, bit for bit, the plain grouped GEMM on the permuted copy."""
    m = 128 * len(blocks)
    rng = np.random.default_rng(k + tokens)
    src = randn((tokens, k), 5)
    codes, sf = o.quant_mx_host(src, o.FP8, 128)                     # [tokens, k] codes, packed SF [k/512, align4(tokens)]
    row_src = rng.integers(0, tokens, m).astype(np.int32)
    row_src[rng.random(m) < 0.1] = -1                                 # padding rows anywhere
    take = np.maximum(row_src, 0)
    a_codes = codes[take].copy()
    a_codes[row_src < 0] = 0
    a_sf = sf[:, take].copy()
    a_sf[:, row_src < 0] = 0
    sft = lambda w: SfTensor(w.shape[0], w.shape[1], SfGran.G128, dev(np.ascontiguousarray(w).view(np.int32)))
    b, _ = _stacked_b("fp8", groups, n, k, 4, gran=128)
    mi = dev(np.array(blocks, dtype=np.int32))
    want = new_output(m, n, fill=0.0)
    m_grouped_gemm_nt_contiguous(Operand.k_major(Dtype.Fp8, m, k, k, sft(a_sf), dev(a_codes)), b, want, mi, groups)
    got = new_output(m, n, fill=0.0)
    m_grouped_gemm_nt_contiguous_gather(Operand.k_major(Dtype.Fp8, m, k, k, sft(a_sf), dev(codes)), dev(row_src), tokens, b, got, mi, groups)
    poll_device_status()
    g, w = to_f32(got), to_f32(want)
    for r in range(m):
        if blocks[r // 128] >= 0 and row_src[r] >= 0:
            assert np.array_equal(g[r], w[r]), f"row {r}"


def test_m_grouped_contiguous_gather_argument_checks():
    m, n, k = 128, 256, 512
    a, _ = quantised_operand(randn((m, k), 3), "fp8", 128)
    b, _ = _stacked_b("fp8", 1, n, k, 4, gran=128)
    mi = dev(np.zeros(1, dtype=np.int32))
    rows = dev(np.arange(m, dtype=np.int32))
    with pytest.raises(Exception):
        m_grouped_gemm_nt_contiguous_gather(a, rows, 0, b, new_output(m, n), mi, 1)            # no source rows
    a4, _ = quantised_operand(randn((m, k), 3), "fp4", 32)
    b4, _ = _stacked_b("fp4", 1, n, k, 4, gran=32)
    with pytest.raises(Exception):
        m_grouped_gemm_nt_contiguous_gather(a4, rows, m, b4, new_output(m, n), mi, 1)          # FP8 only


def test_m_grouped_contiguous_scatter_and_column_range():
    """Extension entry: rows stored through a row map (negative = dropped), only a column range of
    every expert computed; must equal the same rows / columns of the plain grouped GEMM bit for bit."""
    groups, n, k = 3, 384, 512
    blocks = [2, 0, 0, -1, 1]
    m = 128 * len(blocks)
    a, _ = quantised_operand(randn((m, k), 3), "fp8", 128)
    b, _ = _stacked_b("fp8", groups, n, k, 4, gran=128)
    mi = dev(np.array(blocks, dtype=np.int32))
    full = new_output(m, n, fill=0.0)
    m_grouped_gemm_nt_contiguous(a, b, full, mi, groups)
    rng = np.random.default_rng(0)
    rmap = rng.permutation(m).astype(np.int32)
    rmap[5::7] = -1
    n0, nc = 128, 192
    out = torch.full((m, nc), 9.0, dtype=torch.bfloat16, device="cuda")
    m_grouped_gemm_nt_contiguous_scatter(a, b, Output(Dtype.Bf16, m, nc, nc, out), mi, groups, dev(rmap), n0, nc)
    poll_device_status()
    got, want = out.float().cpu().numpy(), to_f32(full)
    written = np.zeros(m, dtype=bool)
    for r in range(m):
        if blocks[r // 128] >= 0 and rmap[r] >= 0:
            assert np.array_equal(got[rmap[r]], want[r, n0:n0 + nc])
            written[rmap[r]] = True
    assert (got[~written] == 9.0).all()


def test_m_grouped_contiguous_reference_test_shape():
    """deepgemm/tests/e2e_gpu.rs:403-484 with a well-formed m_indices: 4 groups, N 128, K 512."""
    groups, n, k = 4, 128, 512
    m = groups * 128
    a, ga = quantised_operand(randn((m, k), 9), "fp8", 32)
    b, gb = _stacked_b("fp8", groups, n, k, 10)
    out = new_output(m, n)
    m_grouped_fp8_gemm_nt_contiguous(a, b, out, dev(np.arange(groups, dtype=np.int32)), groups)
    poll_device_status()
    got = to_f32(out)
    for g in range(groups):
        rows = np.arange(128 * g, 128 * (g + 1))
        assert_close_to_oracle(got[rows], bf16_round(o.gemm_ref(ga, gb, rows=rows, n=n, b_row0=g * n)), "fp8")


@pytest.mark.parametrize("cluster", [1, 2])
@pytest.mark.parametrize("kind", ["fp8", "fp4", "bf16"])
def test_m_grouped_masked(kind, cluster):
    os.environ["DG_CLUSTER"] = str(cluster)
    groups, max_m, n, k = 6, 256, 384, 512
    masked = [256, 0, 1, 128, 129, 77]
    xa = randn((groups * max_m, k), 71)
    b, gb = _stacked_b(kind, groups, n, k, 72)
    if kind == "bf16":
        a, fa = bf16_operand(xa)
    else:
        a, ga = quantised_operand(xa, kind, 32)
    a.rows = max_m
    out = new_output(groups * max_m, n, fill=5.0)
    out.rows = max_m
    m_grouped_gemm_nt_masked(a, b, out, dev(np.array(masked, dtype=np.int32)), groups, 128)
    poll_device_status()
    got = out.data.float().cpu().numpy()
    for g, mm in enumerate(masked):
        base = g * max_m
        assert (got[base + mm: base + max_m] == 5.0).all(), f"group {g}: rows beyond masked_m were written"
        if mm == 0:
            continue
        rows = np.arange(base, base + mm)
        if kind == "bf16":
            ref = o.gemm_f32_ref(fa[rows], gb[g * n:(g + 1) * n])
        else:
            ref = o.gemm_ref(ga, gb, rows=rows, n=n, b_row0=g * n)
        assert_close_to_oracle(got[rows], bf16_round(ref), kind, f"group {g}")


def test_m_grouped_masked_reference_test_shape():
    """deepgemm/tests/e2e_gpu.rs:328-401: 4 groups, M 64 per group, N 128, K 512, all rows valid."""
    groups, m, n, k = 4, 64, 128, 512
    a, ga = quantised_operand(randn((groups * m, k), 7), "fp8", 32)
    b, gb = _stacked_b("fp8", groups, n, k, 8)
    a.rows = m
    out = new_output(groups * m, n)
    out.rows = m
    m_grouped_fp8_gemm_nt_masked(a, b, out, dev(np.full(groups, m, dtype=np.int32)), groups, m)
    poll_device_status()
    got = out.data.float().cpu().numpy()
    for g in range(groups):
        rows = np.arange(g * m, (g + 1) * m)
        assert_close_to_oracle(got[rows], bf16_round(o.gemm_ref(ga, gb, rows=rows, n=n, b_row0=g * n)), "fp8")


def test_config_introspection():
    cfg = get_gemm_config(Dtype.Fp8, 0, 4096, 7168, 16384)
    assert cfg["block_m"] == 128 * cfg["cluster"] and cfg["block_k"] == 128 and cfg["block_n"] % 32 == 0
    assert cfg["smem_bytes"] <= 232448 and cfg["num_stages"] >= 2
    assert get_gemm_config(Dtype.Fp4, 0, 8192, 8192, 8192)["block_k"] == 256
    assert get_gemm_config(Dtype.Bf16, 0, 2048, 2048, 2048)["block_k"] == 64
