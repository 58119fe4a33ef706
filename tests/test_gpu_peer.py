"""Single-GPU checks of the peer-memory entries: the grouped GEMM that stores rows through an
address table against the plain grouped GEMM (bit for bit), the return-address kernel against its
definition, and the flag barrier with one rank.  The two-rank step is in test_gpu_moe_ep.py."""
import ctypes as C

import numpy as np
import pytest
import torch

from deepgemm import _lib, m_grouped_gemm_nt_contiguous, m_grouped_gemm_nt_contiguous_rowptr, poll_device_status
from helpers import dev, new_output, quantised_operand, randn, to_f32
from test_gpu_gemm import _stacked_b

pytestmark = pytest.mark.gpu


def test_rowptr_gemm_equals_plain_grouped_gemm():
    groups, n, k = 3, 384, 512
    blocks = [2, 0, 0, -1, 1]
    m = 128 * len(blocks)
    a, _ = quantised_operand(randn((m, k), 3), "fp8", 128)
    b, _ = _stacked_b("fp8", groups, n, k, 4, gran=128)
    mi = dev(np.array(blocks, dtype=np.int32))
    full = new_output(m, n, fill=0.0)
    m_grouped_gemm_nt_contiguous(a, b, full, mi, groups)
    rng = np.random.default_rng(1)
    rmap = rng.permutation(m).astype(np.int64)
    rmap[3::5] = -1
    for n0, nc in ((0, 0), (128, 192)):
        cols = nc or n
        pitch = cols + 8                                  # rows of the target need not be dense
        out = torch.full((m, pitch), 9.0, dtype=torch.bfloat16, device="cuda")
        ptrs = np.where(rmap >= 0, out.data_ptr() + rmap * pitch * 2, 0).astype(np.int64)
        m_grouped_gemm_nt_contiguous_rowptr(a, b, mi, groups, torch.from_numpy(ptrs).cuda(), n0, nc)
        poll_device_status()
        got, want = out.float().cpu().numpy(), to_f32(full)
        written = np.zeros(m, dtype=bool)
        for r in range(m):
            if blocks[r // 128] >= 0 and rmap[r] >= 0:
                assert np.array_equal(got[rmap[r], :cols], want[r, n0:n0 + cols])
                written[rmap[r]] = True
        assert (got[~written] == 9.0).all() and (got[:, cols:] == 9.0).all()


def test_return_ptrs_kernel_matches_definition():
    L = _lib.load()
    world, slots, row_bytes = 3, 640, 512
    seg = np.array([0, 150, 150, 420], dtype=np.int32)            # rank 1 sent nothing
    rng = np.random.default_rng(2)
    slot_src = np.full(slots, -1, dtype=np.int32)
    slot_src[rng.permutation(slots)[:420]] = rng.permutation(420).astype(np.int32)
    base = np.array([1 << 40, 2 << 40, 3 << 40], dtype=np.int64)
    row0 = np.array([7, 0, 1000], dtype=np.int32)
    ptrs = torch.zeros(slots, dtype=torch.int64, device="cuda")
    t = [torch.from_numpy(v).cuda() for v in (slot_src, seg, base, row0)]
    assert L.dg_moe_return_ptrs(t[0].data_ptr(), slots, t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), world, row_bytes,
                                ptrs.data_ptr(), None) == 0
    got = ptrs.cpu().numpy()
    for s in range(slots):
        i = slot_src[s]
        if i < 0:
            assert got[s] == 0
        else:
            r = 0 if i < 150 else 2
            assert got[s] == base[r] + (row0[r] + i - seg[r]) * row_bytes


def test_peer_barrier_single_rank_and_copy():
    L = _lib.load()
    p = C.c_void_p()
    assert L.dg_peer_alloc(8192, C.byref(p)) == 0
    try:
        handle = C.create_string_buffer(64)
        assert L.dg_peer_export(p.value, handle) == 0
        table = torch.tensor([p.value], dtype=torch.int64, device="cuda")
        for seq in (1, 2, 3):
            assert L.dg_peer_barrier(table.data_ptr(), p.value, 0, 1, seq, None) == 0
        poll_device_status()
        src = torch.arange(256, dtype=torch.int32, device="cuda")
        assert L.dg_peer_copy(p.value + 4096, src.data_ptr(), 1024, None) == 0
        back = torch.empty_like(src)
        assert L.dg_peer_copy(back.data_ptr(), p.value + 4096, 1024, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(back, src)
        flags = torch.empty(1, dtype=torch.int64, device="cuda")
        assert L.dg_peer_copy(flags.data_ptr(), p.value, 8, None) == 0
        torch.cuda.synchronize()
        assert int(flags.item()) == 3
        assert L.dg_peer_barrier(table.data_ptr(), p.value, 1, 1, 4, None) != 0     # rank outside the world
    finally:
        assert L.dg_peer_free(p.value) == 0


@pytest.mark.parametrize("slices", [1, 3])
def test_push_transport_against_itself_equals_local_step(slices):
    """The push transport run by one rank against its own window (route -> push -> tickets ->
    row-pointer GEMM -> combine, worst-case capacity, device-side block bound) must reproduce the
    local step bit for bit, also when the buffers are reused by a second and third step."""
    import os
    from deepgemm import Dtype, moe, quant_mx, synth
    E, TOPK, T, K, N = 6, 2, 300, 512, 256
    dev_ = torch.device("cuda")
    w = synth.random_expert_weights(E, N, K, seed=5, device=dev_)
    local = moe.ExpertParallelMoE(w, E, None)
    layer = moe.ExpertParallelMoE(w, E, None, chunks=slices, transport="push", single_rank_transport=True)
    os.environ.pop("DG_EP_CHUNKS", None)
    try:
        for step in range(3):
            g = torch.Generator(device=dev_).manual_seed(80 + step % 2)
            x = torch.randn((T, K), device=dev_, generator=g)
            x8, x_sf = quant_mx(x, T, K, Dtype.Fp8, 128)
            idx, tw = synth.random_topk_routing(T, E, TOPK, seed=90 + step % 2, device=dev_)
            if step == 2:
                idx = torch.where(idx == 4, torch.full_like(idx, 3), idx)   # an expert without rows, duplicates allowed
            want = local.forward(x8, x_sf, idx, tw)
            got = layer.forward(x8, x_sf, idx, tw)
            poll_device_status()
            assert torch.equal(got, want), f"step {step}"
    finally:
        layer.close()


def test_barrier_gives_up_on_a_missing_rank_and_reports_it(monkeypatch):
    """Failure detection without a fault: rank 1 of a two-rank barrier never writes its flag; the
    wait runs out (shortened to 0.3 s), the kernel returns, the status word names the rank and the
    context stays usable."""
    from deepgemm import DeviceTimeout
    L = _lib.load()
    monkeypatch.setenv("DG_PEER_WAIT_MS", "300")
    mine, other = C.c_void_p(), C.c_void_p()
    assert L.dg_peer_alloc(4096, C.byref(mine)) == 0 and L.dg_peer_alloc(4096, C.byref(other)) == 0
    try:
        table = torch.tensor([mine.value, other.value], dtype=torch.int64, device="cuda")
        assert L.dg_peer_barrier(table.data_ptr(), mine.value, 0, 2, 1, None) == 0
        with pytest.raises(DeviceTimeout, match="rank 1"):
            poll_device_status()
        poll_device_status()                                   # the word was cleared; the GPU still answers
        assert int(torch.arange(4, device="cuda").sum().item()) == 6
    finally:
        assert L.dg_peer_free(mine.value) == 0 and L.dg_peer_free(other.value) == 0


def test_route_reports_a_layout_overflow():
    """More rows than the owner's layout holds: dg_ep_route marks the expert's copies as dropped
    (dest_base -1) and the status word says so."""
    from deepgemm import DgError
    L = _lib.load()
    counts = torch.tensor([[100, 300, 50, 20]], dtype=torch.int32, device="cuda")     # one rank, four experts
    dest = torch.empty(4, dtype=torch.int32, device="cuda")
    blocks = torch.empty(4, dtype=torch.int32, device="cuda")
    used = torch.empty(1, dtype=torch.int32, device="cuda")
    assert L.dg_ep_route(counts.data_ptr(), 1, 0, 4, 128, 512, 1, None, dest.data_ptr(), blocks.data_ptr(), used.data_ptr(), None) == 0
    with pytest.raises(DgError, match="exceed"):
        poll_device_status()
    assert dest.cpu().tolist() == [0, 128, -1, -1]             # 128 + 384 rows fit into 512, the rest does not
    assert blocks.cpu().tolist() == [0, 1, 1, 1] and used.item() == 4


@pytest.mark.parametrize("world,slices", [(2, 1), (3, 2), (4, 2), (8, 1)])
def test_push_dispatch_with_emulated_ranks_equals_local_steps(world, slices):
    """The whole push transport for `world` ranks played on one GPU: every rank has its own buffers
    (plain device tensors standing in for the peer windows), the kernels of the ranks run one after
    the other (none waits for another), and every rank's combined output must equal its single-rank
    step with all experts resident, bit for bit.  Covers the slot arithmetic of dg_ep_route for any
    rank count (rotated source order, padded expert bases, slices), dg_ep_push, the tickets and the
    row-pointer GEMM."""
    from deepgemm import Dtype, Operand, SfGran, SfTensor, moe, quant_mx, synth
    L = _lib.load()
    e_local, topk, T, K, N = 2, 2, 50, 512, 128
    E = world * e_local
    d0 = torch.device("cuda")
    full = synth.random_expert_weights(E, N, K, seed=21, device=d0)
    local_layer = moe.ExpertParallelMoE(full, E, None)
    ranks = []
    for r in range(world):
        g = torch.Generator(device=d0).manual_seed(100 + r)
        x8, x_sf = quant_mx(torch.randn((T, K), device=d0, generator=g), T, K, Dtype.Fp8, 128)
        idx, tw = synth.random_topk_routing(T, E, topk, seed=200 + r, device=d0)
        ranks.append(dict(x=x8, sf=x_sf, idx=idx, tw=tw, want=local_layer.forward(x8, x_sf, idx, tw),
                          plan=moe.device_plan(idx, E, 1, div=topk, capacity=T * topk)))
    n = T * topk
    cap = (world * n + e_local * 127 + 127) // 128 * 128
    sf_rows = ranks[0]["sf"].rows
    i32, i64 = dict(dtype=torch.int32, device=d0), dict(dtype=torch.int64, device=d0)
    for rk in ranks:
        rk.update(a=torch.zeros((cap, K), dtype=torch.uint8, device=d0), asf=torch.zeros((sf_rows, cap), **i32),
                  tickets=torch.zeros(cap, **i64), ret=torch.full((n, N), 7.0, dtype=torch.bfloat16, device=d0),
                  dest=torch.empty(E, **i32), blocks=torch.empty((slices, cap // 128), **i32), used=torch.empty(slices, **i32),
                  ptrs=torch.zeros(cap, **i64))
    table = lambda key: torch.tensor([rk[key].data_ptr() for rk in ranks], **i64)
    a_bases, sf_bases, ticket_bases, ret_bases = table("a"), table("asf"), table("tickets"), table("ret")
    counts = torch.stack([rk["plan"].counts for rk in ranks]).contiguous()
    for me, rk in enumerate(ranks):
        assert L.dg_ep_route(counts.data_ptr(), world, me, E, 128, cap, slices, None, rk["dest"].data_ptr(), rk["blocks"].data_ptr(),
                             rk["used"].data_ptr(), None) == 0
    bounds = [e_local * s // slices for s in range(slices + 1)]
    for s in range(slices):
        for me, rk in enumerate(ranks):
            assert L.dg_ep_push(rk["x"].data_ptr(), K, K, rk["sf"].buf.data_ptr(), sf_rows, rk["sf"].cols, rk["plan"].slot_src.data_ptr(),
                                rk["plan"].offsets.data_ptr(), rk["dest"].data_ptr(), E, world, me, bounds[s], bounds[s + 1], n, cap,
                                a_bases.data_ptr(), sf_bases.data_ptr(), ticket_bases.data_ptr(), 0 if s == 0 else 8, None) == 0
        for d, rk in enumerate(ranks):
            assert L.dg_ep_return_ptrs(rk["tickets"].data_ptr(), cap, ret_bases.data_ptr(), world, N * 2, rk["blocks"][s].data_ptr(), 128,
                                       rk["ptrs"].data_ptr(), None) == 0
            rows = slice(d * e_local * N, (d + 1) * e_local * N)
            w_local = Operand.k_major(Dtype.Fp8, N, K, K, SfTensor(full.sf.rows, e_local * N, SfGran.G128, full.sf.buf[:, rows].contiguous()),
                                      full.data[rows].contiguous())
            a_op = Operand.k_major(Dtype.Fp8, cap, K, K, SfTensor(sf_rows, cap, SfGran.G128, rk["asf"]), rk["a"])
            m_grouped_gemm_nt_contiguous_rowptr(a_op, w_local, rk["blocks"][s], e_local, rk["ptrs"], m_blocks_used=rk["used"][s:])
    poll_device_status()
    for r, rk in enumerate(ranks):
        assert int(rk["tickets"].abs().sum().item()) == 0, "tickets must be cleared for the next step"
        got = moe.combine(rk["ret"], rk["plan"].slot_of_row.view(T, topk), rk["tw"])
        assert torch.equal(got, rk["want"]), f"rank {r} of {world}"
