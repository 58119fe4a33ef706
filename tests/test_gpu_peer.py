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
