"""Expert-parallel MoE layer step around `m_grouped_gemm_nt_contiguous`.

One process per GPU; rank r owns experts [r*E/n, (r+1)*E/n) with their FP8 weights resident.
A step is: route -> dispatch (all-to-all of FP8 token rows and their scale factors over
NCCL) -> build the 128-row-padded contiguous layout and `m_indices` -> grouped GEMM ->
return (all-to-all of bf16 output rows) -> combine the top-k copies of every token.
The reference has no host-side communication layer (its only expert-parallel code is the
device-side MegaMoE protocol, deepgemm/src/api_mega_moe.rs:1154-1221); the layout conventions
are those of api::m_grouped_gemm_nt_contiguous (deepgemm/src/api.rs:852-903): `m_indices[b]` is
the expert of the b-th 128-row block, negative for padding blocks.

The step's index arithmetic exists twice with one contract: in plain torch (`plan_dispatch`,
`build_contiguous_layout`: device-agnostic, checked on CPU ranks over gloo) and as library
kernels (`device_plan`, used by `ExpertParallelMoE` so that a step needs no host
synchronisation on one GPU and exactly one on several).
"""
import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from .api import _check, _stream_ptr, m_grouped_gemm_nt_contiguous, m_grouped_gemm_nt_contiguous_scatter
from .types import Dtype, Operand, Output, SfGran, SfTensor

BLOCK = 128  # rows per m_indices entry (heuristics::mk_alignment_for_contiguous_layout)


@dataclass
class ContiguousLayout:
    """Placement of `rows` grouped rows into the padded contiguous layout."""
    m_cap: int                  # allocated rows (a multiple of 128; trailing blocks are padding)
    src_row: torch.Tensor       # int32 [m_cap]: source row of every slot, -1 = padding row
    slot_of_row: torch.Tensor   # int32 [rows]: slot of every source row
    m_indices: torch.Tensor     # int32 [m_cap / 128]: expert of each block, -1 = skip
    counts: torch.Tensor        # int64 [num_experts]


def contiguous_capacity(rows, num_experts):
    """Rows that are always enough: every expert may waste up to 127 padding rows."""
    return (rows + num_experts * (BLOCK - 1) + BLOCK - 1) // BLOCK * BLOCK


def build_contiguous_layout(expert_of_row, num_experts, m_cap=None):
    """expert_of_row: int tensor [rows] (any device).  Rows keep their relative order inside an
    expert's group; each group is padded to a multiple of 128 rows.  No host synchronisation."""
    e = expert_of_row.to(torch.int64)
    rows = e.numel()
    dev = e.device
    if m_cap is None:
        m_cap = contiguous_capacity(rows, num_experts)
    counts = torch.bincount(e, minlength=num_experts)
    padded = (counts + BLOCK - 1) // BLOCK * BLOCK
    pad_end = torch.cumsum(padded, 0)
    pad_off = pad_end - padded
    off = torch.cumsum(counts, 0) - counts
    order = torch.argsort(e, stable=True)
    e_sorted = e[order]
    slot_sorted = pad_off[e_sorted] + (torch.arange(rows, device=dev) - off[e_sorted])
    src_row = torch.full((m_cap,), -1, dtype=torch.int32, device=dev)
    src_row[slot_sorted] = order.to(torch.int32)
    slot_of_row = torch.empty(rows, dtype=torch.int32, device=dev)
    slot_of_row[order] = slot_sorted.to(torch.int32)
    blocks = torch.arange(m_cap // BLOCK, device=dev)
    owner = torch.searchsorted(pad_end // BLOCK, blocks, right=True)
    m_indices = torch.where(blocks < pad_end[-1] // BLOCK, owner, torch.full_like(owner, -1)).to(torch.int32)
    return ContiguousLayout(m_cap, src_row, slot_of_row, m_indices, counts)


@dataclass
class DispatchPlan:
    """Everything a rank needs to ship its token copies to the expert owners and back."""
    order: torch.Tensor          # int64 [T*k]: copies sorted by global expert (= by destination rank)
    send_token: torch.Tensor     # int32 [T*k]: token row of every sorted copy
    copy_pos: torch.Tensor       # int32 [T, k]: position of copy (t, j) in the sorted order
    send_splits: list            # rows to every rank
    recv_splits: list            # rows from every rank
    recv_expert: torch.Tensor    # int64 [R]: local expert of every received row
    layout: ContiguousLayout     # placement of the R received rows


def plan_dispatch(topk_idx, num_experts, group=None):
    """topk_idx: int tensor [T, k] of global expert ids.  Exchanges the per-expert counts (one
    all-to-all of world*E_local integers, plus one device-to-host copy of the split sizes)."""
    world = dist.get_world_size(group) if group is not None else 1
    e_local = num_experts // world
    flat = topk_idx.reshape(-1).to(torch.int64)
    dev = flat.device
    order = torch.argsort(flat, stable=True)
    send_token = (order // topk_idx.shape[1]).to(torch.int32)
    copy_pos = torch.empty_like(order)
    copy_pos[order] = torch.arange(order.numel(), device=dev)
    send_counts = torch.bincount(flat, minlength=num_experts).reshape(world, e_local)
    if world > 1:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
    else:
        recv_counts = send_counts
    both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    # received rows arrive ordered by (source rank, local expert)
    recv_expert = torch.repeat_interleave(torch.arange(e_local, device=dev).repeat(world), recv_counts.reshape(-1),
                                          output_size=sum(recv_splits))
    # capacity from the received row count only (known on the host), so every rank allocates alike per step
    layout = build_contiguous_layout(recv_expert, e_local, contiguous_capacity(sum(recv_splits), e_local))
    return DispatchPlan(order, send_token, copy_pos.reshape(topk_idx.shape).to(torch.int32), send_splits, recv_splits,
                        recv_expert, layout)


# ---- device-side plan (library kernels; same contract as build_contiguous_layout) ---------------
@dataclass
class DevicePlan:
    counts: torch.Tensor        # int32 [E]
    offsets: torch.Tensor       # int32 [E + 1]
    slot_src: torch.Tensor      # int32 [capacity]: row // div of each slot, -1 = padding
    slot_of_row: torch.Tensor   # int32 [rows]
    block_expert: torch.Tensor  # int32 [capacity / align]
    capacity: int


def device_plan(expert_of_row, num_experts, align, div=1, capacity=None):
    """Groups rows by expert on the device without any host synchronisation (dg_moe_plan).
    Unlike build_contiguous_layout the order of rows inside a group is not fixed; nothing
    downstream depends on it."""
    e = expert_of_row.reshape(-1)
    if e.dtype != torch.int32 or not e.is_contiguous():
        e = e.to(torch.int32).contiguous()
    rows = e.numel()
    if capacity is None:
        capacity = (rows + num_experts * (align - 1) + align - 1) // align * align
    dev = e.device
    i32 = dict(dtype=torch.int32, device=dev)
    counts, offsets, cursors = torch.empty(num_experts, **i32), torch.empty(num_experts + 1, **i32), torch.empty(num_experts, **i32)
    slot_src, slot_of_row = torch.empty(max(capacity, 1), **i32), torch.empty(max(rows, 1), **i32)
    block_expert = torch.empty(max(capacity // align, 1), **i32)
    _check(_lib.load().dg_moe_plan(e.data_ptr(), rows, num_experts, align, div, capacity, counts.data_ptr(), offsets.data_ptr(),
                                   cursors.data_ptr(), slot_src.data_ptr(), slot_of_row.data_ptr(), block_expert.data_ptr(),
                                   _stream_ptr(None)))
    return DevicePlan(counts, offsets, slot_src[:capacity], slot_of_row[:rows], block_expert[:capacity // align], capacity)


# ---- data movement (library kernels) -----------------------------------------------------------
def gather_rows(src, idx, out=None):
    """out[i] = src[idx[i]] (zeros for idx < 0) for 2-D byte / bf16 tensors with 16-byte rows."""
    n = idx.numel()
    row_bytes = src.shape[1] * src.element_size()
    if out is None:
        out = torch.empty((n, src.shape[1]), dtype=src.dtype, device=src.device)
    _check(_lib.load().dg_gather_rows(src.data_ptr(), src.stride(0) * src.element_size(), idx.data_ptr(), out.data_ptr(),
                                      out.stride(0) * out.element_size(), n, row_bytes, _stream_ptr(None)))
    return out


def _gather_sf(src, src_rs, src_cs, idx, dst, dst_rs, dst_cs, sf_rows):
    _check(_lib.load().dg_gather_sf(src.data_ptr(), src_rs, src_cs, idx.data_ptr(), dst.data_ptr(), dst_rs, dst_cs,
                                    sf_rows, idx.numel(), _stream_ptr(None)))


def sf_to_wire(sf, idx):
    """Packed SF [sf_rows, cols] -> row-per-token words [len(idx), sf_rows]."""
    wire = torch.empty((idx.numel(), sf.rows), dtype=torch.int32, device=sf.buf.device)
    _gather_sf(sf.buf, sf.cols, 1, idx, wire, 1, sf.rows, sf.rows)
    return wire


def sf_from_wire(wire, idx, gran):
    """Row-per-token words [R, sf_rows] -> packed SF tensor whose column i is wire row idx[i]."""
    sf_rows = wire.shape[1]
    cols = idx.numel()
    buf = torch.empty((sf_rows, cols), dtype=torch.int32, device=wire.device)
    _gather_sf(wire, 1, sf_rows, idx, buf, cols, 1, sf_rows)
    return SfTensor(sf_rows, cols, SfGran(int(gran)), buf)


def sf_permute(sf, idx):
    buf = torch.empty((sf.rows, idx.numel()), dtype=torch.int32, device=sf.buf.device)
    _gather_sf(sf.buf, sf.cols, 1, idx, buf, idx.numel(), 1, sf.rows)
    return SfTensor(sf.rows, idx.numel(), sf.gran, buf)


def combine(src, pos, weights, out=None):
    """out[t] = sum_j weights[t, j] * src[pos[t, j]] (bf16 rows, f32 accumulation)."""
    tokens, topk = pos.shape
    if out is None:
        out = torch.empty((tokens, src.shape[1]), dtype=torch.bfloat16, device=src.device)
    _check(_lib.load().dg_moe_combine(src.data_ptr(), src.stride(0), pos.data_ptr(),
                                      weights.data_ptr() if weights is not None else None, out.data_ptr(), out.stride(0),
                                      tokens, topk, src.shape[1], _stream_ptr(None)))
    return out


class ExpertParallelMoE:
    """Grouped-GEMM MoE projection with experts sharded over the ranks of `group`.

    weights: Operand of the stacked local experts [E_local * n_out, K] (rows = n_out), resident.
    forward(x, x_sf, topk_idx, topk_w): x = FP8 codes [T, K] of this rank's tokens, x_sf their
    packed SF; returns bf16 [T, n_out] = sum_j topk_w[t, j] * (x[t] . W[topk_idx[t, j]]^T).
    """

    def __init__(self, weights: Operand, num_experts: int, group=None, chunks: int = 1, return_parts: int = 1):
        # chunks > 1: token slices pipelined through dispatch / GEMM / return; return_parts > 1: the
        # GEMM of a slice runs in column ranges whose return transfers overlap the next range.  Both
        # overlap NCCL kernels with a GEMM that wants every SM; measured on 2 GPUs they lost more
        # than they hid, so the default is the plain sequence.
        self.chunks = chunks
        self.return_parts = int(os.environ.get("DG_EP_RETURN_PARTS", return_parts))
        self.w = weights
        self.num_experts = num_experts
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.e_local = num_experts // self.world
        self.last_m_indices: Optional[torch.Tensor] = None

    def forward(self, x, x_sf, topk_idx, topk_w=None):
        tokens, topk = topk_idx.shape
        k, n_out = x.shape[1], self.w.rows
        k_elems = k if self.w.dtype != Dtype.Fp4 else k * 2
        if self.world == 1:
            # one device-side plan straight into the padded layout; no host synchronisation
            p = device_plan(topk_idx, self.num_experts, BLOCK, div=topk)
            a = gather_rows(x, p.slot_src)
            a_sf = sf_permute(x_sf, p.slot_src)
            d = torch.empty((p.capacity, n_out), dtype=torch.bfloat16, device=x.device)
            a_op = Operand.k_major(self.w.dtype, p.capacity, k_elems, k_elems, a_sf, a)
            m_grouped_gemm_nt_contiguous(a_op, self.w, Output(Dtype.Bf16, p.capacity, n_out, n_out, d), p.block_expert,
                                         self.e_local)
            self.last_m_indices = p.block_expert
            return combine(d, p.slot_of_row.view(tokens, topk), topk_w)
        # Several GPUs: the tokens are cut into `chunks` slices that flow through
        # dispatch -> GEMM -> return as a pipeline, so that NCCL traffic of one slice overlaps the
        # grouped GEMM of another.  All count exchanges happen first (one all-to-all, one host sync).
        # Every slice re-reads this rank's expert weights, so slices must stay large: about
        # 1024 rows per local expert and slice.
        rows_per_expert = tokens * topk * self.world // self.num_experts
        chunks = max(1, min(self.chunks, rows_per_expert // 1024, tokens // 64 or 1))
        if os.environ.get("DG_EP_CHUNKS"):
            chunks = max(1, int(os.environ["DG_EP_CHUNKS"]))
        bounds = [tokens * c // chunks for c in range(chunks + 1)]
        sps = [device_plan(topk_idx[bounds[c]:bounds[c + 1]], self.num_experts, 1, div=topk,
                           capacity=(bounds[c + 1] - bounds[c]) * topk) for c in range(chunks)]
        send_counts = torch.stack([sp.counts for sp in sps]).view(chunks, self.world, self.e_local)
        send_counts = send_counts.permute(1, 0, 2).contiguous()                       # [dst, chunk, expert]
        recv_counts = torch.empty_like(send_counts)                                   # [src, chunk, expert]
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts.sum(2), recv_counts.sum(2)]).cpu()            # the one host sync of the step
        out = torch.empty((tokens, n_out), dtype=torch.bfloat16, device=x.device)
        experts = torch.arange(self.e_local, device=x.device, dtype=torch.int32).repeat(self.world)
        self.last_m_indices = []

        def dispatch(c):
            send_splits, recv_splits = both[0][:, c].tolist(), both[1][:, c].tolist()
            xs = x[bounds[c]:bounds[c + 1]]
            rows = gather_rows(xs, sps[c].slot_src)
            # scale factors of the slice: columns bounds[c].. of the packed tensor
            sf_view = SfTensor(x_sf.rows, x_sf.cols, x_sf.gran, x_sf.buf[:, bounds[c]:])
            wire = torch.empty((rows.shape[0], x_sf.rows), dtype=torch.int32, device=x.device)
            _gather_sf(sf_view.buf, x_sf.cols, 1, sps[c].slot_src, wire, 1, x_sf.rows, x_sf.rows)
            r = sum(recv_splits)
            recv_rows = torch.empty((r, k), dtype=x.dtype, device=x.device)
            recv_wire = torch.empty((r, x_sf.rows), dtype=torch.int32, device=x.device)
            w1 = dist.all_to_all_single(recv_rows, rows, recv_splits, send_splits, group=self.group, async_op=True)
            w2 = dist.all_to_all_single(recv_wire, wire, recv_splits, send_splits, group=self.group, async_op=True)
            return dict(send_splits=send_splits, recv_splits=recv_splits, recv_rows=recv_rows, recv_wire=recv_wire,
                        works=(w1, w2), keep=(rows, wire), r=r)

        def compute_and_return(c, st):
            for w in st["works"]:
                w.wait()
            r = st["r"]
            # received rows are ordered by (source rank, local expert)
            recv_expert = torch.repeat_interleave(experts, recv_counts[:, c, :].reshape(-1), output_size=r)
            rp = device_plan(recv_expert, self.e_local, BLOCK, div=1, capacity=contiguous_capacity(r, self.e_local))
            a = gather_rows(st["recv_rows"], rp.slot_src)
            a_sf = sf_from_wire(st["recv_wire"], rp.slot_src, x_sf.gran)
            # The GEMM epilogue stores every slot's row at its position in the received order, the
            # order the return all-to-all needs.  With a single slice the GEMM runs in column
            # halves, so that the first half travels back while the second is computed.
            a_op = Operand.k_major(self.w.dtype, rp.capacity, k_elems, k_elems, a_sf, a)
            self.last_m_indices.append(rp.block_expert)
            rows_back = (bounds[c + 1] - bounds[c]) * topk
            parts = self.return_parts if n_out % (64 * self.return_parts) == 0 else 1
            st["ret"], st["back"], st["ret_work"] = [], [], []
            for h in range(parts):
                n0, nc = n_out // parts * h, n_out // parts
                back = torch.empty((max(r, 1), nc), dtype=torch.bfloat16, device=x.device)
                m_grouped_gemm_nt_contiguous_scatter(a_op, self.w, Output(Dtype.Bf16, max(r, 1), nc, nc, back),
                                                     rp.block_expert, self.e_local, rp.slot_src, n0, nc)
                ret = torch.empty((rows_back, nc), dtype=torch.bfloat16, device=x.device)
                st["back"].append(back)
                st["ret"].append(ret)
                st["ret_work"].append(dist.all_to_all_single(ret, back[:r], st["send_splits"], st["recv_splits"],
                                                             group=self.group, async_op=True))

        def finish(c, st):
            tw = topk_w[bounds[c]:bounds[c + 1]] if topk_w is not None else None
            pos = sps[c].slot_of_row.view(-1, topk)
            col = 0
            for work, ret in zip(st["ret_work"], st["ret"]):
                work.wait()
                combine(ret, pos, tw, out=out[bounds[c]:bounds[c + 1], col:col + ret.shape[1]])
                col += ret.shape[1]

        # issue order on the NCCL stream: d0, d1, r0, d2, r1, ..., r_last
        states = [None] * chunks
        states[0] = dispatch(0)
        for c in range(chunks):
            if c + 1 < chunks:
                states[c + 1] = dispatch(c + 1)
            compute_and_return(c, states[c])
            if c >= 1:
                finish(c - 1, states[c - 1])
        finish(chunks - 1, states[chunks - 1])
        return out
