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

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from .api import (_check, _stream_ptr, m_grouped_gemm_nt_contiguous, m_grouped_gemm_nt_contiguous_gather,
                  m_grouped_gemm_nt_contiguous_rowptr, m_grouped_gemm_nt_contiguous_scatter, swiglu_quant)
from .types import Dtype, Operand, Output, SfGran, SfTensor

BLOCK = 128  # rows per m_indices entry (heuristics::mk_alignment_for_contiguous_layout)


def _gather_in_gemm():
    """DG_MOE_GATHER=1 lets the grouped GEMM of the single-GPU step fetch the token rows itself
    (dg_m_grouped_gemm_nt_contiguous_gather) instead of reading a permuted copy written by gather_rows.  Off by
    default: it saves the 1 GB copy and its 0.28 ms, but the 32 four-row TMA instructions a k-block then needs
    cost the GEMM more than that (measured: the step 4.53 ms against 4.38 ms)."""
    import os
    return os.environ.get("DG_MOE_GATHER", "0") == "1"


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


class GroupedMoEFfn:
    """A whole MoE feed-forward layer on one GPU: gate/up grouped GEMM -> SwiGLU + FP8 re-quantisation ->
    down grouped GEMM -> top-k combine.  The reference's Serving::moe_grouped_layer
    (deepgemm/src/api_serving.rs:293-377) stops after the first GEMM and leaves the rest to its caller.

    w13: Operand of the stacked gate/up weights [E * 2 * inter, hidden] (per expert: `inter` gate rows,
    then `inter` up rows), rows = 2 * inter.  w2: Operand of the stacked down weights
    [E * hidden, inter], rows = hidden.  forward(x, x_sf, topk_idx, topk_w) -> bf16 [T, hidden]."""

    def __init__(self, w13: Operand, w2: Operand, num_experts: int, gran: int = 128):
        if w13.rows % 2 or w2.k != w13.rows // 2:
            raise ValueError("w13 must hold 2 * inter rows per expert and w2 must contract over inter")
        self.w13, self.w2, self.num_experts, self.gran = w13, w2, num_experts, gran
        self.inter = w13.rows // 2

    def forward(self, x, x_sf, topk_idx, topk_w=None):
        tokens, topk = topk_idx.shape
        hidden, out_dim = x.shape[1], self.w2.rows
        p = device_plan(topk_idx, self.num_experts, BLOCK, div=topk)
        a = gather_rows(x, p.slot_src)
        a_sf = sf_permute(x_sf, p.slot_src)
        gate_up = torch.empty((p.capacity, 2 * self.inter), dtype=torch.bfloat16, device=x.device)
        m_grouped_gemm_nt_contiguous(Operand.k_major(self.w13.dtype, p.capacity, hidden, hidden, a_sf, a), self.w13,
                                     Output(Dtype.Bf16, p.capacity, 2 * self.inter, 2 * self.inter, gate_up), p.block_expert,
                                     self.num_experts)
        # rows of unused blocks hold whatever the allocation held: they are quantised like the others
        # and never read, because the second GEMM skips their blocks and the combine step their slots
        h, h_sf = swiglu_quant(gate_up, p.capacity, self.inter, self.gran)
        d = torch.empty((p.capacity, out_dim), dtype=torch.bfloat16, device=x.device)
        m_grouped_gemm_nt_contiguous(Operand.k_major(Dtype.Fp8, p.capacity, self.inter, self.inter, h_sf, h), self.w2,
                                     Output(Dtype.Bf16, p.capacity, out_dim, out_dim, d), p.block_expert, self.num_experts)
        return combine(d, p.slot_of_row.view(tokens, topk), topk_w)


def peer_step_tables(tot, me):
    """Host-side index arithmetic of one expert-parallel step over peer memory, for rank `me`.

    tot[src, chunk, dst] = rows that rank src sends to the experts of rank dst in token slice chunk
    (known to every rank after one all-gather).  Returns
      seg[chunk, world + 1]   first received position of every source rank in `me`'s receive area
                              (rows arrive ordered by source rank, then local expert);
      row0[chunk, src]        row of src's return buffer where the results computed by `me` begin
                              (a return buffer holds the slices in order, inside a slice the
                              destination ranks in order: the order of src's sorted copies);
      chunk_base[src, chunk]  first row of every slice in src's return buffer;
      copies[chunk]           list of (dst, first row in my sorted copies, first row in dst's
                              receive area of that slice, rows), destinations rotated so that the
                              ranks do not all push to the same peer at once."""
    tot = np.asarray(tot, dtype=np.int64)
    world, chunks, _ = tot.shape
    seg = np.zeros((chunks, world + 1), dtype=np.int32)
    seg[:, 1:] = np.cumsum(tot[:, :, me].T, axis=1)
    chunk_rows = tot.sum(2)
    chunk_base = np.cumsum(chunk_rows, axis=1) - chunk_rows
    row0 = (chunk_base + tot[:, :, :me].sum(2)).T.astype(np.int32)
    copies = []
    for c in range(chunks):
        lst = []
        for step in range(world):
            dst = (me + 1 + step) % world
            lst.append((dst, int(tot[me, c, :dst].sum()), int(tot[:me, c, dst].sum()), int(tot[me, c, dst])))
        copies.append(lst)
    return seg, row0, chunk_base, copies


class ExpertParallelMoE:
    """Grouped-GEMM MoE projection with experts sharded over the ranks of `group`.

    weights: Operand of the stacked local experts [E_local * n_out, K] (rows = n_out), resident.
    forward(x, x_sf, topk_idx, topk_w): x = FP8 codes [T, K] of this rank's tokens, x_sf their
    packed SF; returns bf16 [T, n_out] = sum_j topk_w[t, j] * (x[t] . W[topk_idx[t, j]]^T).
    """

    def __init__(self, weights: Operand, num_experts: int, group=None, chunks: Optional[int] = None, return_parts: int = 1,
                 transport: str = "push", single_rank_transport: bool = False, slice_weights=None):
        # Transports between several GPUs (one NVSwitch domain):
        # "push": a kernel stores every token copy (row, scale factors, return ticket) straight into
        #   its slot of the expert owner's padded layout, the grouped GEMM stores its result rows
        #   straight into the token owner's buffer, flag barriers replace collectives, and every
        #   position follows on the device from one all-gather of the per-expert counts: a step
        #   never waits on the host.  `chunks` > 1 cuts the local experts into slices whose rows
        #   are pushed while the previous slice's GEMM runs.
        # "peer": dispatch by copy engine into peer-mapped buffers (the host reads the counts to size
        #   the copies), `chunks` token slices pipelined; same return path as "push".
        # "nccl": all-to-alls over NCCL.  There, chunks > 1 pipelines token slices and
        #   return_parts > 1 runs the GEMM of a slice in column ranges whose return transfers overlap
        #   the next range; both overlap NCCL kernels with a GEMM that wants every SM and, measured
        #   on 2 GPUs, lost more than they hid.
        self.transport = os.environ.get("DG_EP_TRANSPORT", transport)
        if self.transport not in ("push", "peer", "nccl"):
            raise ValueError("transport must be 'push', 'peer' or 'nccl'")
        # one rank normally takes the local path below; True runs the chosen transport against itself
        self.single_rank_transport = single_rank_transport or os.environ.get("DG_EP_SINGLE_RANK", "0") == "1"
        self.slice_weights = slice_weights     # push transport: proportions of the expert slices, e.g. (1, 3)
        self._win = None
        self._win_shape = None
        self._streams = None
        self._pinned = None
        self.return_parts = int(os.environ.get("DG_EP_RETURN_PARTS", return_parts))
        self.w = weights
        self.num_experts = num_experts
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.e_local = num_experts // self.world
        # default: four expert slices for the push transport between GPUs (measured best on 2 and 8
        # GPUs), the plain sequence everywhere else
        self.chunks = chunks if chunks is not None else (4 if self.transport == "push" and self.world > 1 else 1)
        self.last_m_indices: Optional[torch.Tensor] = None

    def forward(self, x, x_sf, topk_idx, topk_w=None):
        tokens, topk = topk_idx.shape
        k, n_out = x.shape[1], self.w.rows
        k_elems = k if self.w.dtype != Dtype.Fp4 else k * 2
        if self.world == 1 and not (self.single_rank_transport and self.transport == "push"):
            # one device-side plan straight into the padded layout; no host synchronisation
            p = device_plan(topk_idx, self.num_experts, BLOCK, div=topk)
            a_sf = sf_permute(x_sf, p.slot_src)
            d = torch.empty((p.capacity, n_out), dtype=torch.bfloat16, device=x.device)
            if self.w.dtype == Dtype.Fp8 and x.stride(0) == k and _gather_in_gemm():
                # the GEMM's producer fetches the token rows itself (four per TMA instruction): no permuted copy
                a_op = Operand.k_major(self.w.dtype, p.capacity, k_elems, k_elems, a_sf, x)
                m_grouped_gemm_nt_contiguous_gather(a_op, p.slot_src, tokens, self.w, Output(Dtype.Bf16, p.capacity, n_out, n_out, d),
                                                    p.block_expert, self.e_local)
            else:
                a = gather_rows(x, p.slot_src)
                a_op = Operand.k_major(self.w.dtype, p.capacity, k_elems, k_elems, a_sf, a)
                m_grouped_gemm_nt_contiguous(a_op, self.w, Output(Dtype.Bf16, p.capacity, n_out, n_out, d), p.block_expert,
                                             self.e_local)
            self.last_m_indices = p.block_expert
            return combine(d, p.slot_of_row.view(tokens, topk), topk_w)
        if self.transport in ("push", "peer"):
            from .peer import PeerMappingError
            try:
                if self.transport == "push":
                    return self._forward_push(x, x_sf, topk_idx, topk_w)
                return self._forward_peer(x, x_sf, topk_idx, topk_w)
            except PeerMappingError as ex:
                # raised on all ranks alike, before anything of the step was queued: the GPUs cannot
                # map each other's memory here, so the step goes over NCCL from now on
                import sys
                print(f"[deepgemm] {ex}; expert parallelism falls back to NCCL all-to-alls", file=sys.stderr)
                self.transport, self.chunks, self._win, self._win_shape = "nccl", 1, None, None
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

    # ---- peer-memory transport -------------------------------------------------------------
    def _ensure_window(self, recv_rows_needed, ret_rows_needed, chunks, row_bytes, wire_bytes, n_out):
        """(Re)allocates the peer window when a step needs more room than it has.  Every rank sees the
        same global counts, so all of them take this branch in the same step."""
        shape = self._win_shape
        if shape and shape["chunks"] == chunks and shape["cap"] >= recv_rows_needed and shape["ret_rows"] >= ret_rows_needed \
                and shape["row_bytes"] == row_bytes and shape["wire_bytes"] == wire_bytes and shape["n_out"] == n_out:
            return
        from .peer import PeerWindow
        if self._win is not None:
            self._win.close()
        cap = (int(recv_rows_needed * 1.25) + 1023) // 1024 * 1024
        ret_rows = (int(ret_rows_needed) + 1023) // 1024 * 1024
        a256 = lambda v: (v + 255) // 256 * 256
        off_rows = 0
        off_wire = off_rows + a256(chunks * cap * row_bytes)
        off_ret = off_wire + a256(chunks * cap * wire_bytes)
        total = off_ret + a256(ret_rows * n_out * 2)
        self._win = PeerWindow(total, self.group)
        self._win_shape = dict(chunks=chunks, cap=cap, ret_rows=ret_rows, row_bytes=row_bytes, wire_bytes=wire_bytes, n_out=n_out,
                               off_rows=off_rows, off_wire=off_wire, off_ret=off_ret)
        dev = self._win.local.device
        self._ret_bases = torch.tensor([self._win.payload_ptr(r, off_ret) for r in range(self.world)], dtype=torch.int64, device=dev)
        if self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream())

    def close(self):
        """Collective: releases the peer window."""
        if self._win is not None:
            self._win.close()
            self._win, self._win_shape = None, None

    def _forward_peer(self, x, x_sf, topk_idx, topk_w):
        """Every rank must pass the same number of tokens (the slices and barrier counts follow from it)."""
        L = _lib.load()
        me, world = dist.get_rank(self.group), self.world
        tokens, topk = topk_idx.shape
        k, n_out = x.shape[1], self.w.rows
        k_elems = k if self.w.dtype != Dtype.Fp4 else k * 2
        dev = x.device
        rows_per_expert = tokens * topk * world // self.num_experts
        chunks = max(1, min(self.chunks, rows_per_expert // 1024, tokens // 64 or 1))
        if os.environ.get("DG_EP_CHUNKS"):
            chunks = max(1, int(os.environ["DG_EP_CHUNKS"]))
        bounds = [tokens * c // chunks for c in range(chunks + 1)]
        sps = [device_plan(topk_idx[bounds[c]:bounds[c + 1]], self.num_experts, 1, div=topk,
                           capacity=(bounds[c + 1] - bounds[c]) * topk) for c in range(chunks)]
        send_counts = torch.stack([sp.counts for sp in sps]).view(chunks, world, self.e_local).contiguous()
        full = torch.empty((world, chunks, world, self.e_local), dtype=torch.int32, device=dev)      # [src, chunk, dst, expert]
        dist.all_gather_into_tensor(full, send_counts, group=self.group)
        tot = full.sum(-1).cpu().numpy().astype("int64")                                              # the one host sync of the step
        row_bytes, wire_bytes = k * x.element_size(), x_sf.rows * 4
        self._ensure_window(int(tot.sum(0).max()), int(tot.sum((1, 2)).max()), chunks, row_bytes, wire_bytes, n_out)
        win, sh = self._win, self._win_shape
        comm, ret_stream = self._streams
        main = torch.cuda.current_stream()
        cap = sh["cap"]
        seg, row0, chunk_base, copies = peer_step_tables(tot, me)                                     # uploaded once per step
        # (the pinned staging array is reused: the host synchronisation above has waited for the previous step's upload)
        flat = np.concatenate([seg.reshape(-1), row0.reshape(-1)])
        if self._pinned is None or self._pinned.numel() < flat.size:
            self._pinned = torch.empty(max(flat.size, 1024), dtype=torch.int32).pin_memory()
        self._pinned[:flat.size].copy_(torch.from_numpy(flat))
        tables = self._pinned[:flat.size].to(dev, non_blocking=True)
        seg_dev = tables[:chunks * (world + 1)].view(chunks, world + 1)
        row0_dev = tables[chunks * (world + 1):].view(chunks, world)
        out = torch.empty((tokens, n_out), dtype=torch.bfloat16, device=dev)
        experts = torch.arange(self.e_local, device=dev, dtype=torch.int32).repeat(world)
        recv_rows_all = win.payload(sh["off_rows"], chunks * cap * row_bytes).view(chunks, cap, row_bytes)
        recv_wire_all = win.payload(sh["off_wire"], chunks * cap * wire_bytes).view(torch.int32).view(chunks, cap, x_sf.rows)
        ret_all = win.payload(sh["off_ret"], sh["ret_rows"] * n_out * 2).view(torch.bfloat16).view(sh["ret_rows"], n_out)
        self.last_m_indices = []

        def dispatch(c):
            xs = x[bounds[c]:bounds[c + 1]]
            rows = gather_rows(xs, sps[c].slot_src)
            wire = torch.empty((rows.shape[0], x_sf.rows), dtype=torch.int32, device=dev)
            _gather_sf(x_sf.buf[:, bounds[c]:], x_sf.cols, 1, sps[c].slot_src, wire, 1, x_sf.rows, x_sf.rows)
            ready = torch.cuda.Event()
            ready.record(main)
            arrived = torch.cuda.Event()
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                for dst, src_off, dst_off, n in copies[c]:
                    dst_off += c * cap
                    win.copy_to(dst, sh["off_rows"] + dst_off * row_bytes, rows.data_ptr() + src_off * row_bytes, n * row_bytes)
                    win.copy_to(dst, sh["off_wire"] + dst_off * wire_bytes, wire.data_ptr() + src_off * wire_bytes, n * wire_bytes)
                win.barrier(0)
                arrived.record(comm)
            return dict(keep=(rows, wire), arrived=arrived)

        def compute_and_return(c, st):
            main.wait_event(st["arrived"])
            r = int(tot[:, c, me].sum())
            recv_expert = torch.repeat_interleave(experts, full[:, c, me, :].reshape(-1), output_size=r)
            rp = device_plan(recv_expert, self.e_local, BLOCK, div=1, capacity=contiguous_capacity(r, self.e_local))
            a = gather_rows(recv_rows_all[c, :max(r, 1)].view(x.dtype), rp.slot_src)
            a_sf = sf_from_wire(recv_wire_all[c, :max(r, 1)], rp.slot_src, x_sf.gran)
            ptrs = torch.empty(rp.capacity, dtype=torch.int64, device=dev)
            _check(L.dg_moe_return_ptrs(rp.slot_src.data_ptr(), rp.capacity, seg_dev[c].data_ptr(), self._ret_bases.data_ptr(),
                                        row0_dev[c].data_ptr(), world, n_out * 2, ptrs.data_ptr(), _stream_ptr(None)))
            a_op = Operand.k_major(self.w.dtype, rp.capacity, k_elems, k_elems, a_sf, a)
            self.last_m_indices.append(rp.block_expert)
            m_grouped_gemm_nt_contiguous_rowptr(a_op, self.w, rp.block_expert, self.e_local, ptrs)
            done = torch.cuda.Event()
            done.record(main)
            returned = torch.cuda.Event()
            with torch.cuda.stream(ret_stream):
                ret_stream.wait_event(done)
                win.barrier(1)
                returned.record(ret_stream)
            st["returned"] = returned
            st["keep"] += (a, a_sf, ptrs, rp)

        def finish(c, st):
            main.wait_event(st["returned"])
            tw = topk_w[bounds[c]:bounds[c + 1]] if topk_w is not None else None
            r0 = int(chunk_base[me, c])
            combine(ret_all[r0:r0 + (bounds[c + 1] - bounds[c]) * topk], sps[c].slot_of_row.view(-1, topk), tw,
                    out=out[bounds[c]:bounds[c + 1]])

        states = [None] * chunks
        states[0] = dispatch(0)
        for c in range(chunks):
            if c + 1 < chunks:
                states[c + 1] = dispatch(c + 1)
            compute_and_return(c, states[c])
            if c >= 1:
                finish(c - 1, states[c - 1])
        finish(chunks - 1, states[chunks - 1])
        self._keep = states   # buffers the side streams read stay referenced until the next step replaces them
        return out

    # ---- push transport: no host synchronisation, no staging copies --------------------------
    def _ensure_push_window(self, tokens, topk, row_bytes, sf_rows, n_out, slices):
        key = ("push", tokens, topk, row_bytes, sf_rows, n_out, slices)
        if self._win_shape and self._win_shape.get("key") == key:
            return
        from .peer import PeerWindow
        if self._win is not None:
            self._win.close()
        world = self.world
        # room for the worst case (every copy of every rank routed to this rank) plus padding: no
        # routing can overflow it, so no step has to look at the counts on the host
        cap = (world * tokens * topk + self.e_local * (BLOCK - 1) + BLOCK - 1) // BLOCK * BLOCK
        a256 = lambda v: (v + 255) // 256 * 256
        off_a = 0
        off_sf = off_a + a256(cap * row_bytes)
        off_ticket = off_sf + a256(sf_rows * cap * 4)
        off_ret = off_ticket + a256(cap * 8)
        total = off_ret + a256(tokens * topk * n_out * 2)
        self._win = win = PeerWindow(total, self.group)
        dev = win.local.device
        table = lambda off: torch.tensor([win.payload_ptr(r, off) for r in range(world)], dtype=torch.int64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self._win_shape = dict(key=key, cap=cap, a_bases=table(off_a), sf_bases=table(off_sf), ticket_bases=table(off_ticket),
                               ret_bases=table(off_ret),
                               a=win.payload(off_a, cap * row_bytes).view(cap, row_bytes),
                               sf=win.payload(off_sf, sf_rows * cap * 4).view(torch.int32).view(sf_rows, cap),
                               tickets=win.payload(off_ticket, cap * 8).view(torch.int64),
                               ret=win.payload(off_ret, tokens * topk * n_out * 2).view(torch.bfloat16).view(tokens * topk, n_out),
                               ptrs=torch.empty(cap, dtype=torch.int64, device=dev),
                               dest_base=torch.empty(self.num_experts, **i32),
                               block_expert=torch.empty((slices, cap // BLOCK), **i32),
                               blocks_used=torch.empty(slices, **i32),
                               counts=torch.empty((world, self.num_experts), **i32))
        if self._streams is None:
            self._streams = (torch.cuda.Stream(), torch.cuda.Stream())

    def _slice_bounds(self):
        """First local expert of every slice, plus e_local.  `chunks` (or DG_EP_CHUNKS) = n gives n
        equal slices; DG_EP_SLICES = "1,3" gives slices in those proportions (a small first slice
        starts the GEMM early while the bulk of the rows is still travelling)."""
        spec = os.environ.get("DG_EP_SLICES", self.slice_weights)
        if spec:
            w = [float(v) for v in (spec.split(",") if isinstance(spec, str) else spec)]
        else:
            w = [1.0] * max(1, min(int(os.environ.get("DG_EP_CHUNKS", self.chunks)), self.e_local, 16))
        cuts, acc = [0], 0.0
        for v in w:
            acc += v
            cuts.append(min(self.e_local, max(cuts[-1] + 1, round(self.e_local * acc / sum(w)))))
        cuts[-1] = self.e_local
        cuts = sorted(set(cuts))
        return cuts if len(cuts) >= 2 else [0, self.e_local]

    def _forward_push(self, x, x_sf, topk_idx, topk_w):
        """Every rank must pass the same number of tokens.  The whole step is queued without the host
        ever waiting for the device.  With `chunks` > 1 the local experts are cut into that many
        slices: the rows of slice s + 1 are pushed (by a kernel limited to a few blocks per SM, on a
        second stream) while the GEMM of slice s runs."""
        L = _lib.load()
        world = self.world
        me = dist.get_rank(self.group) if world > 1 else 0
        tokens, topk = topk_idx.shape
        k, n_out = x.shape[1], self.w.rows
        k_elems = k if self.w.dtype != Dtype.Fp4 else k * 2
        row_bytes = k * x.element_size()
        n = tokens * topk
        bounds = self._slice_bounds()
        slices = len(bounds) - 1
        self._ensure_push_window(tokens, topk, row_bytes, x_sf.rows, n_out, slices)
        win, sh = self._win, self._win_shape
        cap = sh["cap"]
        main = torch.cuda.current_stream()
        comm = self._streams[0]
        # my copies sorted by global expert (= by owner rank): counts, first position per expert,
        # token of every position, position of every copy
        p = device_plan(topk_idx, self.num_experts, 1, div=topk, capacity=n)
        if world > 1:
            dist.all_gather_into_tensor(sh["counts"], p.counts, group=self.group)
            counts = sh["counts"]
        else:
            counts = p.counts
        _check(L.dg_ep_route(counts.data_ptr(), world, me, self.num_experts, BLOCK, cap, slices, (C.c_uint32 * len(bounds))(*bounds),
                             sh["dest_base"].data_ptr(), sh["block_expert"].data_ptr(), sh["blocks_used"].data_ptr(),
                             main.cuda_stream))

        def push(s, stream, max_blocks):
            _check(L.dg_ep_push(x.data_ptr(), x.stride(0) * x.element_size(), row_bytes, x_sf.buf.data_ptr(), x_sf.rows, x_sf.cols,
                                p.slot_src.data_ptr(), p.offsets.data_ptr(), sh["dest_base"].data_ptr(), self.num_experts, world,
                                me, bounds[s], bounds[s + 1], n, cap, sh["a_bases"].data_ptr(),
                                sh["sf_bases"].data_ptr(), sh["ticket_bases"].data_ptr(), max_blocks, stream.cuda_stream))
            win.barrier(0, stream.cuda_stream)      # every rank's rows, scale factors and tickets of the slice have landed here

        arrived = []
        if slices > 1:
            routed = torch.cuda.Event()
            routed.record(main)
            comm.wait_event(routed)
            side_blocks = int(os.environ.get("DG_EP_PUSH_BLOCKS", 64))
            for s in range(slices):
                push(s, comm, 0 if s == 0 else side_blocks)
                ev = torch.cuda.Event()
                ev.record(comm)
                arrived.append(ev)
        a_op = Operand.k_major(self.w.dtype, cap, k_elems, k_elems, SfTensor(x_sf.rows, cap, x_sf.gran, sh["sf"]),
                               sh["a"].view(x.dtype))
        self.last_m_indices = sh["block_expert"]
        for s in range(slices):
            if slices > 1:
                main.wait_event(arrived[s])
            else:
                push(0, main, 0)
            blocks = sh["block_expert"][s]
            _check(L.dg_ep_return_ptrs(sh["tickets"].data_ptr(), cap, sh["ret_bases"].data_ptr(), world, n_out * 2,
                                       blocks.data_ptr(), BLOCK, sh["ptrs"].data_ptr(), main.cuda_stream))
            m_grouped_gemm_nt_contiguous_rowptr(a_op, self.w, blocks, self.e_local, sh["ptrs"], m_blocks_used=sh["blocks_used"][s:])
        win.barrier(1, main.cuda_stream)   # every rank's GEMMs have stored their result rows, mine included, into the owners' buffers
        self._keep = p
        return combine(sh["ret"], p.slot_of_row.view(tokens, topk), topk_w)
