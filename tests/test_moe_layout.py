"""Host-side logic of the expert-parallel MoE step (index arithmetic and count exchange), on
CPU: single rank, and world_size 2 over gloo with the data movement emulated in numpy."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepgemm.moe import BLOCK, build_contiguous_layout, contiguous_capacity, plan_dispatch


def _routing(tokens, experts, topk, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int32)


def test_contiguous_layout_groups_and_pads():
    e = torch.tensor([3, 1, 3, 3, 0, 1, 3], dtype=torch.int32)
    lay = build_contiguous_layout(e, 5)
    assert lay.m_cap == contiguous_capacity(7, 5) and lay.m_cap % BLOCK == 0
    assert lay.counts.tolist() == [1, 2, 0, 4, 0]
    # experts 0, 1, 3 get one 128-row block each; expert 2 and 4 none; the rest is padding
    assert lay.m_indices.tolist()[:4] == [0, 1, 3, -1]
    assert (lay.m_indices[3:] == -1).all()
    src = lay.src_row.numpy()
    assert src[0] == 4 and list(src[128:130]) == [1, 5] and list(src[256:260]) == [0, 2, 3, 6]
    assert (src[1:128] == -1).all() and (src[260:] == -1).all()
    assert all(src[lay.slot_of_row[i]] == i for i in range(7))


def test_contiguous_layout_empty_and_exact_blocks():
    lay = build_contiguous_layout(torch.zeros(256, dtype=torch.int32), 2)
    assert lay.m_indices.tolist()[:3] == [0, 0, -1]
    lay = build_contiguous_layout(torch.zeros(0, dtype=torch.int32), 4)
    assert (lay.m_indices == -1).all() and (lay.src_row == -1).all()


def test_plan_single_rank_round_trip():
    T, E, K = 50, 16, 4
    idx = _routing(T, E, K, 0)
    plan = plan_dispatch(idx, E)
    lay = plan.layout
    x = np.arange(T, dtype=np.int64)
    sorted_tokens = x[plan.send_token.numpy()]
    assert plan.send_splits == [T * K] and plan.recv_splits == [T * K]
    slots = np.full(lay.m_cap, -1)
    valid = lay.src_row.numpy() >= 0
    slots[valid] = sorted_tokens[lay.src_row.numpy()[valid]]
    for b, e in enumerate(lay.m_indices.tolist()):
        blk = slots[b * BLOCK:(b + 1) * BLOCK]
        if e < 0:
            assert (blk == -1).all()
            continue
        for t in blk[blk >= 0]:
            assert e in idx[t].tolist()
    # every copy (t, j) sits in a block of its expert and maps back to token t
    pos = lay.slot_of_row[plan.copy_pos.long()].numpy()
    for t in range(T):
        for j in range(K):
            assert slots[pos[t, j]] == t
            assert lay.m_indices[pos[t, j] // BLOCK] == idx[t, j]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ep_worker(rank, world, port, T, E, K, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        idx = _routing(T, E, K, 100 + rank)
        plan = plan_dispatch(idx, E, dist.group.WORLD)
        e_local = E // world
        # emulate the wire with an all-to-all of (token id, source rank, global expert) triples
        flat = idx.reshape(-1).long()
        payload = torch.stack([plan.send_token.long(), torch.full_like(flat, rank), flat[plan.order]], 1).contiguous()
        recv = torch.empty((sum(plan.recv_splits), 3), dtype=torch.int64)
        dist.all_to_all_single(recv, payload, plan.recv_splits, plan.send_splits)
        lay = plan.layout
        # every received row belongs to a local expert and the plan predicted which one
        assert ((recv[:, 2] // e_local) == rank).all()
        assert (recv[:, 2] % e_local == plan.recv_expert).all()
        # rows sit in blocks of their expert
        src = lay.src_row.long()
        for b, e in enumerate(lay.m_indices.tolist()):
            rows = src[b * BLOCK:(b + 1) * BLOCK]
            rows = rows[rows >= 0]
            if e < 0:
                assert rows.numel() == 0
            else:
                assert (plan.recv_expert[rows] == e).all()
        assert lay.counts.sum().item() == recv.shape[0]
        # return path: "output" of a slot = (token, source, expert) of the row placed there
        out_slots = torch.full((lay.m_cap, 3), -1, dtype=torch.int64)
        out_slots[src >= 0] = recv[src[src >= 0]]
        back = out_slots[lay.slot_of_row.long()].contiguous()
        ret = torch.empty((T * K, 3), dtype=torch.int64)
        dist.all_to_all_single(ret, back, plan.send_splits, plan.recv_splits)
        got = ret[plan.copy_pos.long()]                       # [T, K, 3]
        assert (got[:, :, 0] == torch.arange(T)[:, None]).all()
        assert (got[:, :, 1] == rank).all()
        assert (got[:, :, 2] == idx.long()).all()
        results[rank] = "ok"
    except Exception as ex:  # surfaces in the parent
        results[rank] = repr(ex)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_plan_two_ranks_over_gloo():
    world, T, E, K = 2, 40, 8, 3
    mgr = mp.Manager()
    results = mgr.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_ep_worker, args=(r, world, port, T, E, K, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert dict(results) == {0: "ok", 1: "ok"}


@pytest.mark.parametrize("world,chunks", [(2, 1), (3, 2), (4, 3)])
def test_peer_step_tables_route_every_copy_home(world, chunks):
    """Plays one expert-parallel step over peer memory on the host: the copy list moves row ids
    into the owners' receive areas, the padded layout and the row-address arithmetic of
    dg_moe_return_ptrs (restated here) send every result row back, and every rank must find copy
    (token, j) at the position its combine step reads."""
    from deepgemm.moe import peer_step_tables
    rng = np.random.default_rng(world * 10 + chunks)
    e_local, topk, tokens = 2, 2, 37
    experts = world * e_local
    idx = np.stack([np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]) for _ in range(world)])  # [rank, T, k]
    bounds = [tokens * c // chunks for c in range(chunks + 1)]
    full = np.zeros((world, chunks, world, e_local), dtype=np.int64)
    sorted_ids, pos_of_copy = {}, {}
    for r in range(world):
        for c in range(chunks):
            flat = idx[r, bounds[c]:bounds[c + 1]].reshape(-1)
            order = np.argsort(flat, kind="stable")
            sorted_ids[r, c] = [(r, bounds[c] + int(o) // topk, int(o) % topk) for o in order]
            pos = np.empty_like(order)
            pos[order] = np.arange(order.size)
            pos_of_copy[r, c] = pos.reshape(-1, topk)
            full[r, c] = np.bincount(flat, minlength=experts).reshape(world, e_local)
    tot = full.sum(-1)
    tables = [peer_step_tables(tot, me) for me in range(world)]
    cap = int(tot.sum(0).max())
    recv = {(d, c): [None] * cap for d in range(world) for c in range(chunks)}
    for me in range(world):
        for c in range(chunks):
            seen = set()
            for dst, src_off, dst_off, n in tables[me][3][c]:
                seen.add(dst)
                for i in range(n):
                    assert recv[dst, c][dst_off + i] is None
                    recv[dst, c][dst_off + i] = sorted_ids[me, c][src_off + i]
            assert seen == set(range(world))
    ret = {r: [None] * int(tot[r].sum()) for r in range(world)}
    for d in range(world):
        seg, row0, chunk_base, _ = tables[d]
        for c in range(chunks):
            r_rows = int(tot[:, c, d].sum())
            assert seg[c, world] == r_rows and all(v is not None for v in recv[d, c][:r_rows])
            recv_expert = np.repeat(np.tile(np.arange(e_local), world), full[:, c, d, :].reshape(-1))
            for i in range(r_rows):
                src, t, j = recv[d, c][i]
                assert idx[src, t, j] == d * e_local + recv_expert[i]
            lay = build_contiguous_layout(torch.from_numpy(recv_expert), e_local, contiguous_capacity(r_rows, e_local))
            for s, i in enumerate(lay.src_row.tolist()):
                if i < 0:
                    continue
                r = 0
                while r + 1 < world and i >= seg[c, r + 1]:
                    r += 1
                row = int(row0[c, r]) + i - int(seg[c, r])
                assert ret[r][row] is None
                ret[r][row] = recv[d, c][i]
    for r in range(world):
        chunk_base = tables[r][2]
        for c in range(chunks):
            for t in range(bounds[c], bounds[c + 1]):
                for j in range(topk):
                    assert ret[r][int(chunk_base[r, c]) + int(pos_of_copy[r, c][t - bounds[c], j])] == (r, t, j)
