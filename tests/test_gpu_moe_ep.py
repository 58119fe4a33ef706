"""Expert-parallel MoE step on 2 GPUs against the single-GPU step with all experts resident:
identical routing and tokens must give bit-identical outputs, because every copy is multiplied by
the same weights and combined in the same order.  All transports run over repeated steps (the
buffers are reused): "push" (rows stored into the expert owner's layout by a kernel, result rows
stored into the token owner's buffer by the GEMM epilogue, flag barriers, no host synchronisation),
"peer" (copy-engine dispatch with one and two token slices, same return path) and NCCL all-to-alls.
Skipped with fewer than 2 GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

E, TOPK, T, K, N = 8, 2, 200, 512, 256


def _inputs(rank, dev):
    from deepgemm import Dtype, quant_mx, synth
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    x = torch.randn((T, K), device=dev, generator=g)
    x8, x_sf = quant_mx(x, T, K, Dtype.Fp8, 128)
    idx, w = synth.random_topk_routing(T, E, TOPK, seed=60 + rank, device=dev)
    return x8, x_sf, idx, w


def _all_weights(dev):
    from deepgemm import synth
    return synth.random_expert_weights(E, N, K, seed=70, device=dev)


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from deepgemm import Dtype, Operand, SfGran, SfTensor, moe, poll_device_status
        full = _all_weights(dev)
        e_local = E // world
        rows = slice(rank * e_local * N, (rank + 1) * e_local * N)
        local = Operand.k_major(Dtype.Fp8, N, K, K,
                                SfTensor(full.sf.rows, e_local * N, SfGran.G128, full.sf.buf[:, rows].contiguous()),
                                full.data[rows].contiguous())
        x8, x_sf, idx, w = _inputs(rank, dev)
        want = moe.ExpertParallelMoE(full, E, None).forward(x8, x_sf, idx, w)
        x8b, x_sfb, idxb, wb = _inputs(rank + 10, dev)
        wantb = moe.ExpertParallelMoE(full, E, None).forward(x8b, x_sfb, idxb, wb)
        verdicts = []
        for transport, chunks in (("push", 1), ("push", 2), ("peer", 1), ("peer", 2), ("nccl", 1)):
            os.environ["DG_EP_CHUNKS"] = str(chunks)
            layer = moe.ExpertParallelMoE(local, E, dist.group.WORLD, transport=transport)
            for step in range(3):
                xa, sa, ia, wa, ref = (x8, x_sf, idx, w, want) if step != 1 else (x8b, x_sfb, idxb, wb, wantb)
                got = layer.forward(xa, sa, ia, wa)
                poll_device_status()
                if not torch.equal(got, ref):
                    verdicts.append(f"{transport} chunks={chunks} step {step}: max diff {(got.float() - ref.float()).abs().max().item()}")
            layer.close()
        out[rank] = "ok" if not verdicts else "; ".join(verdicts)
    except Exception as ex:
        out[rank] = repr(ex)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_ep_equals_single_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    assert dict(out) == {0: "ok", 1: "ok"}
