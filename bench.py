#!/usr/bin/env python
"""Benchmark of the block-scaled GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Headline workload (every N): the grouped-MoE prefill step of the benchmark configuration --
256 experts, top-8 routing, 16384 tokens per GPU, hidden K = 7168, gate+up N = 4096, FP8 E4M3
with UE8M0 scales at granularity 128.  Experts are sharded over the N GPUs (256/N each, weights
resident); one step = routing plan -> dispatch (all-to-all over NCCL when N > 1) -> 128-row
padded contiguous layout -> m_grouped_fp8_gemm_nt_contiguous -> return all-to-all -> top-k
combine.  `value` = valid-row FLOPs of all ranks / max-over-ranks device time (TFLOPS, weak
scaling: per-GPU work is fixed).  At N = 1 the same line carries, under "extra", the dense FP8 /
FP4 GEMMs, the masked grouped GEMM, mqa_logits and quant_mx of the other configurations.

`--impl reference` times the reference's CPU golden model of the same path (the C
restatement under oracle/, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "deepgemm-rs_b200"))

CFG = dict(num_experts=256, topk=8, tokens_per_gpu=16384, hidden=7168, n_out=4096, gran=128)
METRIC = "grouped-MoE FP8 GEMM throughput (m_grouped_fp8_gemm_nt_contiguous, expert-parallel)"
NOMINAL_FP8_TFLOPS = 4500.0


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows, reasons = [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                rows.append((float(f[1]), float(f[2]), float(f[3])))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # the sampler also sees the moments before and after the timed steps: the clock under load is
        # the median over the samples that draw at least 60 % of the highest power seen
        top = max((r[2] for r in rows), default=0.0)
        loaded = sorted(r[0] for r in rows if r[2] >= 0.6 * top)
        return {"sm_mhz": loaded[len(loaded) // 2] if loaded else None, "sm_max_mhz": max((r[1] for r in rows), default=None),
                "reasons": sorted(reasons), "samples": len(rows), "samples_under_load": len(loaded),
                "power_w_max": top or None}


# ------------------------------------------------------------------------------ reference arm
def cpu_gemm_sample(rows, cols, k, seed=0):
    """Times the oracle's gemm_ref (quantised inputs prepared outside the timed region) on a
    rows x cols x k sample of the grouped workload; returns (TFLOPS, seconds, threads).  The OpenMP
    thread count is set to the host's cores explicitly: launchers such as torch.distributed.run
    export OMP_NUM_THREADS=1, and the CPU arm must run alike under every launch."""
    import numpy as np
    import oracle as o
    threads = o.set_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    xa = rng.standard_normal((rows, k)).astype(np.float32)
    xb = rng.standard_normal((cols, k)).astype(np.float32)
    qa, sa = o.quant_mx_host(xa, o.FP8, 128)
    qb, sb = o.quant_fp8_block128_host(xb) if cols % 128 == 0 else o.quant_mx_host(xb, o.FP8, 128)
    a, b = o.GoldenOperand(qa, sa, o.FP8, 128, k), o.GoldenOperand(qb, sb, o.FP8, 128, k)
    t0 = time.perf_counter()
    o.gemm_ref(a, b, m=rows, n=cols)
    dt = time.perf_counter() - t0
    return 2.0 * rows * cols * k / dt / 1e12, dt, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows, cols, k = 512, 512, CFG["hidden"]
    for _ in range(args.warmup):
        cpu_gemm_sample(rows, cols, k)
    # only the gemm_ref calls count: re-time them precisely
    samples = [cpu_gemm_sample(rows, cols, k, seed=s) for s in range(args.steps)]
    times, threads = [t[1] for t in samples], samples[0][2]
    dt = sum(times) / len(times)
    val = 2.0 * rows * cols * k / dt / 1e12
    sample = f"{rows} token rows x {cols} weight rows x K={k} of one expert (gemm_ref, f64 accumulation), per step"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (f64 accumulate on CPU)", "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(n):
    c = dict(CFG)
    return {"workload": "moe_prefill_m_grouped_fp8_gemm_nt_contiguous", "experts": c["num_experts"], "topk": c["topk"],
            "tokens_per_gpu": c["tokens_per_gpu"], "hidden_k": c["hidden"], "n": c["n_out"], "sf_granularity": c["gran"],
            "experts_per_gpu": c["num_experts"] // n, "parallelism": f"ep{n}",
            "l2": "inputs (>= 1 GB of weights touched per step) exceed the 126 MB L2; no flush needed"}


# ------------------------------------------------------------------------------ parity of what is timed
PARITY_TOL = {"fp8": 1e-3, "fp4": 2e-3}
PARITY_MAX_ERR = 0.05      # largest element error allowed, in units of the sample's RMS


def parity_ok(par, kind="fp8"):
    return par is not None and par["calc_diff"] <= PARITY_TOL[kind] and par["max_err"] <= PARITY_MAX_ERR


def parity_moe_step(torch, synth, out, x8, x_sf, topk_idx, topk_w, e_local, n_out, k, seed_of_rank, tokens=8, cols=256):
    """Checks the output of one whole step (dispatch, grouped GEMM, return, combine; every GPU's share of it)
    for a sample of this rank's tokens: for each of their top-k experts the oracle multiplies the token's
    codes by the expert's weights, regenerated here from the owner rank's seed, rounds to bf16 like the GEMM,
    and the copies are combined in f32 in top-k order like dg_moe_combine."""
    import numpy as np
    import oracle as o
    from oracle import sampled
    T = x8.shape[0]
    ts = sampled.pick(T, tokens, 21, [0, T - 1])
    cs = sampled.pick(n_out, cols, 22, sampled.edges(n_out, 224))
    ci = torch.as_tensor(cs, device=x8.device)
    idx = topk_idx[torch.as_tensor(ts, device=x8.device)].cpu().numpy()
    tw = topk_w[torch.as_tensor(ts, device=x8.device)].cpu().numpy().astype(np.float32)
    want = np.zeros((len(ts), len(cs)), dtype=np.float32)
    for i, t in enumerate(ts):
        ga = sampled.golden_rows(x8, x_sf.buf, [int(t)], o.FP8, 128, k)
        acc = np.zeros(len(cs), dtype=np.float32)
        for j, g in enumerate(idx[i]):
            codes, words = synth.expert_weight(seed_of_rank(int(g) // e_local), int(g) % e_local, n_out, k, x8.device)
            gb = sampled.golden_rows(codes, words, cs, o.FP8, 128, k)
            y = o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(o.gemm_ref(ga, gb, m=1, n=len(cs))))[0]
            acc = acc + np.float32(tw[i, j]) * y
        want[i] = acc
    got = out[torch.as_tensor(ts, device=x8.device)][:, ci].float().cpu().numpy()
    d, e = sampled.compare(got, want)
    return {"calc_diff": d, "max_err": e, "sample": f"{len(ts)} tokens x {len(cs)} output columns x top-{idx.shape[1]} experts at full K"}


def parity_ffn_layer(torch, out, x8, x_sf, w13, w2, idx, tw, inter, hidden, tokens=4, cols=256):
    """Checks the output of the whole feed-forward layer for a sample of tokens and output columns: for each of a
    token's experts the oracle runs the gate/up GEMM row at full K, rounds to bf16, applies its SwiGLU and the
    FP8 re-quantisation, multiplies by the sampled rows of the down projection, rounds to bf16, and the copies are
    combined in f32 in top-k order."""
    import numpy as np
    import oracle as o
    from oracle import sampled
    T = x8.shape[0]
    ts = sampled.pick(T, tokens, 31, [0, T - 1])
    cs = sampled.pick(hidden, cols, 32, sampled.edges(hidden, 208))
    ti = torch.as_tensor(ts, device=x8.device)
    ex = idx[ti].cpu().numpy()
    wt = tw[ti].cpu().numpy().astype(np.float32)
    want = np.zeros((len(ts), len(cs)), dtype=np.float32)
    for i, t in enumerate(ts):
        ga = sampled.golden_rows(x8, x_sf.buf, [int(t)], o.FP8, 128, hidden)
        acc = np.zeros(len(cs), dtype=np.float32)
        for j, e in enumerate(ex[i]):
            g13 = sampled.golden_rows(w13.data, w13.sf.buf, np.arange(2 * inter), o.FP8, 128, hidden, row_offset=int(e) * 2 * inter)
            up = o.f32_to_bf16_bits_np(o.gemm_ref(ga, g13, m=1, n=2 * inter))
            hd, hsf = o.quant_mx_host(o.swiglu_f32(up, inter), o.FP8, 128)
            g2 = sampled.golden_rows(w2.data, w2.sf.buf, cs, o.FP8, 128, inter, row_offset=int(e) * hidden)
            y = o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(o.gemm_ref(o.GoldenOperand(hd, hsf, o.FP8, 128, inter), g2, m=1, n=len(cs))))[0]
            acc = acc + np.float32(wt[i, j]) * y
        want[i] = acc
    got = out[ti][:, torch.as_tensor(cs, device=x8.device)].float().cpu().numpy()
    d, e = sampled.compare(got, want)
    return {"calc_diff": d, "max_err": e,
            "sample": f"{len(ts)} tokens x {len(cs)} output columns x top-{ex.shape[1]} experts, both GEMMs at full K"}


def ep_check(torch, dist, moe, synth, group, rank, world, dev):
    """Before the timed steps at N > 1: a small expert-parallel case in which every rank also holds all the
    experts and runs the single-GPU step on its own tokens; the expert-parallel output must equal it bit
    for bit (same weights, same combination order), over two steps through the reused buffers."""
    from deepgemm import Dtype, Operand, SfGran, SfTensor, quant_mx
    E, topk, T, K, N = 4 * world, 2, 256, 512, 256
    full = synth.random_expert_weights(E, N, K, seed=70, device=dev)
    e_local = E // world
    rows = slice(rank * e_local * N, (rank + 1) * e_local * N)
    local = Operand.k_major(Dtype.Fp8, N, K, K, SfTensor(full.sf.rows, e_local * N, SfGran.G128, full.sf.buf[:, rows].contiguous()),
                            full.data[rows].contiguous())
    ep = moe.ExpertParallelMoE(local, E, group)
    single = moe.ExpertParallelMoE(full, E, None)
    same = True
    for step in range(2):
        g = torch.Generator(device=dev).manual_seed(50 + rank + 100 * step)
        x8, x_sf = quant_mx(torch.randn((T, K), device=dev, generator=g), T, K, Dtype.Fp8, 128)
        idx, w = synth.random_topk_routing(T, E, topk, seed=60 + rank + 100 * step, device=dev)
        same = same and torch.equal(ep.forward(x8, x_sf, idx, w), single.forward(x8, x_sf, idx, w))
    ep.close()
    flag = torch.tensor([1 if same else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return "bit-identical" if flag.item() == 1 else "MISMATCH"


# ------------------------------------------------------------------------------ our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the additional single-GPU workloads")
    ap.add_argument("--tokens", type=int, default=CFG["tokens_per_gpu"], help="tokens per GPU (smaller cases for profiling)")
    ap.add_argument("--experts", type=int, default=CFG["num_experts"], help="total experts (smaller cases for profiling)")
    ap.add_argument("--only", default=None, help="run only the extra single-GPU workloads whose name starts with this "
                                                 "(e.g. mqa_logits, fp4_gemm_nt_M4096, quant_mx_fp8_g32) and print them; for profiling")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    CFG["tokens_per_gpu"] = args.tokens
    CFG["num_experts"] = args.experts

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    import deepgemm as dg
    from deepgemm import moe, synth, _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)
    dg.device_check()
    peaks, peak_kind = load_peaks()
    if args.only:
        print(json.dumps({"only": args.only, "results": extra_workloads(torch, dg, synth, dev, peaks, only=args.only)}))
        return

    E, topk, T, K, N = CFG["num_experts"], CFG["topk"], CFG["tokens_per_gpu"], CFG["hidden"], CFG["n_out"]
    e_local = E // world
    ep_verdict = ep_check(torch, dist, moe, synth, group, rank, world, dev) if world > 1 else None
    weights = synth.random_expert_weights(e_local, N, K, seed=1000 + rank, device=dev)
    layer = moe.ExpertParallelMoE(weights, E, group)
    gx = torch.Generator(device=dev).manual_seed(rank)
    x_host = torch.empty((T, K), dtype=torch.float32).pin_memory()
    x_dev = torch.randn((T, K), device=dev, generator=gx)
    x_host.copy_(x_dev)
    topk_idx, topk_w = synth.random_topk_routing(T, E, topk, seed=7 + rank, device=dev)
    idx_host = topk_idx.cpu().pin_memory()
    w_host = topk_w.cpu().pin_memory()
    x8, x_sf = synth.quantised_tokens(x_dev)

    gemm_events = []
    gemm_names = ("m_grouped_gemm_nt_contiguous", "m_grouped_gemm_nt_contiguous_gather", "m_grouped_gemm_nt_contiguous_scatter",
                  "m_grouped_gemm_nt_contiguous_rowptr")
    orig_gemms = {n: getattr(moe, n) for n in gemm_names}

    def timed_variant(fn):
        def wrapped(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(*a, **kw)
            e1.record()
            gemm_events.append((e0, e1))
        return wrapped

    def step_resident():
        return layer.forward(x8, x_sf, topk_idx, topk_w)

    # End to end: every step copies its inputs from pinned host memory and its result back.  The
    # three legs run on three streams over two sets of buffers, so the upload of step i overlaps
    # the compute of step i-1 and the download of step i-2, the way a caller streaming batches
    # through the layer would do it; every step still moves all of its bytes inside the timed region.
    e2e_streams = [torch.cuda.Stream() for _ in range(3)]
    e2e_bufs = [dict(x=torch.empty((T, K), dtype=torch.float32, device=dev), idx=torch.empty_like(topk_idx),
                     w=torch.empty_like(topk_w), out_host=torch.empty((T, N), dtype=torch.bfloat16).pin_memory(),
                     consumed=None, downloaded=None) for _ in range(2)]

    def run_e2e(steps):
        s_in, s_cmp, s_out = e2e_streams
        cur = torch.cuda.current_stream()
        for st in e2e_streams:
            st.wait_stream(cur)
        for i in range(steps):
            b = e2e_bufs[i % 2]
            with torch.cuda.stream(s_in):
                if b["consumed"] is not None:
                    s_in.wait_event(b["consumed"])          # the step that last read this set has quantised its tokens
                b["x"].copy_(x_host, non_blocking=True)
                b["idx"].copy_(idx_host, non_blocking=True)
                b["w"].copy_(w_host, non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(uploaded)
                c, sf = synth.quantised_tokens(b["x"])
                out = layer.forward(c, sf, b["idx"], b["w"])
                b["consumed"] = torch.cuda.Event()
                b["consumed"].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(b["consumed"])
                out.record_stream(s_out)
                b["out_host"].copy_(out, non_blocking=True)
        for st in e2e_streams:
            cur.wait_stream(st)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, profile=False):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0 = _lib.launch_count()
        if profile:
            torch.cuda.profiler.start()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        if profile:
            torch.cuda.profiler.stop()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps, (_lib.launch_count() - c0)

    # valid rows of all ranks = tokens * topk per rank (every copy is computed exactly once)
    flops_per_step = 2.0 * T * topk * N * K * world

    sampler = ClockSampler(local)
    for n in gemm_names:
        setattr(moe, n, timed_variant(orig_gemms[n]))
    if rank == 0:
        sampler.start()
    # `ncu --profile-from-start off` sees exactly the timed steps (a no-op without a profiler)
    ms_step, launches = timed(step_resident, args.steps, args.warmup, profile=True)
    clocks = sampler.stop() if rank == 0 else None
    dg.poll_device_status()
    per_step = len(gemm_events) // (args.steps + args.warmup)       # GEMM launches per step (pipeline slices)
    ev = gemm_events[-args.steps * per_step:]
    gemm_ms = sum(a.elapsed_time(b) for a, b in ev) / args.steps    # all slices of one step
    for n in gemm_names:
        setattr(moe, n, orig_gemms[n])
    e2e_steps = max(4, min(args.steps, 8))
    run_e2e(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_e2e(e2e_steps)
    e1.record()
    barrier()
    ms_t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_e2e = ms_t.item() / e2e_steps

    # parity of what was timed: one more resident step, sampled tokens of rank 0 against the oracle
    parity = None
    if rank == 0 or world > 1:
        out_check = step_resident()
        dg.poll_device_status()
        if rank == 0:
            parity = parity_moe_step(torch, synth, out_check, x8, x_sf, topk_idx, topk_w, e_local, N, K, lambda r: 1000 + r)
        del out_check
    value = flops_per_step / (ms_step * 1e-3) / 1e12
    e2e_value = flops_per_step / (ms_e2e * 1e-3) / 1e12
    gemm_tflops = 2.0 * T * topk * N * K / (gemm_ms * 1e-3) / 1e12       # this rank's launch
    # the timed region lasts a fraction of a second at boost clocks: the burst figure is the denominator
    # (the sustained one was measured over seconds under the power cap)
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    h2d_bytes = x_host.numel() * 4 + idx_host.numel() * 4 + w_host.numel() * 4
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic", "config": dict(workload_config(world), **({"transport": layer.transport,
                                                                         "expert_slices": len(layer._slice_bounds()) - 1}
                                                                        if world > 1 else {})),
        "e2e": {"value": e2e_value, "unit": "TFLOPS", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": T * N * 2,
                # every rank uploads its own tokens: bytes of one rank over the step time all ranks share
                "h2d_gbs_per_rank": h2d_bytes / (ms_e2e * 1e-3) / 1e9,
                "steps": e2e_steps,
                "path": "pinned host f32 tokens -> quant_mx -> expert-parallel grouped GEMM -> combine -> pinned host bf16; "
                        "upload, compute and download of consecutive steps overlap on three streams"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "gemm_kernel<fp8, contiguous>", "achieved": gemm_tflops, "peak": fp8_peak,
                     "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                     # ncu DRAM traffic of one full-size launch (256 experts, 16384 tokens): 8.679 GB read + 1.197 GB written
                     "traffic": 9.876e9 * (T / 16384.0) if CFG["num_experts"] == 256 and world == 1 else None,
                     "traffic_source": "profiles/gemm_fp8_grouped_contiguous__moe_prefill.md",
                     "algorithmic_bytes_per_launch": float(T * topk * 1.125 * K + e_local * N * K + T * topk * 1.125 * N * 2),
                     "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({peak_kind}); FP8 runs at twice the bf16 rate; "
                                    "the timed region is shorter than a second",
                     "frac_of_nominal_4500": gemm_tflops / NOMINAL_FP8_TFLOPS, "launch_ms": gemm_ms,
                     "algorithmic_flops_per_launch": 2.0 * T * topk * N * K},
    }
    if rank == 0:
        line["parity"] = parity
        if not parity_ok(parity):
            # a step whose sampled outputs disagree with the oracle has no throughput to report
            line["error"] = "parity check failed"
            line["value"], line["e2e"]["value"], line["roofline"]["achieved"], line["roofline"]["frac"] = None, None, None, None
        if world > 1:
            line["ep_check"] = ep_verdict
            if ep_verdict != "bit-identical":
                line["error"] = "expert-parallel check failed"
                line["value"], line["e2e"]["value"] = None, None
    if rank == 0 and world == 1:
        v, dt, cores = cpu_gemm_sample(1024, 1024, K)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOPS", "cores": cores, "kind": "port", "seconds": dt,
                                "sample": f"1024 token rows x 1024 weight rows x K={K} of one expert through the oracle's gemm_ref"}
        if not args.no_extra:
            try:
                line["extra"] = extra_workloads(torch, dg, synth, dev, peaks)
            except Exception as ex:  # the headline number stands on its own
                line["extra"] = {"error": repr(ex)}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def extra_workloads(torch, dg, synth, dev, peaks, only=None):
    """Single-GPU numbers of the other benchmark configurations (CUDA events, >= 3 warm-ups,
    inputs larger than L2 or rotated)."""
    from deepgemm import Dtype, Operand, Output

    def timeit(fn, iters=10, warm=3):
        """Device time per call between CUDA events after `warm` warm-up calls.  Calls that take
        less than 0.1 ms are re-timed as a CUDA graph of `iters` calls replayed 5 times: their
        host launch cost exceeds their GPU time, and it is the GPU time that is reported.
        Every workload starts from an idle GPU (0.3 s pause): these are kernels timed alone against burst
        peaks, and without the pause a workload inherits the clocks the one before it was throttled to."""
        torch.cuda.synchronize()
        time.sleep(0.3)
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if ms >= 0.1:
            return ms
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=s):
                for _ in range(iters):
                    fn()
        gr.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * iters)

    g = torch.Generator(device=dev).manual_seed(0)
    res = {}
    import numpy as np
    import oracle as o
    from oracle import sampled

    def want(name):
        return only is None or name.startswith(only)

    def gated(entry, kind="fp8"):
        """A workload whose sampled outputs disagree with the oracle reports its parity figures and no throughput."""
        if parity_ok(entry.get("parity"), kind):
            return entry
        return {"parity": entry.get("parity"), "error": "parity check failed"}

    def dense(kind, m, n, k):
        if kind == "fp8":
            da, sa = dg.quant_mx(torch.randn((m, k), device=dev, generator=g), m, k, Dtype.Fp8, 128)
            wb = torch.randn((-(-n // 128) * 128, k), device=dev, generator=g)
            cb, sb = synth.block128_quant_fp8(wb) if k % 512 == 0 else (None, None)
            if cb is None:
                cb, sfb = dg.quant_mx(wb[:n], n, k, Dtype.Fp8, 128)
            else:
                from deepgemm import SfGran, SfTensor
                sfb = SfTensor(k // 512, wb.shape[0], SfGran.G128, sb)
            a, b = Operand.k_major(Dtype.Fp8, m, k, k, sa, da), Operand.k_major(Dtype.Fp8, n, k, k, sfb, cb)
            peak = 2 * peaks["bf16_tflops"]
        else:
            da, sa = dg.quant_mx(torch.randn((m, k), device=dev, generator=g), m, k, Dtype.Fp4, 32)
            db, sb = dg.quant_mx(torch.randn((n, k), device=dev, generator=g), n, k, Dtype.Fp4, 32)
            a, b = Operand.k_major(Dtype.Fp4, m, k, k, sa, da), Operand.k_major(Dtype.Fp4, n, k, k, sb, db)
            peak = 4 * peaks["bf16_tflops"]
        out = Output(Dtype.Bf16, m, n, n, torch.empty((m, n), dtype=torch.bfloat16, device=dev))
        # A weight-streaming shape (M = 128) re-reads its weights on every call: consecutive calls take copies of B in
        # turn, enough of them to exceed the 126 MB L2, so that every call streams its weights from HBM.
        bs = [b]
        if m <= 128:
            per = n * k * (1 if kind == "fp8" else 0.5)
            for _ in range(int(-(-300e6 // per)) - 1):
                bs.append(Operand.k_major(b.dtype, n, k, k, type(b.sf)(b.sf.rows, b.sf.cols, b.sf.gran, b.sf.buf.clone()), b.data.clone()))
        turn = [0]

        def call():
            dg.gemm_nt(a, bs[turn[0] % len(bs)], out)
            turn[0] += 1
        ms = timeit(call, iters=max(10, len(bs)))
        b = bs[(turn[0] - 1) % len(bs)]          # the operand of the last call: the parity check below reads its output
        tf = 2.0 * m * n * k / ms / 1e9
        byts = (m * k + n * k) * (1 if kind == "fp8" else 0.5) + m * n * 2
        # the output of the last timed call, sampled: 128 rows x 256 columns over the full K against gemm_ref
        odt, gran = (o.FP8, 128) if kind == "fp8" else (o.FP4, 32)
        cfg = dg.get_gemm_config(Dtype.Fp8 if kind == "fp8" else Dtype.Fp4, 0, m, n, k)
        rows = sampled.pick(m, 128, 31, sampled.edges(m, cfg["block_m"]))
        cols = sampled.pick(n, 256, 32, sampled.edges(n, cfg["block_n"]))
        par = sampled.check_gemm_sample(a.data, a.sf.buf, b.data, b.sf.buf, out.data, rows, cols, odt, gran, odt, b.sf.gran.k(), k)
        return gated({"ms": ms, "tflops": tf, "frac_of_measured_tensor_peak": tf / peak, "hbm_gbs": byts / ms / 1e6,
                      "frac_of_measured_hbm": byts / ms / 1e6 / peaks["hbm_gbs"],
                      "tile": f"{cfg['block_m']}x{cfg['block_n']}", "parity": par,
                      **({"l2": f"{len(bs)} copies of B in turn ({len(bs) * n * k / 1e6:.0f} MB > L2)"} if len(bs) > 1 else {})}, kind)

    for m in (128, 4096):
        for n, k in ((24576, 1536), (7168, 16384), (4096, 7168)):
            if want(f"fp8_gemm_nt_M{m}_N{n}_K{k}"):
                res[f"fp8_gemm_nt_M{m}_N{n}_K{k}"] = dense("fp8", m, n, k)
    if want("fp4_gemm_nt_M8192_N8192_K8192"):
        res["fp4_gemm_nt_M8192_N8192_K8192"] = dense("fp4", 8192, 8192, 8192)
    if want("fp4_gemm_nt_M4096_N7168_K7168"):
        res["fp4_gemm_nt_M4096_N7168_K7168"] = dense("fp4", 4096, 7168, 7168)

    # masked decode: 32 experts, expected_m 128, masked_m uniform in [0, 256]
    if want("m_grouped_fp8_gemm_nt_masked_G32"):
        G, max_m, n, k = 32, 256, 4096, 7168
        w = synth.random_expert_weights(G, n, k, seed=5, device=dev)
        da, sa = dg.quant_mx(torch.randn((G * max_m, k), device=dev, generator=g), G * max_m, k, Dtype.Fp8, 128)
        a = Operand.k_major(Dtype.Fp8, max_m, k, k, sa, da)
        masked = torch.randint(0, 257, (G,), device=dev, generator=g, dtype=torch.int32)
        out = Output(Dtype.Bf16, max_m, n, n, torch.empty((G * max_m, n), dtype=torch.bfloat16, device=dev))
        ms = timeit(lambda: dg.m_grouped_fp8_gemm_nt_masked(a, w, out, masked, G, 128))
        sm = int(masked.sum().item())
        byts = sm * k + G * n * k + sm * n * 2
        mm = masked.cpu().numpy()
        cols = sampled.pick(n, 256, 33, sampled.edges(n, 224))
        worst = {"calc_diff": 0.0, "max_err": 0.0}
        for gi in [int(x) for x in np.nonzero(mm > 0)[0][[0, len(np.nonzero(mm > 0)[0]) // 2, -1]]]:
            rows = gi * max_m + sampled.pick(int(mm[gi]), 24, gi, [0, int(mm[gi]) - 1, 127, 128])
            par = sampled.check_gemm_sample(da, sa.buf, w.data, w.sf.buf, out.data, rows, cols, o.FP8, 128, o.FP8, 128, k, b_row_offset=gi * n)
            worst = {key: max(worst[key], par[key]) for key in worst}
        res["m_grouped_fp8_gemm_nt_masked_G32"] = gated({"ms": ms, "sum_masked_m": sm, "tflops": 2.0 * sm * n * k / ms / 1e9,
                                                         "hbm_gbs": byts / ms / 1e6,
                                                         "frac_of_measured_hbm": byts / ms / 1e6 / peaks["hbm_gbs"], "parity": worst})

    # whole MoE feed-forward layer (gate/up GEMM -> SwiGLU + FP8 re-quantisation -> down GEMM -> combine),
    # 256 experts, top-8, 16384 tokens, hidden 7168, intermediate 2048: the layer around the headline GEMM
    if want("moe_ffn_layer_T16384_E256_top8_H7168_I2048"):
        from deepgemm import moe
        E, topk, T, H, I = 256, 8, 16384, 7168, 2048
        w13 = synth.random_expert_weights(E, 2 * I, H, seed=11, device=dev)
        w2 = synth.random_expert_weights(E, H, I, seed=12, device=dev)
        x8, x_sf = synth.quantised_tokens(torch.randn((T, H), device=dev, generator=g))
        idx, tw = synth.random_topk_routing(T, E, topk, seed=13, device=dev)
        layer = moe.GroupedMoEFfn(w13, w2, E)
        ms = timeit(lambda: layer.forward(x8, x_sf, idx, tw), iters=5, warm=2)
        flops = 2.0 * T * topk * (2 * I * H + H * I)
        out = layer.forward(x8, x_sf, idx, tw)
        dg.poll_device_status()
        res["moe_ffn_layer_T16384_E256_top8_H7168_I2048"] = gated(
            {"ms": ms, "tflops": flops / ms / 1e9,
             "frac_of_measured_tensor_peak": flops / ms / 1e9 / (2 * peaks["bf16_tflops_sustained"]),
             "parity": parity_ffn_layer(torch, out, x8, x_sf, w13, w2, idx, tw, I, H)})
        del layer, w13, w2, out
        torch.cuda.empty_cache()

    # mqa_logits, fp32 contract
    if want("mqa_logits_T4096_S32768_H64_D128"):
        T, S, H, D = 4096, 32768, 64, 128
        q = torch.randn((T, H, D), device=dev, generator=g).to(torch.float8_e4m3fn).view(torch.uint8)
        kvf = torch.randn((S, D), device=dev, generator=g)
        scale = kvf.abs().amax(dim=1) / 448.0
        kv = (kvf / scale[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
        wq = torch.randn((T, H), device=dev, generator=g)
        ks = torch.zeros(T, dtype=torch.int32, device=dev)
        ke = (S - T + torch.arange(T, device=dev) + 1).to(torch.int32)
        logits = torch.empty((T, S), dtype=torch.float32, device=dev)
        ms = timeit(lambda: dg.mqa_logits_f32(q, kv, scale, wq, ks, ke, T, S, H, D, logits, S), iters=5)
        pairs = int(ke.sum().item())
        tf = 2.0 * H * D * pairs / ms / 1e9
        qs = sampled.pick(T, 32, 34, [0, 1, T - 1, 2047, 2048])
        ends = S - T + qs + 1
        js = sampled.pick(S, 2048, 35, [0, 127, 128, S - 1] + [int(e) - 1 for e in ends])
        qi, ji = torch.as_tensor(qs, device=dev), torch.as_tensor(js, device=dev)
        ref = o.mqa_logits_ref(q.view(torch.float8_e4m3fn)[qi].float().cpu().numpy(),
                               (kv.view(torch.float8_e4m3fn)[ji].float() * scale[ji][:, None]).cpu().numpy(), wq[qi].cpu().numpy(),
                               np.zeros(len(qs), np.uint32), np.full(len(qs), len(js), np.uint32))
        got = logits[qi][:, ji].cpu().numpy()
        valid = js[None, :] < ends[:, None]
        dq, eq = sampled.compare(got[valid], ref[valid], out_is_bf16=False)
        res["mqa_logits_T4096_S32768_H64_D128"] = gated({"ms": ms, "tflops": tf,
                                                         "frac_of_measured_tensor_peak": tf / (2 * peaks["bf16_tflops"]),
                                                         "parity": {"calc_diff": dq, "max_err": eq}})

    # mqa_logits, the reference's own SM100 contract: UE8M0 scales per 32 along head_dim on q and kv, bf16 weights and logits
    if want("mqa_logits_ue8m0_T4096_S32768_H64_D128"):
        from deepgemm import Operand
        T, S, H, D = 4096, 32768, 64, 128
        q8, qsf = dg.quant_mx(torch.randn((T * H, D), device=dev, generator=g), T * H, D, Dtype.Fp8, 32)
        kv8, kvsf = dg.quant_mx(torch.randn((S, D), device=dev, generator=g) * 3.0, S, D, Dtype.Fp8, 32)
        wq = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        ks = torch.zeros(T, dtype=torch.int32, device=dev)
        ke = (S - T + torch.arange(T, device=dev) + 1).to(torch.int32)
        logits = torch.empty((T, S), dtype=torch.bfloat16, device=dev)
        qop = Operand.k_major(Dtype.Fp8, T * H, D, D, qsf, q8)
        kvop = Operand.k_major(Dtype.Fp8, S, D, D, kvsf, kv8)
        ms = timeit(lambda: dg.mqa_logits(qop, kvop, wq, ks, ke, T, S, H, D, logits, S), iters=5)
        pairs = int(ke.sum().item())
        tf = 2.0 * H * D * pairs / ms / 1e9
        qs = sampled.pick(T, 16, 36, [0, 1, T - 1, 2047, 2048])
        ends = S - T + qs + 1
        js = sampled.pick(S, 1024, 37, [0, 127, 128, S - 1] + [int(e) - 1 for e in ends])
        qrows = (np.asarray(qs)[:, None] * H + np.arange(H)[None, :]).reshape(-1)
        qg = sampled.golden_rows(q8, qsf.buf, qrows, o.FP8, 32, D)
        kg = sampled.golden_rows(kv8, kvsf.buf, js, o.FP8, 32, D)
        qd = o.dequant_mx_host(qg.data, qg.sf, len(qrows), D, o.FP8, 32).reshape(len(qs), H, D)
        kd = o.dequant_mx_host(kg.data, kg.sf, len(js), D, o.FP8, 32)
        ref = o.mqa_logits_ref(qd, kd, wq[torch.as_tensor(qs, device=dev)].float().cpu().numpy(),
                               np.zeros(len(qs), np.uint32), np.full(len(qs), len(js), np.uint32))
        got = logits[torch.as_tensor(qs, device=dev)][:, torch.as_tensor(js, device=dev)].float().cpu().numpy()
        valid = js[None, :] < ends[:, None]
        dq, eq = sampled.compare(got[valid], ref[valid], out_is_bf16=True)
        res["mqa_logits_ue8m0_T4096_S32768_H64_D128"] = gated({"ms": ms, "tflops": tf,
                                                               "frac_of_measured_tensor_peak": tf / (2 * peaks["bf16_tflops"]),
                                                               "parity": {"calc_diff": dq, "max_err": eq}})

    # mqa_logits over a paged KV cache (decode): 128 requests of 32768 tokens, two query tokens each, pages of 64 tokens
    if want("mqa_logits_paged_B128_ctx32768_n2_H64_D128"):
        from deepgemm import Operand, mqa_logits_paged
        B, CTX, NN, PAGE, H, D = 128, 32768, 2, 64, 64, 128
        T, pages_per = B * NN, CTX // PAGE
        num_pages = B * pages_per + 3
        q8, qsf = dg.quant_mx(torch.randn((T * H, D), device=dev, generator=g), T * H, D, Dtype.Fp8, 32)
        kv8, kvsf = dg.quant_mx(torch.randn((num_pages * PAGE, D), device=dev, generator=g) * 2.0, num_pages * PAGE, D, Dtype.Fp8, 32)
        kv_words = kvsf.buf[0, :num_pages * PAGE].contiguous()            # head_dim 128: one packed word per token
        wq = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        perm = torch.randperm(num_pages, device=dev, generator=g).to(torch.int32)
        stride = pages_per + 1
        table = torch.full((T, stride), 10 ** 6, dtype=torch.int32, device=dev)       # only a request's first row is read
        table[::NN, :pages_per] = perm[:B * pages_per].view(B, pages_per)
        req = torch.arange(B, device=dev, dtype=torch.int32).repeat_interleave(NN)
        ctx = (CTX - (NN - 1) + torch.arange(NN, device=dev)).repeat(B).to(torch.int32)
        width = CTX + 8
        logits = torch.full((T, width), -7.0, dtype=torch.bfloat16, device=dev)
        qop = Operand.k_major(Dtype.Fp8, T * H, D, D, qsf, q8)
        ms = timeit(lambda: mqa_logits_paged(qop, kv8, kv_words, wq, PAGE, num_pages, ctx, req, table, stride, T, H, D, logits, width), iters=5)
        byts = B * CTX * (D + 4) + T * CTX * 2
        worst = {"calc_diff": 0.0, "max_err": 0.0}
        for b in (0, B // 2, B - 1):                                                   # three whole requests against the oracle
            rows = (table[b * NN, :pages_per].long()[:, None] * PAGE + torch.arange(PAGE, device=dev)[None, :]).reshape(-1)
            kg = sampled.golden_rows(kv8, kvsf.buf, rows.cpu().numpy(), o.FP8, 32, D)
            kd = o.dequant_mx_host(kg.data, kg.sf, CTX, D, o.FP8, 32)
            qrows = np.arange(b * NN * H, (b + 1) * NN * H)
            qg = sampled.golden_rows(q8, qsf.buf, qrows, o.FP8, 32, D)
            qd = o.dequant_mx_host(qg.data, qg.sf, NN * H, D, o.FP8, 32).reshape(NN, H, D)
            ends = ctx[b * NN:(b + 1) * NN].cpu().numpy().astype(np.uint32)
            ref = o.mqa_logits_ref(qd, kd, wq[b * NN:(b + 1) * NN].float().cpu().numpy(), np.zeros(NN, np.uint32), ends)
            got = logits[b * NN:(b + 1) * NN, :CTX].float().cpu().numpy()
            valid = np.arange(CTX)[None, :] < ends[:, None]
            dq, eq = sampled.compare(got[valid], ref[valid], out_is_bf16=True)
            worst = {"calc_diff": max(worst["calc_diff"], dq), "max_err": max(worst["max_err"], eq)}
            if not (got[~valid] == -7.0).all():
                worst["max_err"] = float("inf")                                        # something was written past a context length
        res["mqa_logits_paged_B128_ctx32768_n2_H64_D128"] = gated({"ms": ms, "gbs": byts / ms / 1e6,
                                                                    "frac_of_measured_hbm": byts / ms / 1e6 / peaks["hbm_gbs"],
                                                                    "tflops": 2.0 * H * D * T * CTX / ms / 1e9, "parity": worst})

    # quant_mx bandwidth
    for (m, k, dt, gran, name) in ((16384, 7168, Dtype.Fp8, 128, "fp8_g128"), (16384, 7168, Dtype.Fp8, 32, "fp8_g32"),
                                   (16384, 7168, Dtype.Fp4, 32, "fp4_g32"), (4096, 16384, Dtype.Fp8, 128, "fp8_g128")):
        if not want(f"quant_mx_{name}_{m}x{k}"):
            continue
        x = torch.randn((m, k), device=dev, generator=g)
        ms = timeit(lambda: dg.quant_mx(x, m, k, dt, gran))
        byts = 4 * m * k + (m * k if dt == Dtype.Fp8 else m * k // 2) + 4 * (-(-(k // gran) // 4)) * m
        # bytes of 64 sampled rows (codes and their scale-factor columns) against the oracle's quantiser
        rs = sampled.pick(m, 64, 36, [0, 1, 31, 32, m - 1])
        ri = torch.as_tensor(rs, device=dev)
        codes, sft = dg.quant_mx(x, m, k, dt, gran)
        wc, ws = o.quant_mx_host(x[ri].cpu().numpy(), o.FP8 if dt == Dtype.Fp8 else o.FP4, gran)
        same = bool(np.array_equal(codes[ri].cpu().numpy(), wc) and
                    np.array_equal(sft.buf[:, ri].cpu().numpy().view(np.uint32), ws[:, :len(rs)]))
        entry = {"ms": ms, "gbs": byts / ms / 1e6, "frac_of_measured_hbm": byts / ms / 1e6 / peaks["hbm_gbs"],
                 "parity": "bytes equal on 64 sampled rows" if same else "MISMATCH"}
        res[f"quant_mx_{name}_{m}x{k}"] = entry if same else {"parity": "MISMATCH", "error": "parity check failed"}
    # SwiGLU + FP8 re-quantisation between the two GEMMs of the FFN layer (HBM-bound): 139264 rows
    # (131072 copies + padding) x 2 * 2048 bf16 in, 2048 codes + scale factors out
    if want("swiglu_quant_139264x2048"):
        m, inter = 139264, 2048
        gu = torch.randn((m, 2 * inter), device=dev, generator=g).to(torch.bfloat16)
        ms = timeit(lambda: dg.swiglu_quant(gu, m, inter, 128))
        byts = m * inter * 5 + m * (inter // 128)
        res["swiglu_quant_139264x2048"] = {"ms": ms, "gbs": byts / ms / 1e6, "frac_of_measured_hbm": byts / ms / 1e6 / peaks["hbm_gbs"]}
        del gu
    dg.poll_device_status()
    return res


if __name__ == "__main__":
    main()
