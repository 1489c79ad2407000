#!/usr/bin/env python3
"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode|prefill|ep]

Prints ONE JSON line on rank 0.  Workloads (seeded synthetic inputs of the benchmark plan's shapes):
  decode   (default on 1 GPU)  one token through 11 stacked MoE layers (hidden 1280, 64 experts top-6 + shared
           1792, FFN 896, Q4_0 group-64 weights, seed 1); metric = microseconds per token; a step is one pass
           of the token through the 11 layers.  On N > 1 GPUs with --workload decode: N independent replicas.
  prefill  one MoE layer on 4096 tokens, Q4_0, Zipf(1.1)-skewed routing, seed 3; metric = tokens per second.
  ep       (default on N > 1 GPUs)  one MoE layer on 8 x 2048 = 16384 tokens, Q4_0, Zipf(1.1) routing, seed 4, the 64
           experts sharded over the N GPUs with all-to-all dispatch/combine; metric = tokens per second of the
           whole job (fixed total work: strong scaling).  Rank 0 also times the same layer alone (G = 1).

  value  device time per step (CUDA events on the launching stream), inputs resident in HBM;
  e2e    wall time of the host-buffer C-ABI call (host->device copy, 11 layers, device->host copy);
  roofline.achieved  algorithmic bytes per step (11 x 14 786 560 B of weights + activations) / step time;
  cpu_baseline       the reference's CPU layer function (oracle/_ref) on this host's cores, bounded sample.

Between timed iterations a buffer larger than L2 is written so that no step finds its weights cached.
With --impl reference the reference's CPU path alone is timed on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FULL = dict(H=1280, E=64, K=6, F=896, S=1792)
N_LAYERS = 11
SEED_DECODE = 1
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def layer_bytes(qtype_name: str, n_tokens: int = 1, distinct_experts: int = 6) -> int:
    """Algorithmic bytes of one layer step: router + distinct selected experts + shared MLP + activations."""
    H, E, F, S = FULL["H"], FULL["E"], FULL["F"], FULL["S"]
    per = {"f16": lambda r, c: 2 * r * c, "q8_0": lambda r, c: r * c + 2 * r * (c // 64),
           "q4_0": lambda r, c: r * c // 2 + 2 * r * (c // 64)}[qtype_name]
    expert = 2 * per(F, H) + per(H, F)
    shared = 2 * per(S, H) + per(H, S)
    return E * H * 2 + distinct_experts * expert + shared + n_tokens * H * 2 * 3


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(device_index)], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def samples(self) -> int:
        try:
            return sum(1 for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8)
        except OSError:
            return 0

    def hold(self, step, minimum: int = 2, limit_s: float = 4.0) -> None:
        """Keep the same load running (untimed) until nvidia-smi has delivered `minimum` samples: a timed region of a
        few milliseconds is over before its first sample."""
        if self.proc is None:
            return
        import torch
        t0 = time.perf_counter()
        while self.samples() < minimum and time.perf_counter() - t0 < limit_s:
            for _ in range(20):
                step()
            torch.cuda.synchronize()

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def synth_stack(n_layers: int, qtype_name: str, seed: int):
    from oracle import quant
    rng = np.random.default_rng(seed)
    layers = [quant.synth_layer(rng, expert_qtype=quant.QTYPE_BY_NAME[qtype_name], **FULL) for _ in range(n_layers)]
    hidden = quant.synth_activations(np.random.default_rng(seed + 1000), 1, FULL["H"])
    return layers, hidden


def run_reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.host_threads()
    # only the sampled layers are generated (the first ones of the same seeded stack)
    layers, hidden = synth_stack(min(args.cpu_layers, N_LAYERS), "q4_0", SEED_DECODE)
    t0 = time.perf_counter()
    us, kind, sample = _cpu_arm(layers, hidden, args, threads)
    line = {
        "impl": "reference", "metric": "moe_decode_us_per_token", "value": us, "unit": "us/token", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us * threads / 1000.0, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": us, "unit": "us/token", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": us, "unit": "us/token", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def _cpu_arm(sampled_layers, hidden, args, threads):
    from oracle import oracle as orc
    try:
        impl, kind = orc.Ref(), "reference"
    except FileNotFoundError:
        impl, kind = orc.Port(), "port"
    rng = np.random.default_rng(1234)
    extra = rng.standard_normal((max(threads - 1, 0), FULL["H"]), dtype=np.float32).astype("<f2").view(np.uint16)
    tokens = np.concatenate([hidden, extra]) if threads > 1 else hidden
    f32 = [orc.layer_to_f32(L) for L in sampled_layers] if kind == "reference" else None

    def one_pass():
        cur = tokens
        for i, L in enumerate(sampled_layers):
            o = impl.layer(L, cur, cur, threads=threads, f32_weights=f32[i]) if kind == "reference" \
                else impl.layer(L, cur, cur, threads=threads)
            cur = impl.f32_to_f16(o.out)

    for _ in range(min(args.warmup, 1)):
        one_pass()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    done = 0
    while done < steps and (done == 0 or time.perf_counter() - t0 < 60.0):   # bounded: stop after a minute
        one_pass()
        done += 1
    dt = (time.perf_counter() - t0) / done
    us = dt * 1e6 / threads * (N_LAYERS / len(sampled_layers))
    sample = (f"{threads} tokens in parallel (one per host thread) through {len(sampled_layers)} of the {N_LAYERS} "
              f"layers, {done} passes, scaled x{N_LAYERS}/{len(sampled_layers)}; f32 dequantised weights")
    return us, kind, sample


def workload_config() -> dict:
    return {"workload": "decode: 1 token x 11 stacked MoE layers, hidden 1280, 64 experts top-6 + shared 1792, "
                        "FFN 896, Q4_0 group-64 experts and shared MLP, seed 1",
            "layers": N_LAYERS, "tokens_per_step": 1, "qtype": "q4_0",
            "l2": "flushed between timed iterations (256 MiB written, then 256 MiB read)"}


NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
FLOPS_PER_TOKEN = 2 * FULL["E"] * FULL["H"] + FULL["K"] * 3 * 2 * FULL["F"] * FULL["H"] + 3 * 2 * FULL["S"] * FULL["H"]


def measured_tensor_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_BF16_TFLOPS, "fallback"


def token_workload(kind: str) -> dict:
    if kind == "prefill":
        return {"n_tokens": 4096, "seed": 3, "metric": "moe_prefill_tokens_per_s",
                "workload": "prefill: one MoE layer, 4096 tokens, hidden 1280, 64 experts top-6 + shared 1792, FFN 896, "
                            "Q4_0, Zipf(1.1)-skewed routing via logit bias, seed 3"}
    return {"n_tokens": 16384, "seed": 4, "metric": "moe_ep_prefill_tokens_per_s",
            "workload": "expert-parallel prefill: one MoE layer, 8 requests x 2048 = 16384 tokens, Q4_0, 64 experts sharded "
                        "evenly over the GPUs, all-to-all dispatch/combine, Zipf(1.1)-skewed routing, seed 4"}


def synth_token_layer(seed: int, n_tokens: int, qtype_name: str = "q4_0", routing: str = "zipf"):
    from oracle import quant
    rng = np.random.default_rng(seed)
    bias = quant.zipf_logit_bias(rng, FULL["E"])       # drawn in both cases so that the weights do not depend on the choice
    if routing == "uniform":
        bias = None
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_BY_NAME[qtype_name], logit_bias=bias, **FULL)
    hidden = quant.synth_activations(rng, n_tokens, FULL["H"])
    resid = quant.synth_activations(rng, n_tokens, FULL["H"])
    return L, hidden, resid


def cpu_tokens_per_s(L, hidden, resid, threads: int, rows_per_thread: int = 4, max_seconds: float = 40.0):
    """The reference CPU layer function on a seeded subset of the tokens (rows_per_thread per host thread)."""
    from oracle import oracle as orc
    try:
        impl, kind = orc.Ref(), "reference"
    except FileNotFoundError:
        impl, kind = orc.Port(), "port"
    rows = min(hidden.shape[0], threads * rows_per_thread)
    import dataclasses
    sub_h, sub_r = hidden[:rows], resid[:rows]
    if kind == "reference":
        # the unmodified function has no logit bias input: time it on the same weights without the bias
        # (routing differs, cost per token does not)
        plain = dataclasses.replace(L, logit_bias=None)
        f32 = orc.layer_to_f32(plain)
        run = lambda: impl.layer(plain, sub_h, sub_r, threads=threads, f32_weights=f32)
    else:
        run = lambda: impl.layer(L, sub_h, sub_r, threads=threads)
    run()
    t0, done = time.perf_counter(), 0
    while done < 3 and (done == 0 or time.perf_counter() - t0 < max_seconds):
        run()
        done += 1
    dt = (time.perf_counter() - t0) / done
    return rows / dt, kind, (f"{rows} of the {hidden.shape[0]} tokens ({rows_per_thread} per host thread, {threads} threads), "
                             f"{done} passes, f32 dequantised weights; tokens/s extrapolates linearly")


def run_reference_tokens(args, rank: int, kind: str) -> None:
    if rank != 0:
        return
    from oracle import oracle as orc
    w = token_workload(kind)
    threads = orc.host_threads()
    L, hidden, resid = synth_token_layer(w["seed"], 1024)        # the sample never needs more tokens than this
    t0 = time.perf_counter()
    tps, ckind, sample = cpu_tokens_per_s(L, hidden, resid, threads)
    line = {"impl": "reference", "metric": w["metric"], "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": w["n_tokens"] / tps * 1e3, "higher_is_better": True,
            "scaling": "strong" if kind == "ep" else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["workload"], "tokens_per_step": w["n_tokens"], "qtype": "q4_0"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": ckind, "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


def make_flush(torch):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    reader = torch.empty(256 << 20, dtype=torch.uint8, device="cuda").view(torch.int32)

    def flush_l2(i: int):
        # write a buffer larger than L2, then read a second one through the cache so that the weights are
        # cold AND the cache is not left full of dirty lines whose write-back would compete with the step
        flush.fill_(i & 0xFF)
        reader.max()
    return flush_l2


def run_tokens(args, kind: str, rank: int, local_rank: int, world: int) -> None:
    """prefill (one GPU) and expert-parallel prefill (N GPUs): one MoE layer on many tokens."""
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    w = token_workload(kind)
    n_total = w["n_tokens"]
    if n_total % world:
        raise SystemExit(f"{n_total} tokens do not divide over {world} ranks")
    L, hidden, resid = synth_token_layer(w["seed"], n_total, routing=args.routing)
    n_local = n_total // world
    lo = rank * n_local
    stream = torch.cuda.current_stream()
    ctx = pkg.Context()
    ctx.map_layer(L)
    # a rank can receive every pair of the job (worst case), and rank 0 also runs the whole job alone
    ctx.allocate_runtime_arenas(n_total)
    ctx.set_stream(stream.cuda_stream)
    flush_l2 = make_flush(torch)
    h_local = torch.from_numpy(hidden[lo:lo + n_local].copy()).pin_memory()
    r_local = torch.from_numpy(resid[lo:lo + n_local].copy()).pin_memory()
    d_h = h_local.cuda().view(torch.float16)
    d_r = r_local.cuda().view(torch.float16)
    d_out = torch.zeros_like(d_h)
    host_out = torch.empty((n_local, FULL["H"]), dtype=torch.float16).pin_memory()
    # the exchange: fused into the library's kernels over peer memory (default), or NCCL all-to-all between its phases
    exchange, layer = "nccl all_to_all_single", None
    if kind == "ep" and world > 1 and args.exchange == "peer":
        why = ""
        try:
            layer = pkg.ep.PeerExpertParallelLayer(ctx, 0, FULL["E"], FULL["K"], FULL["H"], row_capacity=n_total * FULL["K"],
                                                   rank=rank, world=world, dist_module=dist)
            exchange = "peer memory (CUDA IPC over NVLink), fused into gather and combine"
        except Exception as e:      # e.g. no peer access between the devices: every rank must then take the other path
            why = str(e)[:200]
        ok = torch.tensor([1 if layer is not None else 0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            if layer is not None:
                layer.close(group_barrier=False)      # nothing has run on the exchange buffers yet
            layer = None
            exchange = f"nccl all_to_all_single (peer-memory set-up failed on a rank: {why})"
    if layer is None:
        layer = pkg.ep.ExpertParallelLayer(ctx, 0, FULL["E"], FULL["K"], FULL["H"], rank=rank, world=world,
                                           dist_module=dist if world > 1 else None)
        layer.reserve(n_local, n_total * FULL["K"])

    def step():
        if kind == "prefill":
            ctx.layer_forward(0, d_h, n_local, d_out, residual=d_r)
            return None
        return layer.forward(d_h, d_out, residual=d_r)

    def timed(fn, steps, warmup):
        for i in range(warmup):
            flush_l2(i)
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush_l2(i)
            if world > 1:
                dist.barrier()                     # every rank starts the step together; the barrier is not timed
            starts[i].record(stream)
            fn()
            ends[i].record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in zip(starts, ends)]

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = ctx.kernel_launches
    times = timed(step, args.steps, warm)
    launches = (ctx.kernel_launches - launches0) * args.steps // (args.steps + warm)
    if world == 1:
        if sampler:
            sampler.hold(step)
    else:                      # the same number of extra steps on every rank (the step holds collectives)
        for _ in range(300):
            step()
        torch.cuda.synchronize()
    plan = layer.last_plan

    def e2e_step():
        d_h.view(torch.uint16).copy_(h_local, non_blocking=True)
        d_r.view(torch.uint16).copy_(r_local, non_blocking=True)
        step()
        host_out.copy_(d_out, non_blocking=True)

    e2e_wall = []
    for i in range(3 + args.steps):
        flush_l2(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        e2e_step()
        torch.cuda.synchronize()
        e2e_wall.append(time.perf_counter() - t0)
    e2e_ms = sum(e2e_wall[3:]) / args.steps * 1e3
    clocks = sampler.stop() if sampler else None

    ms = sum(times) / len(times)
    t = torch.tensor([ms, e2e_ms, float(plan.rows_received) if plan else float(n_local * FULL["K"])], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, max_rows = float(t[0]), float(t[1]), float(t[2])

    g1 = None
    if kind == "ep" and world > 1 and rank == 0:
        # the same job on one GPU, for the scaling reference (other ranks idle)
        d_all = torch.from_numpy(hidden).cuda().view(torch.float16)
        r_all = torch.from_numpy(resid).cuda().view(torch.float16)
        o_all = torch.zeros_like(d_all)
        solo = pkg.ep.ExpertParallelLayer(ctx, 0, FULL["E"], FULL["K"], FULL["H"])
        solo.reserve(n_total, n_total * FULL["K"])
        ts = []
        for i in range(3 + 5):
            flush_l2(i)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); solo.forward(d_all, o_all, residual=r_all); b.record(stream)
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        g1 = n_total / (sum(ts[3:]) / 5 * 1e-3)
        # and the sharded result equals the single-GPU result on this rank's tokens
        assert torch.equal(o_all[lo:lo + n_local], d_out), "expert-parallel output differs from the single-GPU output"
    if world > 1:
        dist.barrier()

    if rank == 0:
        peak, peak_kind = measured_tensor_peak()
        flops = n_total * FLOPS_PER_TOKEN
        achieved = flops / (ms * 1e-3) / 1e12 / world        # per GPU
        tps = n_total / (ms * 1e-3)
        line = {
            "metric": w["metric"], "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if kind == "ep" else "weak", "vs_baseline": None,
            "dtype": "fp16 tensor-core inputs (weights dequantised from Q4_0 on the fly), f32 accumulate", "data": "synthetic",
            "config": {"workload": w["workload"] if args.routing == "zipf" else w["workload"].replace("Zipf(1.1)-skewed", "uniform"),
                       "tokens_per_step": n_total, "qtype": "q4_0", "routing": args.routing,
                       "parallelism": f"ep{world}" if kind == "ep" else "1 gpu",
                       **({"exchange": exchange} if kind == "ep" and world > 1 else {}),
                       "l2": "flushed between timed iterations (256 MiB written, then 256 MiB read)"},
            "e2e": {"value": n_total / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * n_local * FULL["H"] * 2,
                    "d2h_bytes_per_step": n_local * FULL["H"] * 2,
                    "timer": "host wall clock: pinned H2D of hidden and residual, layer, D2H of the output (per rank, max over ranks)"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (whole layer time used)", "achieved": achieved,
                         "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "TFLOP/s", "frac": achieved / peak,
                         "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS, "algorithmic_flops_per_step": flops,
                         # DRAM bytes of the dominant launch (routed gate/up GEMM) from one ncu capture of the 4096-token workload
                         "traffic": 159.2e6 if (kind == "prefill" and args.routing == "zipf") else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the routed gate/up launch "
                                           "(profiles/grouped_gemm_kernel__prefill_q4_4096.md)"},
            "clocks": clocks, "step_ms_min_max": [min(times), max(times)],
        }
        if kind == "ep":
            mean_rows = n_total * FULL["K"] / world
            line["load"] = {"max_rows_received_per_gpu": max_rows, "mean_rows_per_gpu": mean_rows, "max_over_mean": max_rows / mean_rows}
            if g1 is not None:
                line["single_gpu_tokens_per_s_same_job"] = g1
        if not args.no_cpu_baseline and world == 1:
            from oracle import oracle as orc
            cps, ckind, sample = cpu_tokens_per_s(L, hidden, resid, orc.host_threads())
            line["cpu_baseline"] = {"value": cps, "unit": "tokens/s", "cores": orc.host_threads(), "kind": ckind, "sample": sample}
        print(json.dumps(line), flush=True)
    ctx.close()


def run_decode(args, rank: int, local_rank: int, world: int) -> None:
    """One token through the 11-layer stack (N replicas when launched on N GPUs)."""
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    layers, hidden = synth_stack(N_LAYERS, "q4_0", SEED_DECODE)
    ctx = pkg.Context()
    for L in layers:
        ctx.map_layer(L)
    ctx.allocate_runtime_arenas(1)
    stream = torch.cuda.current_stream()
    ctx.set_stream(stream.cuda_stream)

    d_hidden = torch.from_numpy(hidden).cuda().view(torch.float16)
    d_out = torch.zeros_like(d_hidden)
    flush_l2 = make_flush(torch)

    def step():
        ctx.stack_forward(0, N_LAYERS, d_hidden, 1, d_out)

    for _ in range(max(args.warmup, 3)):
        flush_l2(1)
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = ctx.kernel_launches
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for i in range(args.steps):
        flush_l2(i)
        starts[i].record(stream)
        step()
        ends[i].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = ctx.kernel_launches - launches0
    times_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    if sampler:
        sampler.hold(step)
    ms_per_step = sum(times_ms) / len(times_ms)
    ctx.synchronize()

    # end to end through the host-buffer entry point: pinned staging, H2D, 11 layers, D2H, wait
    e2e_times = []
    for i in range(max(3, min(args.warmup, 5)) + args.steps):
        flush_l2(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        host_out = ctx.stack_forward_host(0, N_LAYERS, hidden)
        e2e_times.append(time.perf_counter() - t0)
    e2e_times = e2e_times[-args.steps:]
    e2e_ms = sum(e2e_times) / len(e2e_times) * 1e3
    assert np.array_equal(host_out, d_out.cpu().numpy().view(np.uint16)), "host and device entry points disagree"
    clocks = sampler.stop() if sampler else None

    t = torch.tensor([ms_per_step, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        step_bytes = N_LAYERS * layer_bytes("q4_0")
        achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        if achieved > 1.25 * peak:
            raise SystemExit(f"implausible timing: {achieved:.0f} GB/s against a measured peak of {peak:.0f}; "
                             "the timed stream did not carry the kernels")
        us_per_token = ms_per_step * 1e3 / world          # N replicas: job-level time per token
        line = {
            "metric": "moe_decode_us_per_token", "value": us_per_token, "unit": "us/token", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16 activations and Q4_0 weights",
            "data": "synthetic", "config": {**workload_config(), "parallelism": "replicas only" if world > 1 else "1 gpu"},
            "e2e": {"value": e2e_ms * 1e3 / world, "unit": "us/token", "h2d_bytes_per_step": FULL["H"] * 2,
                    "d2h_bytes_per_step": FULL["H"] * 2, "timer": "host wall clock around uocr_cuda_moe_stack_forward_host"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "decode_sliced_kernel (one launch = one step)", "achieved": achieved,
                         "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "algorithmic_bytes_per_step": step_bytes,
                         "traffic": 165.4e6, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture "
                         "of this kernel on this workload, taken before its latest changes, which read the same bytes "
                         "(profiles/decode_sliced_kernel__decode_q4_11layers.md)"},
            "clocks": clocks,
            "per_layer_us": ms_per_step * 1e3 / N_LAYERS,
            "step_ms_min_max": [min(times_ms), max(times_ms)],
        }
        if not args.no_cpu_baseline:
            from oracle import oracle as orc
            threads = orc.host_threads()
            us, kind, sample = _cpu_arm(layers[: args.cpu_layers], hidden, argparse.Namespace(steps=3, warmup=1), threads)
            line["cpu_baseline"] = {"value": us, "unit": "us/token", "cores": threads, "kind": kind, "sample": sample}
        print(json.dumps(line), flush=True)
    ctx.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["decode", "prefill", "ep"])
    ap.add_argument("--cpu-layers", type=int, default=2, help="layers of the stack the CPU baseline samples")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--routing", default="zipf", choices=["zipf", "uniform"], help="expert popularity of the prefill / ep workloads")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="ep workload: how rows travel between the GPUs")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kind = args.workload or ("decode" if max(world, args.gpus) == 1 else "ep")
    if args.steps is None:
        args.steps = 50 if kind == "decode" else 20

    if args.impl == "reference":
        if kind == "decode":
            run_reference_arm(args, rank)
        else:
            run_reference_tokens(args, rank, kind)
        return

    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not (entry.PKG_DIR / "libuocr_cuda_moe.so").exists():
        entry.build()
    if kind == "decode":
        run_decode(args, rank, local_rank, world)
    else:
        run_tokens(args, kind, rank, local_rank, world)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
