#!/usr/bin/env python3
"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|prefill|ep|batched|lm_head] [--extras all|none]

Prints ONE JSON line on rank 0.  Workloads (seeded synthetic inputs of the benchmark plan's shapes):
  decode   (default, the headline)  one token through 11 stacked MoE layers (hidden 1280, 64 experts top-6 + shared
           1792, FFN 896, Q4_0 group-64 weights, seed 1); metric = microseconds per token; a step is one pass of
           the token through the 11 layers.  On N > 1 GPUs: N independent replicas (the path does not shard for one
           token), value = step time / N.
  prefill  one MoE layer on 4096 tokens, Q4_0 (or --qtype f16), Zipf(1.1)-skewed routing, seed 3; tokens per second.
  batched  one MoE layer on 8 / 32 / 64 tokens, Q8_0, per-expert logit bias N(0,1), seed 2; microseconds per step and
           the fraction of the HBM roofline for the bytes of the experts the step really selects.
  ep       one MoE layer on 8 x 2048 = 16384 tokens, Q4_0, Zipf(1.1) and uniform routing, seed 4, the 64 experts
           sharded over the N GPUs with the exchange over peer memory (or NCCL all-to-all); tokens per second of the
           whole job (fixed total work: strong scaling).  Every rank checks its shard against the single-GPU layer.
With --extras all (default) the headline line also carries short timed passes of the other workloads under the keys
"prefill", "batched_decode" (one GPU only) and "ep" (every N, with an explicit scaling_efficiency).

  value  device time per step (CUDA events on the launching stream), inputs resident in HBM;
  e2e    wall time of the host-buffer C-ABI call (host->device copy, 11 layers, device->host copy);
  roofline.achieved  algorithmic bytes per step (11 x 14 786 560 B of weights + activations) / step time;
  cpu_baseline       the reference's CPU layer function (oracle/_ref) on this host's cores, bounded sample.

Between timed iterations a buffer larger than L2 is written so that no step finds its weights cached.
With --impl reference the reference's CPU path alone is timed on the same workload.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
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
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
FLOPS_PER_TOKEN = 2 * FULL["E"] * FULL["H"] + FULL["K"] * 3 * 2 * FULL["F"] * FULL["H"] + 3 * 2 * FULL["S"] * FULL["H"]
L2_NOTE = "flushed between timed iterations (256 MiB written, then 256 MiB read)"


def layer_bytes(qtype_name: str, n_tokens: int = 1, distinct_experts: int = 6) -> int:
    """Algorithmic bytes of one layer step: router + distinct selected experts + shared MLP + activations."""
    H, E, F, S = FULL["H"], FULL["E"], FULL["F"], FULL["S"]
    per = {"f16": lambda r, c: 2 * r * c, "q8_0": lambda r, c: r * c + 2 * r * (c // 64),
           "q4_0": lambda r, c: r * c // 2 + 2 * r * (c // 64)}[qtype_name]
    expert = 2 * per(F, H) + per(H, F)
    shared = 2 * per(S, H) + per(H, S)
    return E * H * 2 + distinct_experts * expert + shared + n_tokens * H * 2 * 3


def _peak(key: str, fallback: float) -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())[key]), "measured"
        except Exception:
            pass
    return fallback, "fallback"


def measured_peaks() -> tuple[float, str]:
    return _peak("hbm_gbs", FALLBACK_HBM_GBS)


def measured_tensor_peak() -> tuple[float, str]:
    return _peak("bf16_tflops", FALLBACK_BF16_TFLOPS)


def captured_traffic(summary: str, kernel_source: str) -> tuple[float | None, str]:
    """DRAM bytes per launch from the ncu summary under profiles/, valid only for the kernel source it was taken on:
    the summary carries a line `dram_bytes_per_launch: <bytes> source_sha16: <first 16 hex of the sha256 of the .cu file>`."""
    path = ROOT / "profiles" / summary
    src = ROOT / "unlimitedocr.c_b200" / "csrc" / kernel_source
    if not path.exists() or not src.exists():
        return None, f"no ncu capture on record (profiles/{summary})"
    m = re.search(r"^dram_bytes_per_launch:\s*(\d+)\s+source_sha16:\s*([0-9a-f]{16})", path.read_text(), re.M)
    if not m:
        return None, f"profiles/{summary} holds no ncu capture of the kernel as it is now (see the summary for why)"
    sha = hashlib.sha256(src.read_bytes()).hexdigest()[:16]
    if m.group(2) != sha:
        return None, f"the capture in profiles/{summary} is of an earlier version of {kernel_source}"
    return float(m.group(1)), f"dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture (profiles/{summary})"


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

    def hold(self, step, minimum: int = 6, limit_s: float = 4.0) -> None:
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


def workload_config(world: int = 1) -> dict:
    return {"workload": "decode: 1 token x 11 stacked MoE layers, hidden 1280, 64 experts top-6 + shared 1792, "
                        "FFN 896, Q4_0 group-64 experts and shared MLP, seed 1",
            "layers": N_LAYERS, "tokens_per_step": 1, "qtype": "q4_0",
            "parallelism": "replicas only" if world > 1 else "1 gpu", "l2": L2_NOTE}


# ------------------------------------------------------------------------------------------ the CPU arm

def run_reference_arm(args, rank: int, world: int) -> None:
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
        "config": workload_config(max(world, args.gpus)),
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


# ------------------------------------------------------------------------------------------ GPU helpers

def make_flush(torch):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    reader = torch.empty(256 << 20, dtype=torch.uint8, device="cuda").view(torch.int32)

    def flush_l2(i: int):
        # write a buffer larger than L2, then read a second one through the cache so that the weights are
        # cold AND the cache is not left full of dirty lines whose write-back would compete with the step
        flush.fill_(i & 0xFF)
        reader.max()
    return flush_l2


def timed_steps(torch, dist, world, stream, flush_l2, fn, steps: int, warmup: int) -> list[float]:
    """W untimed steps, then K steps each between two CUDA events on the launching stream (ms per step).
    On several GPUs every step starts behind a barrier of all ranks that is ordered on the stream (a one-element
    all-reduce), not one that blocks the host: with a host-blocking barrier the host could not run ahead of the GPU and
    its launch latency (and the scheduling noise of N processes on one host) would sit between the two events."""
    token = torch.zeros(1, dtype=torch.int32, device="cuda") if world > 1 else None
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
            dist.all_reduce(token)             # every rank starts the step together; the barrier is not timed
        starts[i].record(stream)
        fn()
        ends[i].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def tensor_roofline(n_tokens: int, ms: float, world: int = 1) -> dict:
    peak, peak_kind = measured_tensor_peak()
    flops = n_tokens * FLOPS_PER_TOKEN
    achieved = flops / (ms * 1e-3) / 1e12 / world        # per GPU
    return {"bound": "tensor", "kernel": "grouped_gemm_kernel (whole layer time used)", "achieved": achieved, "peak": peak,
            "peak_kind": f"of {peak_kind}", "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS, "algorithmic_flops_per_step": flops}


# ------------------------------------------------------------------------------------------ prefill (one GPU)

def measure_prefill(pkg, torch, flush_l2, qtype_name: str, steps: int, warmup: int, with_e2e: bool = True) -> dict:
    """One MoE layer on 4096 tokens (benchmark plan config 4): device time per call and the call with pinned
    host-to-device / device-to-host copies of the activations."""
    w = token_workload("prefill")
    n = w["n_tokens"]
    L, hidden, resid = synth_token_layer(w["seed"], n, qtype_name)
    stream = torch.cuda.current_stream()
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(n)
        ctx.set_stream(stream.cuda_stream)
        h_host = torch.from_numpy(hidden.copy()).pin_memory()
        r_host = torch.from_numpy(resid.copy()).pin_memory()
        d_h, d_r = h_host.cuda().view(torch.float16), r_host.cuda().view(torch.float16)
        d_out = torch.zeros_like(d_h)
        host_out = torch.empty((n, FULL["H"]), dtype=torch.float16).pin_memory()
        launches0 = ctx.kernel_launches
        times = timed_steps(torch, None, 1, stream, flush_l2, lambda: ctx.layer_forward(0, d_h, n, d_out, residual=d_r), steps, warmup)
        launches = (ctx.kernel_launches - launches0) // (steps + warmup)
        ms = sum(times) / len(times)
        out = {"workload": w["workload"].replace("Q4_0", qtype_name.upper()), "qtype": qtype_name, "tokens_per_step": n,
               "tokens_per_s": n / (ms * 1e-3), "ms_per_step": ms, "step_ms_min_max": [min(times), max(times)],
               "gpu_launches_per_step": int(launches), "roofline": tensor_roofline(n, ms)}
        if with_e2e:
            wall = []
            for i in range(3 + steps):
                flush_l2(i)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                d_h.view(torch.uint16).copy_(h_host, non_blocking=True)
                d_r.view(torch.uint16).copy_(r_host, non_blocking=True)
                ctx.layer_forward(0, d_h, n, d_out, residual=d_r)
                host_out.copy_(d_out, non_blocking=True)
                torch.cuda.synchronize()
                wall.append(time.perf_counter() - t0)
            e2e_ms = sum(wall[3:]) / steps * 1e3
            out["e2e"] = {"value": n / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * n * FULL["H"] * 2,
                          "d2h_bytes_per_step": n * FULL["H"] * 2}
        ctx.synchronize()
    return out


# ------------------------------------------------------------------------------------------ dense MLP of layer 0 (one GPU)

def measure_dense_mlp(pkg, torch, flush_l2, steps: int, warmup: int) -> dict:
    """The first decoder layer's dense SwiGLU MLP (hidden 1280, intermediate 6848, Q8_0 as the mixed profiles store it),
    with its RMSNorm prologue: one token (weight bytes against the HBM roofline) and 4096 tokens (tensor roofline)."""
    from oracle import quant
    H, S = FULL["H"], 6848
    rng = np.random.default_rng(5)
    mats = [quant.make_matrix(quant.QTYPE_Q8_0, rng.standard_normal(shape, dtype=np.float32) * 0.02) for shape in ((S, H), (S, H), (H, S))]
    weight_bytes = 3 * (S * H + S * H // 64 * 2)
    peak_hbm, kind_hbm = measured_peaks()
    peak_tc, kind_tc = measured_tensor_peak()
    stream = torch.cuda.current_stream()
    out = {"workload": "dense SwiGLU MLP of decoder layer 0: hidden 1280, intermediate 6848, Q8_0, RMSNorm prologue, seed 5", "l2": L2_NOTE,
           "tokens": {}}
    with pkg.Context() as ctx:
        idx = ctx.map_dense_mlp(*mats, token_capacity=4096)
        ctx.set_stream(stream.cuda_stream)
        w = torch.from_numpy(rng.uniform(0.5, 1.5, H).astype("<f2").view(np.uint16)).cuda().view(torch.float16)
        for n in (1, 4096):
            x = torch.from_numpy(quant.synth_activations(rng, n, H)).cuda().view(torch.float16)
            y = torch.zeros_like(x)
            launches0 = ctx.kernel_launches
            times = timed_steps(torch, None, 1, stream, flush_l2, lambda: ctx.dense_mlp_forward_normed(idx, x, w, 1e-6, n, y), steps, warmup)
            launches = (ctx.kernel_launches - launches0) // (steps + warmup)
            ms = sum(times) / len(times)
            r = {"us_per_step": ms * 1e3, "gpu_launches_per_step": int(launches)}
            if n == 1:
                gbs = weight_bytes / (ms * 1e-3) / 1e9
                r["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak_hbm, "peak_kind": f"of {kind_hbm}", "unit": "GB/s",
                                 "frac": gbs / peak_hbm, "algorithmic_bytes_per_step": weight_bytes}
            else:
                tf = 2.0 * 3 * S * H * n / (ms * 1e-3) / 1e12
                r["tokens_per_s"] = n / (ms * 1e-3)
                r["roofline"] = {"bound": "tensor", "achieved": tf, "peak": peak_tc, "peak_kind": f"of {kind_tc}", "unit": "TFLOP/s",
                                 "frac": tf / peak_tc, "algorithmic_flops_per_step": 2.0 * 3 * S * H * n}
            out["tokens"][str(n)] = r
        ctx.synchronize()
    return out


# ------------------------------------------------------------------------------------------ LM head (one GPU)

def measure_lm_head(pkg, torch, flush_l2, steps: int, warmup: int) -> dict:
    """The vocabulary projection fused with the argmax, one token: [129280, 1280] in Q4_0 and Q8_0 (83 / 165 MB per
    decoded token), weight bytes against the HBM roofline."""
    from oracle import quant
    V, H = 129280, FULL["H"]
    rng = np.random.default_rng(6)
    w = rng.standard_normal((V, H), dtype=np.float32) * 0.02
    peak, kind = measured_peaks()
    stream = torch.cuda.current_stream()
    out = {"workload": "LM head fused with argmax: vocabulary 129280, hidden 1280, one token, seed 6", "l2": L2_NOTE, "qtype": {}}
    x = torch.from_numpy(quant.synth_activations(rng, 1, H)).cuda().view(torch.float16)
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    for qname in ("q4_0", "q8_0"):
        m = quant.make_matrix(quant.QTYPE_BY_NAME[qname], w)
        nbytes = int(m.qweight.size + (0 if m.qscale is None else m.qscale.size * 2))
        with pkg.Context() as ctx:
            ctx.map_lm_head(m)
            ctx.set_stream(stream.cuda_stream)
            times = timed_steps(torch, None, 1, stream, flush_l2, lambda: ctx.lm_head_argmax(x, 1, ids), steps, warmup)
            ctx.synchronize()
        ms = sum(times) / len(times)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out["qtype"][qname] = {"us_per_token": ms * 1e3, "gpu_launches_per_step": 1,
                               "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": f"of {kind}", "unit": "GB/s",
                                            "frac": gbs / peak, "algorithmic_bytes_per_step": nbytes}}
    return out


# ------------------------------------------------------------------------------------------ batched decode (one GPU)

def measure_batched_decode(pkg, torch, flush_l2, steps: int, warmup: int) -> dict:
    """One Q8_0 layer on 8 / 32 / 64 tokens with a per-expert logit bias N(0,1) (benchmark plan config 3).  The step is
    bound by reading the weights of the experts it selects: bytes = router + U distinct experts + shared MLP +
    activations, against the measured copy bandwidth."""
    from oracle import quant
    rng = np.random.default_rng(2)
    bias = rng.standard_normal(FULL["E"]).astype(np.float32)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q8_0, logit_bias=bias, **FULL)
    peak, peak_kind = measured_peaks()
    stream = torch.cuda.current_stream()
    out = {"workload": "batched decode: one MoE layer, Q8_0, per-expert logit bias N(0,1), seed 2", "qtype": "q8_0",
           "peak_gbs": peak, "peak_kind": f"of {peak_kind}", "l2": L2_NOTE, "tokens": {}}
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(64)
        ctx.set_stream(stream.cuda_stream)
        for n in (8, 32, 64):
            hidden = quant.synth_activations(rng, n, FULL["H"])
            d_h = torch.from_numpy(hidden).cuda().view(torch.float16)
            d_out = torch.zeros_like(d_h)
            d_ids = torch.zeros((n, FULL["K"]), dtype=torch.int32, device="cuda")
            ctx.layer_forward(0, d_h, n, d_out, residual=d_h, top_ids=d_ids)
            ctx.synchronize()
            distinct = int(np.unique(d_ids.cpu().numpy()).size)
            launches0 = ctx.kernel_launches
            times = timed_steps(torch, None, 1, stream, flush_l2, lambda: ctx.layer_forward(0, d_h, n, d_out, residual=d_h), steps, warmup)
            launches = (ctx.kernel_launches - launches0) // (steps + warmup)
            ms = sum(times) / len(times)
            nbytes = layer_bytes("q8_0", n, distinct)
            achieved = nbytes / (ms * 1e-3) / 1e9
            out["tokens"][str(n)] = {"us_per_step": ms * 1e3, "us_per_token": ms * 1e3 / n, "distinct_experts": distinct,
                                     "algorithmic_bytes_per_step": nbytes, "achieved_gbs": achieved, "frac": achieved / peak,
                                     "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "gpu_launches_per_step": int(launches),
                                     "served_by": ctx.regime_name(0, n)}
    traffic, source = captured_traffic("decode_batched_kernel__batched_q8.md", "moe_decode_batched.cu")
    out["tokens"]["8"]["traffic"], out["tokens"]["8"]["traffic_source"] = traffic, source + " (the weight-streaming kernel of the three)"
    return out


# ------------------------------------------------------------------------------------------ expert parallelism

def measure_ep(pkg, torch, dist, rank: int, world: int, flush_l2, steps: int, warmup: int, exchange_kind: str,
               routings=("zipf", "uniform"), with_e2e: bool = True) -> dict:
    """One Q4_0 MoE layer on 16384 tokens (benchmark plan config 5), its experts sharded over the ranks; for each
    routing: tokens/s of the whole job, the same job on one GPU (rank 0), every rank's shard checked bit for bit
    against the single-GPU output, and the rows the busiest rank received."""
    import dataclasses
    w = token_workload("ep")
    n_total = w["n_tokens"]
    if n_total % world:
        raise SystemExit(f"{n_total} tokens do not divide over {world} ranks")
    n_local, lo = n_total // world, rank * (n_total // world)
    H, E, K = FULL["H"], FULL["E"], FULL["K"]
    L, hidden, resid = synth_token_layer(w["seed"], n_total, routing="zipf")
    stream = torch.cuda.current_stream()
    ctx = pkg.Context()
    layer_of = {"zipf": ctx.map_layer(L), "uniform": ctx.map_layer(dataclasses.replace(L, logit_bias=None))}
    ctx.allocate_runtime_arenas(n_total)     # a rank can receive every pair of the job, and every rank also runs the whole job alone
    ctx.set_stream(stream.cuda_stream)
    d_all = torch.from_numpy(hidden).cuda().view(torch.float16)
    r_all = torch.from_numpy(resid).cuda().view(torch.float16)
    h_local = torch.from_numpy(hidden[lo:lo + n_local].copy()).pin_memory()
    r_local = torch.from_numpy(resid[lo:lo + n_local].copy()).pin_memory()
    d_h, d_r = d_all[lo:lo + n_local].clone(), r_all[lo:lo + n_local].clone()
    d_out = torch.zeros_like(d_h)
    o_all = torch.zeros_like(d_all)
    host_out = torch.empty((n_local, H), dtype=torch.float16).pin_memory()
    result = {"workload": w["workload"].replace("Zipf(1.1)-skewed routing", "Zipf(1.1)-skewed and uniform routing"),
              "tokens_per_step": n_total, "qtype": "q4_0", "n_gpus": world, "parallelism": f"ep{world}", "l2": L2_NOTE}
    exchange = "none (one GPU)"
    pair_counts = {}

    def run_variant(name: str, li: int, collectives: bool = False) -> None:
        """Time one mapped layer (index li) sharded over the ranks; result[name] gets the figures.  collectives: the
        peer-memory form with torch.distributed collectives between its phases instead of the device-side flags."""
        nonlocal exchange
        layer = None
        if world > 1 and exchange_kind == "peer":
            why = ""
            try:
                layer = pkg.ep.PeerExpertParallelLayer(ctx, li, E, K, H, row_capacity=n_total * K, rank=rank, world=world,
                                                       dist_module=dist)
                exchange = ("peer memory (CUDA IPC over NVLink), fused into gather and combine; counts, row offsets and the "
                            "synchronisation of the ranks (flags in peer memory) stay on the device")
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
            if world > 1 and exchange_kind != "peer":
                exchange = "nccl all_to_all_single"
            layer = pkg.ep.ExpertParallelLayer(ctx, li, E, K, H, rank=rank, world=world, dist_module=dist if world > 1 else None)
            layer.reserve(n_local, n_total * K)
        peer_form = isinstance(layer, pkg.ep.PeerExpertParallelLayer)
        if collectives and not peer_form:
            return
        step = (lambda: layer.forward_collectives(d_h, d_out, residual=d_r)) if collectives else (lambda: layer.forward(d_h, d_out, residual=d_r))
        launches0 = ctx.kernel_launches
        times = timed_steps(torch, dist, world, stream, flush_l2, step, steps, warmup)
        launches = (ctx.kernel_launches - launches0) // (steps + warmup)
        plan = layer.last_plan
        pair_counts[name] = layer.gathered_counts().sum(axis=0)
        e2e_ms = 0.0
        if with_e2e:
            wall = []
            for i in range(2 + steps):
                flush_l2(i)
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                t0 = time.perf_counter()
                d_h.view(torch.uint16).copy_(h_local, non_blocking=True)
                d_r.view(torch.uint16).copy_(r_local, non_blocking=True)
                step()
                host_out.copy_(d_out, non_blocking=True)
                torch.cuda.synchronize()
                wall.append(time.perf_counter() - t0)
            e2e_ms = sum(wall[2:]) / steps * 1e3
        ms = sum(times) / len(times)
        # the same job on one GPU: every rank runs it once (the check), rank 0 also times it (the scaling reference)
        solo = pkg.ep.ExpertParallelLayer(ctx, li, E, K, H)
        solo.reserve(n_total, n_total * K)
        ts = []
        for i in range(1 + (3 + 5 if rank == 0 else 0)):
            flush_l2(i)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); solo.forward(d_all, o_all, residual=r_all); b.record(stream)
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        if world > 1:
            dist.barrier()
        step()                                   # the sharded result once more, after the single-GPU run
        torch.cuda.synchronize()
        mismatch = 0 if torch.equal(o_all[lo:lo + n_local], d_out) else 1
        t = torch.tensor([ms, e2e_ms, float(plan.rows_received) if plan else float(n_local * K), float(mismatch)],
                         dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, max_rows, mismatches = float(t[0]), float(t[1]), float(t[2]), int(t[3])
        if mismatches:
            raise SystemExit(f"expert-parallel output differs from the single-GPU output on at least one rank ({name})")
        tps = n_total / (ms * 1e-3)
        mean_rows = n_total * K / world
        r = {"tokens_per_s": tps, "ms_per_step": ms, "step_ms_min_max": [min(times), max(times)],
             "gpu_launches_per_step": int(launches), "roofline": tensor_roofline(n_total, ms, world),
             "all_ranks_equal_single_gpu_bit_for_bit": True,
             "load": {"max_rows_received_per_gpu": max_rows, "mean_rows_per_gpu": mean_rows, "max_over_mean": max_rows / mean_rows}}
        if with_e2e:
            r["e2e"] = {"value": n_total / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * n_local * H * 2,
                        "d2h_bytes_per_step": n_local * H * 2,
                        "timer": "host wall clock: pinned H2D of hidden and residual, layer, D2H of the output (per rank, max over ranks)"}
        if rank == 0:
            g1 = n_total / (sum(ts[-5:]) / 5 * 1e-3)
            r["single_gpu_tokens_per_s_same_job"] = g1
            r["scaling_efficiency"] = tps / g1 / world
        result[name] = r
        if isinstance(layer, pkg.ep.PeerExpertParallelLayer):
            layer.close()                          # every rank together: waits for all ranks' kernels before freeing

    for routing in routings:
        run_variant(routing, layer_of[routing])
    if world > 1 and "zipf" in routings:
        # The named configuration shards contiguous expert ranges.  Beside it: the same layer with its experts relabelled
        # so that the ranks' loads are even (longest-processing-time placement from the pair counts just observed).
        from oracle import quant
        order = pkg.ep.balanced_placement(pair_counts["zipf"], world)
        run_variant("zipf_balanced_placement", ctx.map_layer(quant.permute_experts(L, order)))
        result["zipf_balanced_placement"]["placement"] = "experts relabelled by ep.balanced_placement(observed pair counts)"
        run_variant("zipf_synchronised_by_collectives", layer_of["zipf"], collectives=True)
        if "zipf_synchronised_by_collectives" in result:
            result["zipf_synchronised_by_collectives"]["note"] = ("the same peer-memory exchange with one all_gather of the counts and two "
                                                                  "all-reduce barriers of torch.distributed per call instead of flags in peer memory")
    result["exchange"] = exchange
    ctx.synchronize()
    ctx.close()
    return result


# ------------------------------------------------------------------------------------------ decode (headline)

TRACE_POINTS = [("activations_in_smem", 0), ("own_router_logits", 8), ("logits_exchanged", 9), ("expert_chosen", 1),
                ("weight_fetch_issued", 2), ("first_chunk_in_smem", 3), ("gate_up_chunk0", 10), ("chunk2_arrived", 11),
                ("gate_up_chunk2", 12), ("last_groups_arrived", 13), ("own_sums", 14), ("all_warps_sums", 15),
                ("swiglu_products", 4), ("partial_outputs", 5), ("partial_sums_sent", 6), ("layer_output_complete", 7)]


def decode_timeline(ctx, torch, d_hidden, d_out, flush_l2, sm_mhz: float) -> dict:
    """Per-layer timeline of the one-launch decode kernel from its own clock stamps (uocr_cuda_context_set_profile_detail):
    microseconds since the previous layer's output was complete, mean over CTAs and layers 1..10 and mean over layers of
    the slowest CTA, for the 84 routed-expert CTAs and the 28 shared-MLP CTAs."""
    n_cta, n_pts = 128, 16
    trace = torch.zeros(n_cta * N_LAYERS * n_pts, dtype=torch.int64, device="cuda")
    ctx.set_profile_detail(trace)
    for i in range(3):
        flush_l2(i)
        ctx.stack_forward(0, N_LAYERS, d_hidden, 1, d_out)
        torch.cuda.synchronize()
    ctx.set_profile_detail(None)
    t = trace.cpu().numpy().reshape(n_cta, N_LAYERS, n_pts).astype(np.float64)
    if not t[:112, :, 7].all():
        return {"unavailable": "the decode kernel in use writes no clock stamps"}
    per_us = sm_mhz

    def table(rows):
        rel = (t[rows, 1:, :] - t[rows, :-1, 7:8]) / per_us
        mean, slow = rel.mean((0, 1)), rel.max(0).mean(0)
        return {name: [round(float(mean[i]), 3), round(float(slow[i]), 3)] for name, i in TRACE_POINTS}

    return {"columns": "[mean, slowest CTA] in us since the previous layer's output was complete", "sm_mhz_assumed": sm_mhz,
            "routed_ctas": table(slice(0, 84)), "shared_mlp_ctas": table(slice(84, 112)),
            "kernel_entry_to_first_layer_us": round(float((t[0, 0, 0] - t[127, 0, 0]) / per_us), 3),
            "kernel_entry_to_exit_us": round(float((t[127, 0, 1] - t[127, 0, 0]) / per_us), 3)}


def measure_decode(pkg, torch, dist, rank: int, local_rank: int, world: int, flush_l2, args) -> dict | None:
    """One token through the 11-layer stack (N replicas when launched on N GPUs)."""
    layers, hidden = synth_stack(N_LAYERS, "q4_0", SEED_DECODE)
    ctx = pkg.Context()
    for L in layers:
        ctx.map_layer(L)
    ctx.allocate_runtime_arenas(1)
    stream = torch.cuda.current_stream()
    ctx.set_stream(stream.cuda_stream)
    d_hidden = torch.from_numpy(hidden).cuda().view(torch.float16)
    d_out = torch.zeros_like(d_hidden)
    warm = max(args.warmup, 3)

    def step():
        ctx.stack_forward(0, N_LAYERS, d_hidden, 1, d_out)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = ctx.kernel_launches
    times_ms = timed_steps(torch, dist, world, stream, flush_l2, step, args.steps, warm)
    launches = (ctx.kernel_launches - launches0) * args.steps // (args.steps + warm)
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
    timeline = None
    per_layer = None
    if rank == 0 and args.extras == "all":
        timeline = decode_timeline(ctx, torch, d_hidden, d_out, flush_l2, float((clocks or {}).get("sm_mhz") or 1965.0))
        # The same token as eleven separate calls, each with its post-attention RMSNorm, the way a decoder whose attention
        # sits between the MoE layers has to make them (uocr_cuda_moe_layer_forward_normed; the attention itself is not here).
        norm_w = torch.ones(FULL["H"], dtype=torch.float16, device="cuda")
        ping, pong = d_hidden.clone(), torch.zeros_like(d_hidden)

        def layer_calls():
            a, b = ping, pong
            for l in range(N_LAYERS):
                ctx.layer_forward_normed(l, a, norm_w, 1.0e-6, 1, b)
                a, b = b, a

        l0 = ctx.kernel_launches
        pl_ms = timed_steps(torch, None, 1, stream, flush_l2, layer_calls, max(5, min(args.steps, 20)), 3)
        per_layer = {"workload": "the decode token as 11 calls of RMSNorm + MoE layer (one call per decoder layer)",
                     "us_per_token": sum(pl_ms) / len(pl_ms) * 1e3,
                     "gpu_launches_per_token": (ctx.kernel_launches - l0) // (max(5, min(args.steps, 20)) + 3)}
        ctx.synchronize()

    t = torch.tensor([ms_per_step, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms = float(t[0]), float(t[1])
    ctx.close()
    if rank != 0:
        return None
    peak, peak_kind = measured_peaks()
    step_bytes = N_LAYERS * layer_bytes("q4_0")
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    if achieved > 1.25 * peak:
        raise SystemExit(f"implausible timing: {achieved:.0f} GB/s against a measured peak of {peak:.0f}; "
                         "the timed stream did not carry the kernels")
    traffic, traffic_source = captured_traffic("decode_sliced_kernel__decode_q4_11layers.md", "moe_decode_sliced.cu")
    us_per_token = ms_per_step * 1e3 / world          # N replicas: job-level time per token
    line = {
        "metric": "moe_decode_us_per_token", "value": us_per_token, "unit": "us/token", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16 activations and Q4_0 weights",
        "data": "synthetic", "config": workload_config(world),
        "e2e": {"value": e2e_ms * 1e3 / world, "unit": "us/token", "h2d_bytes_per_step": FULL["H"] * 2,
                "d2h_bytes_per_step": FULL["H"] * 2, "timer": "host wall clock around uocr_cuda_moe_stack_forward_host"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "decode_sliced_kernel (one launch = one step)", "achieved": achieved,
                     "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "algorithmic_bytes_per_step": step_bytes,
                     "traffic": traffic, "traffic_source": traffic_source},
        "clocks": clocks,
        "per_layer_us": ms_per_step * 1e3 / N_LAYERS,
        "step_ms_min_max": [min(times_ms), max(times_ms)],
    }
    if timeline is not None:
        line["decode_timeline_us"] = timeline
    if per_layer is not None:
        line["decode_per_layer_calls"] = per_layer
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        threads = orc.host_threads()
        us, kind, sample = _cpu_arm(layers[: args.cpu_layers], hidden, argparse.Namespace(steps=3, warmup=1), threads)
        line["cpu_baseline"] = {"value": us, "unit": "us/token", "cores": threads, "kind": kind, "sample": sample}
    return line


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "ep", "batched", "lm_head"])
    ap.add_argument("--extras", default="all", choices=["all", "none"],
                    help="decode workload: also time short passes of the other workloads and append them to the line")
    ap.add_argument("--qtype", default="q4_0", choices=["q4_0", "f16", "q8_0"], help="prefill workload: weight format")
    ap.add_argument("--cpu-layers", type=int, default=2, help="layers of the stack the CPU baseline samples")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--routing", default="both", choices=["both", "zipf", "uniform"], help="ep workload: expert popularity")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="ep workload: how rows travel between the GPUs")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kind = args.workload
    if args.steps is None:
        args.steps = 50 if kind == "decode" else 20

    if args.impl == "reference":
        if kind == "lm_head":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU function for the fused LM head + argmax (Metal kernels only)"}))
            return
        if kind in ("decode", "batched"):
            run_reference_arm(args, rank, world)
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
    pkg = entry.load_package()
    flush_l2 = make_flush(torch)
    routings = ("zipf", "uniform") if args.routing == "both" else (args.routing,)
    short = max(5, min(args.steps, 10))
    line = None

    if kind == "decode":
        line = measure_decode(pkg, torch, dist, rank, local_rank, world, flush_l2, args)
        if args.extras == "all":
            t0 = time.perf_counter()
            extras = {}
            if world == 1:
                extras["prefill"] = {q: measure_prefill(pkg, torch, flush_l2, q, short, 3) for q in ("q4_0", "f16")}
                extras["batched_decode"] = measure_batched_decode(pkg, torch, flush_l2, short, 3)
                extras["dense_mlp"] = measure_dense_mlp(pkg, torch, flush_l2, short, 3)
                extras["lm_head"] = measure_lm_head(pkg, torch, flush_l2, short, 3)
            extras["ep"] = measure_ep(pkg, torch, dist, rank, world, flush_l2, short, 3, args.exchange, routings)
            if rank == 0:
                line.update(extras)
                line["extras_wall_s"] = time.perf_counter() - t0
    elif kind == "prefill":
        if world > 1:
            raise SystemExit("the prefill workload runs on one GPU (use --workload ep for several)")
        sampler = ClockSampler(local_rank)
        r = measure_prefill(pkg, torch, flush_l2, args.qtype, args.steps, max(args.warmup, 3))
        w = token_workload("prefill")
        line = {"metric": w["metric"], "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "fp16 tensor-core inputs (weights dequantised on the fly), f32 accumulate",
                "data": "synthetic", "config": {"workload": r["workload"], "tokens_per_step": r["tokens_per_step"],
                                                "qtype": args.qtype, "parallelism": "1 gpu", "l2": L2_NOTE},
                "e2e": r["e2e"], "gpu_launches": r["gpu_launches_per_step"] * args.steps, "roofline": r["roofline"],
                "clocks": sampler.stop(), "step_ms_min_max": r["step_ms_min_max"]}
        traffic, source = captured_traffic("grouped_gemm_kernel__prefill_q4_4096.md", "moe_grouped_gemm.cu")
        line["roofline"].update(traffic=traffic if args.qtype == "q4_0" else None, traffic_source=source)
        if not args.no_cpu_baseline:
            from oracle import oracle as orc
            L, hidden, resid = synth_token_layer(w["seed"], 1024, args.qtype)
            cps, ckind, sample = cpu_tokens_per_s(L, hidden, resid, orc.host_threads())
            line["cpu_baseline"] = {"value": cps, "unit": "tokens/s", "cores": orc.host_threads(), "kind": ckind, "sample": sample}
    elif kind == "lm_head":
        if world > 1:
            raise SystemExit("the LM-head workload runs on one GPU")
        r = measure_lm_head(pkg, torch, flush_l2, args.steps, max(args.warmup, 3))
        q4 = r["qtype"]["q4_0"]
        line = {"metric": "lm_head_argmax_us_per_token", "value": q4["us_per_token"], "unit": "us/token (Q4_0)", "n_gpus": 1,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": q4["us_per_token"] / 1e3,
                "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                "dtype": "int8 x int8 -> int32 on block-floating fp16 activations and Q4_0 / Q8_0 weights", "data": "synthetic",
                "config": {"workload": r["workload"], "tokens_per_step": 1, "qtype": "q4_0", "l2": L2_NOTE},
                "gpu_launches": 2 * args.steps, "roofline": dict(q4["roofline"], traffic=None), "lm_head": r}
    elif kind == "batched":
        if world > 1:
            raise SystemExit("the batched-decode workload runs on one GPU")
        r = measure_batched_decode(pkg, torch, flush_l2, args.steps, max(args.warmup, 3))
        t64 = r["tokens"]["64"]
        line = {"metric": "moe_batched_decode_us_per_step", "value": t64["us_per_step"], "unit": "us/step (64 tokens)", "n_gpus": 1,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t64["us_per_step"] / 1e3,
                "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32 accumulate over fp16 activations and Q8_0 weights", "data": "synthetic",
                "config": {"workload": r["workload"], "tokens_per_step": 64, "qtype": "q8_0", "l2": L2_NOTE},
                "gpu_launches": t64["gpu_launches_per_step"] * args.steps,
                "roofline": {"bound": "hbm", "achieved": t64["achieved_gbs"], "peak": r["peak_gbs"], "peak_kind": r["peak_kind"],
                             "unit": "GB/s", "frac": t64["frac"], "traffic": None}, "batched_decode": r}
    else:
        sampler = ClockSampler(local_rank) if rank == 0 else None
        ep = measure_ep(pkg, torch, dist, rank, world, flush_l2, args.steps, max(args.warmup, 3), args.exchange, routings)
        clocks = sampler.stop() if sampler else None
        if rank == 0:
            w = token_workload("ep")
            first = ep[routings[0]]
            line = {"metric": w["metric"], "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                    "warmup": max(args.warmup, 3), "ms_per_step": first["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "fp16 tensor-core inputs (weights dequantised from Q4_0 on the fly), f32 accumulate",
                    "data": "synthetic", "config": {"workload": ep["workload"], "tokens_per_step": ep["tokens_per_step"], "qtype": "q4_0",
                                                    "routing": routings[0], "parallelism": ep["parallelism"], "exchange": ep["exchange"],
                                                    "l2": L2_NOTE},
                    "e2e": first.get("e2e"), "gpu_launches": first["gpu_launches_per_step"] * args.steps, "roofline": first["roofline"],
                    "clocks": clocks, "ep": ep}
            if not args.no_cpu_baseline:
                from oracle import oracle as orc
                L, hidden, resid = synth_token_layer(w["seed"], 1024)
                cps, ckind, sample = cpu_tokens_per_s(L, hidden, resid, orc.host_threads())
                line["cpu_baseline"] = {"value": cps, "unit": "tokens/s", "cores": orc.host_threads(), "kind": ckind, "sample": sample}
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
