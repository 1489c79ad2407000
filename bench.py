#!/usr/bin/env python3
"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode]

Prints ONE JSON line on rank 0.  The default workload is the full-size decode stack: one token through
11 stacked MoE layers (hidden 1280, 64 experts top-6 + shared 1792, FFN 896, Q4_0 group-64 weights,
seed 1), metric = microseconds per token.  A step is one pass of the token through the 11 layers.

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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode"])
    ap.add_argument("--cpu-layers", type=int, default=2, help="layers of the stack the CPU baseline samples")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    entry.build() if not (entry.PKG_DIR / "libuocr_cuda_moe.so").exists() else None
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
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush_reader = torch.empty(256 << 20, dtype=torch.uint8, device="cuda").view(torch.int32)

    def flush_l2(i: int):
        # write a buffer larger than L2, then read a second one through the cache so that the weights are
        # cold AND the cache is not left full of dirty lines whose write-back would compete with the step
        flush.fill_(i & 0xFF)
        flush_reader.max()

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
            "roofline": {"bound": "hbm", "kernel": "decode stack (all kernels of one step)", "achieved": achieved,
                         "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "algorithmic_bytes_per_step": step_bytes,
                         "traffic": None},
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
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
