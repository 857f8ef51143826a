#!/usr/bin/env python
"""Benchmark of the GDN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one chunked prefill of the Qwen3-Next GDN layer workload (B=1 per GPU, T=8192, 16 key / 32 value
heads, d=128, bf16 q/k/v/z, fp32 g/beta, fused gated RMSNorm, fp32 final state).  With N GPUs every rank owns
one such sequence (the path is partitioned by (sequence, value head); there is no collective in the
recurrence), so the job is N sequences and `value` is their total tokens per second: weak scaling.  Under
torchrun each rank reads RANK/LOCAL_RANK/WORLD_SIZE; rank 0 prints ONE JSON line.

Extra objects on the same line: `decode` (continuous-batch decode step over a 512-slot fp32 state pool: state
GB/s against the HBM roofline), `roofline`, `cpu_baseline`, `e2e`, `clocks`.
`--impl reference` times the CPU restatement of the recurrence on the host cores instead (the reference
project has no implementation of this path, so the restatement is the only CPU arm there is).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FLOP_PER_CHUNK_HEAD = 10_485_760  # 8 dense contractions of the chunked form, K K^T and Q K^T shared by 2 value heads
T_PREFILL, HK, HV, D = 8192, 16, 32, 128


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "10"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, warmup, world, flush):
    """W untimed warm-ups, then K steps each bracketed by its own CUDA event pair on the launching stream,
    with an L2 flush (untimed) between them; returns total milliseconds of the K steps."""
    for _ in range(warmup):
        fn()
    barrier(world)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush.add_(1.0)  # 256 MiB write: larger than the 126 MB L2
        a.record()
        fn()
        b.record()
    barrier(world)
    return sum(a.elapsed_time(b) for a, b in evs)


def bench_prefill(args, rank, world):
    from avelang_b200 import gdn, synth
    inp = synth.config1(seed=rank)
    g = inp.to("cuda")
    out = torch.empty_like(g.v)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")

    def step():
        return gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, output_final_state=True, z=g.z, out=out)

    with ClockSampler(torch.cuda.current_device()) as clocks:
        total_ms = time_steps(step, args.steps, args.warmup, world, flush)
    total_ms = max_over_ranks(total_ms, world)
    ms = total_ms / args.steps

    # end to end: pinned host buffers -> device -> kernel -> host, every step.  The three legs run on their own streams
    # with double-buffered device tensors, so the copy-in of step i+1 and the copy-out of step i-1 overlap the kernels of
    # step i (PCIe is full duplex); every step still moves all of its inputs and results inside the timed region.
    host = {k: getattr(inp, k).pin_memory() for k in ("q", "k", "v", "z", "g", "beta")}
    dev = [{k: torch.empty_like(getattr(g, k)) for k in host} for _ in range(2)]
    outs = [torch.empty_like(g.v) for _ in range(2)]
    o_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    s_host = torch.empty(1, HV, D, D, dtype=torch.float32).pin_memory()
    s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    states = [None, None]

    def e2e_run(n_steps):
        for i in range(n_steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[b])          # the kernels that read this buffer two steps ago are done
                for k in host:
                    dev[b][k].copy_(host[k], non_blocking=True)
                ev_in[b].record(s_in)
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])             # the copy-out of the result that lived in outs[b] is done
            o, st = gdn.chunk_gated_delta_rule(dev[b]["q"], dev[b]["k"], dev[b]["v"], dev[b]["g"], dev[b]["beta"],
                                               output_final_state=True, z=dev[b]["z"], out=outs[b])
            states[b] = st
            ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                o_host.copy_(o, non_blocking=True)
                s_host.copy_(st, non_blocking=True)
                ev_out[b].record(s_out)
        s_cmp.wait_stream(s_out)
        s_cmp.wait_stream(s_in)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_run(2)
    barrier(world)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_run(e2e_steps)
    t1.record()
    barrier(world)
    e2e_ms = max_over_ranks(t0.elapsed_time(t1) / e2e_steps, world)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = o_host.numel() * o_host.element_size() + s_host.numel() * s_host.element_size()
    return ms, clocks.summary(), e2e_ms, h2d, d2h


def bench_decode(steps=1000, warmup=20):
    """256 sequences x 32 heads, one token each, state pool of 512 fp32 slots updated in place; a ring of 8
    pre-generated q/k/v/g/beta sets so the small inputs are not replayed from cache."""
    from avelang_b200 import gdn, synth
    base = synth.config2().to("cuda")
    ring = [synth.config2(seed=100 + i).to("cuda") for i in range(8)]
    pool, idx = base.state_pool, base.state_indices
    out = torch.empty_like(base.v)

    def step(i):
        r = ring[i % 8]
        gdn.fused_recurrent_gated_delta_rule(r.q, r.k, r.v, r.g, r.beta, initial_state=pool, state_indices=idx, out=out)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        step(i)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / steps
    state_bytes = 256 * HV * D * D * 4 * 2
    other = 256 * (HK * D * 2 * 2 + HV * D * 2 * 2 + HV * 4 * 2 + 4)
    return us, state_bytes, state_bytes + other


def cpu_baseline(sample_tokens=T_PREFILL, reps=None, budget_s=12.0):
    """The C restatement of the token recurrence (fp32, OpenMP over sequence x head) on the host cores; repeated
    until about `budget_s` seconds of CPU work have been timed (or `reps` runs)."""
    from avelang_b200 import synth
    from oracle import c_oracle
    inp = synth.config1(T=sample_tokens)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cores = c_oracle.set_threads(cores) or 1  # all the cores this process may use, whatever OMP_NUM_THREADS the launcher set
    t = time.perf_counter()
    c_oracle.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, precision="f32")  # untimed warm-up
    if reps is None:
        reps = max(3, min(100, int(budget_s / max(time.perf_counter() - t, 1e-3))))
    times = []
    for _ in range(reps):
        t = time.perf_counter()
        c_oracle.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, precision="f32")
        times.append(time.perf_counter() - t)
    sec = statistics.median(times)
    return {"value": sample_tokens / sec, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"full workload (T={sample_tokens}, 32 value heads, d=128), fp32 token recurrence in C with "
                      f"OpenMP, median of {reps} runs, {sec:.3f} s each"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t = time.perf_counter()
    base = cpu_baseline(reps=max(3, args.steps))
    wall = time.perf_counter() - t
    line = {"impl": "reference", "metric": "gdn_prefill_tokens_per_s", "value": base["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * T_PREFILL / base["value"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": f"CPU restatement of the recurrence (the reference ships no GDN code); wall {wall:.1f} s"}
    print(json.dumps(line))


def workload_config(n):
    return {"workload": "qwen3-next-80b-a3b GDN layer chunked prefill, B=1 per GPU, T=8192, Hk=16, Hv=32, d=128, "
                        "chunk 64, bf16 q/k/v/z, fp32 g/beta, fused gated RMSNorm, fp32 final state",
            "global_batch": n, "seq_len": T_PREFILL, "parallelism": f"sequence-sharded x{n}, no collective",
            "l2": "256 MiB flush write before every timed step; inputs 272 MB > 126 MB L2"}


def bench_varlen(args, rank, world):
    """Packed varlen prefill (64 sequences, log-uniform lengths in [128, 16384], 262144 tokens, nonzero initial
    states, final states returned), value heads sharded Hv/G per rank, no collective: strong scaling."""
    from avelang_b200 import gdn, synth
    from avelang_b200.block import HeadShard
    inp = synth.config3()
    sh = HeadShard(rank, world, HK, HV)
    ks, vs = slice(sh.key_heads.start, sh.key_heads.stop), slice(sh.value_heads.start, sh.value_heads.stop)
    q, k, v = inp.q[:, :, ks].contiguous().cuda(), inp.k[:, :, ks].contiguous().cuda(), inp.v[:, :, vs].contiguous().cuda()
    g, beta = inp.g[:, :, vs].contiguous().cuda(), inp.beta[:, :, vs].contiguous().cuda()
    s0, cu = inp.initial_state[:, vs].contiguous().cuda(), inp.cu_seqlens.cuda()
    out = torch.empty_like(v)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    longest = max(inp.extras["lengths"])  # the host built the batch, so it knows the longest sequence
    step = lambda: gdn.chunk_gated_delta_rule(q, k, v, g, beta, initial_state=s0, output_final_state=True, cu_seqlens=cu, out=out,
                                              max_seqlen=longest)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        total_ms = max_over_ranks(time_steps(step, args.steps, args.warmup, world, flush), world)
    ms = total_ms / args.steps
    chunks = sum((n + 63) // 64 for n in inp.extras["lengths"])
    flops = chunks * HV * FLOP_PER_CHUNK_HEAD
    peaks = measured_peaks()
    tokens = int(inp.cu_seqlens[-1])
    achieved = flops / (ms * 1e-3) / 1e12
    return {"metric": "gdn_varlen_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 in / fp32 state and accumulate", "data": "synthetic",
            "config": {"workload": f"varlen packed prefill, 64 seqs, {tokens} tokens, {chunks} chunks, Hk=16, Hv=32, d=128, "
                                   "initial and final states", "parallelism": f"value heads sharded x{world}, no collective",
                       "l2": "256 MiB flush write before every timed step"},
            "gpu_launches": 3 * args.steps, "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"] * world, "unit": "TFLOP/s",
                         "frac": achieved / (peaks["bf16_tflops"] * world), "traffic": None,
                         "peak_source": peaks["source"] + " (burst) x n_gpus"}}


def bench_block(args, rank, world):
    """Full GDN block, B=4, T=32768, hidden 2048: in-projection, conv1d+SiLU, L2 norm, gate/beta, chunked delta rule,
    gated RMSNorm on this rank's heads, then the NCCL all-gather of head outputs: strong scaling."""
    from avelang_b200.block import GdnBlockShard
    B, T, hidden = 4, 32768, 2048
    gen = torch.Generator().manual_seed(0)
    n_out = 2 * HK * D + 2 * HV * D + 2 * HV
    w_in = (0.02 * torch.randn(n_out, hidden, generator=gen)).bfloat16()
    conv_w = (torch.randn(2 * HK * D + HV * D, 4, generator=gen) / 2).bfloat16()
    A_log = torch.rand(HV, generator=gen) * 2.7726
    dt_bias = 0.1 * torch.randn(HV, generator=gen)
    x = torch.randn(B, T, hidden, generator=gen).bfloat16().cuda()
    blk = GdnBlockShard(w_in, conv_w, A_log, dt_bias, torch.ones(D), Hk=HK, Hv=HV, dk=D, dv=D, rank=rank, world=world)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    fused = os.environ.get("AVE_GDN_FUSED_GATHER", "1") != "0"  # peer-store all-gather fused into the norm kernel
    step = lambda: blk.forward(x, fused_gather=fused)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        total_ms = max_over_ranks(time_steps(step, args.steps, args.warmup, world, flush), world)
    ms = total_ms / args.steps
    flops = 2 * B * T * hidden * n_out + (B * T // 64) * HV * FLOP_PER_CHUNK_HEAD
    peaks = measured_peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    return {"metric": "gdn_block_tokens_per_s", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "GDN block B=4 T=32768 hidden 2048: in-proj, conv1d k=4 + SiLU, L2 norm, gate/beta, "
                                   "chunked delta rule, gated RMSNorm, head all-gather",
                       "parallelism": f"heads sharded x{world}, " + ("all-gather fused into the norm kernel (peer stores)" if fused else "one NCCL all-gather"), "l2": "256 MiB flush write before every timed step"},
            "gpu_launches": 6 * args.steps, "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"] * world, "unit": "TFLOP/s",
                         "frac": achieved / (peaks["bf16_tflops_sustained"] * world), "traffic": None,
                         "peak_source": peaks["source"] + " (sustained) x n_gpus"}}


def profile_case(name: str):
    """Small fixed cases for profiler captures (a few launches, a few hundred MB on the device at most)."""
    from avelang_b200 import gdn, synth
    torch.cuda.set_device(0)
    if name == "decode":
        inp = synth.config2().to("cuda")
        for _ in range(3):
            gdn.fused_recurrent_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, initial_state=inp.state_pool,
                                                 state_indices=inp.state_indices)
    elif name == "prefill2048":
        inp = synth.config1(T=2048).to("cuda")
        for _ in range(2):
            gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, output_final_state=True, z=inp.z)
    elif name == "varlen32k":
        # throughput regime in the small: 64 packed sequences, about 550 chunks x 32 heads, 1.5 GB of scratch
        inp = synth.config3(total=32768, lo=128, hi=2048).to("cuda")
        for _ in range(2):
            gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, initial_state=inp.initial_state,
                                       output_final_state=True, cu_seqlens=inp.cu_seqlens)
    else:
        raise SystemExit(f"unknown profile case {name!r}")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "done": True}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "varlen", "block"],
                    help="prefill (default, the headline line), varlen (head-sharded packed prefill) or block")
    ap.add_argument("--profile-case", default=None, choices=["decode", "prefill2048", "varlen32k"],
                    help="run a small fixed case for a profiler capture and exit")
    args = ap.parse_args()
    if args.profile_case:
        return profile_case(args.profile_case)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    from avelang_b200 import _lib
    _lib.load()  # fail loudly when the CUDA library is missing
    rank, world, local = dist_setup(args.gpus)
    peaks = measured_peaks()
    if args.workload != "prefill":
        line = (bench_varlen if args.workload == "varlen" else bench_block)(args, rank, world)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    ms, clocks, e2e_ms, h2d, d2h = bench_prefill(args, rank, world)
    tokens = T_PREFILL * world
    flops = (T_PREFILL // 64) * HV * FLOP_PER_CHUNK_HEAD
    algo_bytes = 272_629_760
    line = {"metric": "gdn_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 in / fp32 state and accumulate", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": 12 * args.steps,  # four chunk ranges (8, 24, 72, 24 chunks) x (prep, scan, gated norm)
            "clocks": clocks}
    achieved = flops / (ms * 1e-3) / 1e12
    line["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": achieved / peaks["bf16_tflops"], "traffic": 471_699_248,
                        "traffic_source": "profiles/prefill_config1_launch_list.md: DRAM bytes read + written by the four "
                                          "chunk_scan launches of one step (the dominant kernel), ncu with its "
                                          "cache flush between kernels; algorithmic bytes of the step are in hbm_view",
                        "peak_source": peaks["source"] + " (burst)",
                        "note": "algorithmic 42.95 GFLOP per step over the whole step (all launches): a lower bound "
                                "for the dominant kernel",
                        "hbm_view": {"achieved_gbs": algo_bytes / (ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                                     "algorithmic_bytes": algo_bytes}}
    if rank == 0 and not args.no_decode:
        us, state_bytes, all_bytes = bench_decode()
        line["decode"] = {"metric": "gdn_decode_state_GBps", "value": state_bytes / (us * 1e-6) / 1e9, "unit": "GB/s",
                          "us_per_step": us, "steps": 1000,
                          "config": {"workload": "256 seqs x 32 value heads, T=1, 512-slot fp32 pool [128x128], in place"},
                          "roofline": {"bound": "hbm", "achieved": all_bytes / (us * 1e-6) / 1e9, "peak": peaks["hbm_gbs"],
                                       "unit": "GB/s", "frac": all_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"],
                                       "frac_of_nominal_8TBps": all_bytes / (us * 1e-6) / 8e12,
                                       "traffic": 1_020_755_968,  # dram read+write per launch, ncu capture at full size
                                       "traffic_source": "profiles/decode_gdn_decode_kernel_config2.md",
                                       "peak_source": peaks["source"]}}
    if world > 1:
        barrier(world)
    if rank == 0:
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
