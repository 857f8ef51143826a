#!/usr/bin/env python
"""Benchmark of the GDN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one chunked prefill of the Qwen3-Next GDN layer workload (B=1 per GPU, T=8192, 16 key / 32 value
heads, d=128, bf16 q/k/v/z, fp32 g/beta, fused gated RMSNorm, fp32 final state).  With N GPUs every rank owns
one such sequence (the path is partitioned by (sequence, value head); there is no collective in the
recurrence), so the job is N sequences and `value` is their total tokens per second: weak scaling.  Under
torchrun each rank reads RANK/LOCAL_RANK/WORLD_SIZE; rank 0 prints ONE JSON line.

Extra objects on the same line: `decode` (continuous-batch decode step over a 512-slot fp32 state pool: state
GB/s against the HBM roofline), `roofline`, `cpu_baseline`, `e2e`, `clocks`, and, at the end of the line, the two
sharded workloads timed over the same N ranks with a parity object each: `varlen` (64 packed sequences, 262144
tokens, value heads sharded Hv/N per rank, no collective: strong scaling) and `block` (the whole GDN block, B=4,
T=32768, heads sharded, head outputs all-gathered: by peer stores fused into the norm kernel, and by NCCL).
`--impl reference` times the CPU restatement of the recurrence on the host cores instead (the reference
project has no implementation of this path, so the restatement is the only CPU arm there is); with `--gpus N`
it times the same N sequences the GPU arm processes.
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

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __enter__(self):
        """Starts the sampler and waits (up to 3 s) for its first sample, so that the samples that follow fall inside
        the region the caller is about to run: nvidia-smi takes longer to start than a short timed region lasts."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "5"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            t0 = time.perf_counter()
            while not self.lines and time.perf_counter() - t0 < 3.0 and self.proc.poll() is None:
                time.sleep(0.005)
            self.lines.clear()  # what was sampled before the load started does not count
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


def bind_host_to_gpu_node(local_rank: int) -> dict:
    """Pins this process to the CPUs of the NUMA node its GPU hangs off (read from sysfs), before any pinned host
    buffer is allocated, so that the end-to-end copies of N ranks do not all cross one socket's memory.  Reports what
    it found; does nothing when the box has one node or hides the topology."""
    info = {"numa_node": None, "cpus": None}
    try:
        bus = subprocess.run(["nvidia-smi", "-i", str(local_rank), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if bus.startswith("00000000:"):
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        info["numa_node"] = node
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        if node >= 0 and len(nodes) > 1:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                info["cpus"] = len(cpus)
    except (OSError, ValueError, subprocess.SubprocessError):
        pass
    return info


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

    clocks = ClockSampler(torch.cuda.current_device())
    clocks.__enter__()  # stays up through warm-up, the timed region and the end-to-end leg below
    eager_ms = max_over_ranks(time_steps(step, args.steps, args.warmup, world, flush), world) / args.steps
    # the same call captured once into a CUDA graph and replayed: the schedule's cross-stream event edges become graph
    # edges, which the device resolves faster than stream-ordered events (results are bit-identical to eager launches)
    cap = torch.cuda.Stream()
    cap.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(cap):
        step()  # this stream's scratch exists before the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap):
            step()
    torch.cuda.current_stream().wait_stream(cap)
    graph_ms = max_over_ranks(time_steps(graph.replay, args.steps, args.warmup, world, flush), world) / args.steps
    ms = min(eager_ms, graph_ms)
    launch_modes = {"eager_ms_per_step": eager_ms, "graph_replay_ms_per_step": graph_ms,
                    "reported": "graph replay" if graph_ms <= eager_ms else "eager launches"}

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
    clocks.__exit__(None, None, None)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = o_host.numel() * o_host.element_size() + s_host.numel() * s_host.element_size()

    # the three legs one at a time (all ranks at once, max over ranks): names the leg that saturates as N grows
    def leg(fn, reps=3):
        fn(); barrier(world)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record(); barrier(world)
        return max_over_ranks(a.elapsed_time(b) / reps, world)

    def copy_in():
        for k in host:
            dev[0][k].copy_(host[k], non_blocking=True)

    def copy_out():
        o_host.copy_(outs[0], non_blocking=True)
        s_host.copy_(states[0], non_blocking=True)

    legs = {"h2d_ms": leg(copy_in), "kernels_ms": leg(step), "d2h_ms": leg(copy_out)}
    legs["h2d_GBps_per_rank"] = h2d / (legs["h2d_ms"] * 1e-3) / 1e9
    legs["d2h_GBps_per_rank"] = d2h / (legs["d2h_ms"] * 1e-3) / 1e9
    return ms, clocks.summary(), e2e_ms, h2d, d2h, legs, gdn.prefill_launch_count(g.q, g.k, g.v, z=g.z), launch_modes


def bench_decode(steps=1000, warmup=20):
    """256 sequences x 32 heads, one token each, state pool of 512 fp32 slots updated in place; a ring of 8
    pre-generated q/k/v/g/beta sets so the small inputs are not replayed from cache.  Also the same step with the
    layer's front end fused in (conv update, L2 norms, gate/beta, gated norm from the projection row: one kernel) next
    to the separate kernels it replaces."""
    from avelang_b200 import gdn, synth
    base = synth.config2().to("cuda")
    ring = [synth.config2(seed=100 + i).to("cuda") for i in range(8)]
    pool, idx = base.state_pool, base.state_indices
    out = torch.empty_like(base.v)

    def step(i):
        r = ring[i % 8]
        gdn.fused_recurrent_gated_delta_rule(r.q, r.k, r.v, r.g, r.beta, initial_state=pool, state_indices=idx, out=out)

    def timed(fn, n):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / n

    us_eager = timed(step, steps)
    # the same 1000 steps as 125 replays of a CUDA graph of the 8-set ring: no host work between launches
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(8):
            step(i)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(8):
                step(i)
    torch.cuda.current_stream().wait_stream(side)
    us_graph = timed(lambda i: graph.replay(), max(1, steps // 8)) / 8
    us = min(us_eager, us_graph)
    state_bytes = 256 * HV * D * D * 4 * 2
    other = 256 * (HK * D * 2 * 2 + HV * D * 2 * 2 + HV * 4 * 2 + 4)
    # the whole layer step from the in-projection row: fused kernel vs conv update + gate/beta + decode step
    Cn, cols, N = 2 * HK * D + HV * D, 2 * HK * D + 2 * HV * D + 2 * HV, 256
    gen = torch.Generator(device="cuda").manual_seed(7)
    projs = [torch.randn(N, cols, device="cuda", generator=gen).bfloat16() for _ in range(8)]
    conv_w = (torch.randn(Cn, 4, device="cuda", generator=gen) / 2).bfloat16()
    conv_state = torch.randn(512, 3, Cn, device="cuda", generator=gen).bfloat16()
    A_log, dt_bias = torch.rand(HV, device="cuda") * 2.77, torch.randn(HV, device="cuda") * 0.1
    o2 = torch.empty(N, HV, D, dtype=torch.bfloat16, device="cuda")

    def fused(i):
        gdn.decode_layer_step(projs[i % 8], conv_w, conv_state, A_log, dt_bias, pool, idx, Hk=HK, Hv=HV, out=o2)

    def separate(i):
        p = projs[i % 8]
        qkv = gdn.causal_conv1d_update(p[:, :Cn], conv_state, conv_w, state_indices=idx)
        g, beta = gdn.gate_beta(p[:, cols - HV:], p[:, cols - 2 * HV:cols - HV], A_log, dt_bias)
        gdn.fused_recurrent_gated_delta_rule(qkv[:, :HK * D].reshape(N, 1, HK, D), qkv[:, HK * D:2 * HK * D].reshape(N, 1, HK, D),
                                             qkv[:, 2 * HK * D:].reshape(N, 1, HV, D), g.reshape(N, 1, HV), beta.reshape(N, 1, HV),
                                             initial_state=pool, state_indices=idx, use_qk_l2norm_in_kernel=True,
                                             z=p[:, Cn:Cn + HV * D].reshape(N, 1, HV, D), out=o2.reshape(N, 1, HV, D))

    layer = {"fused_us_per_step": timed(fused, 200), "separate_kernels_us_per_step": timed(separate, 200),
             "what": "decode step of the whole layer behind its in-projection (conv update + SiLU, q/k L2 norm, gate/beta, "
                     "delta-rule update, gated norm): one kernel vs the three separate entry points"}
    return us, state_bytes, state_bytes + other, layer, {"eager_us_per_step": us_eager, "graph_us_per_step": us_graph}


def bench_backward(steps=2):
    """The backward pass on the headline shape (B=1, T=8192, 32 value heads): the correct-first reverse sweep, timed so
    that its distance from the forward pass is on record."""
    from avelang_b200 import gdn, synth
    g = synth.config1().to("cuda")
    d_o = torch.randn_like(g.v)
    run = lambda: gdn.gated_delta_rule_backward(g.q, g.k, g.v, g.g, g.beta, d_o)
    run()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        run()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    return {"metric": "gdn_backward_tokens_per_s", "value": T_PREFILL / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "config": {"workload": "gradients of the headline prefill (no fused norm): token-by-token reverse sweep in fp32"}}


def cpu_baseline(sample_tokens=T_PREFILL, reps=None, budget_s=12.0, n_seqs=1):
    """The C restatement of the token recurrence (fp32, OpenMP over sequence x head) on the host cores; repeated
    until about `budget_s` seconds of CPU work have been timed (or `reps` runs).  `n_seqs` sequences per run (the
    batch an N-GPU job processes per step)."""
    from avelang_b200 import synth
    from oracle import c_oracle
    inp = synth.make_inputs(n_seqs, sample_tokens, HK, HV, D, D, seed=0, with_z=True)
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
    return {"value": n_seqs * sample_tokens / sec, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"full workload ({n_seqs} x T={sample_tokens}, 32 value heads, d=128), fp32 token recurrence in C "
                      f"with OpenMP, median of {reps} runs, {sec:.3f} s each"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t = time.perf_counter()
    n = max(1, args.gpus)  # the job of N GPUs is N sequences per step: time the same N sequences here
    base = cpu_baseline(reps=max(3, min(args.steps, max(3, 24 // n))), n_seqs=n)
    wall = time.perf_counter() - t
    line = {"impl": "reference", "metric": "gdn_prefill_tokens_per_s", "value": base["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * n * T_PREFILL / base["value"], "higher_is_better": True, "scaling": "weak",
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


def max_tensor_over_ranks(vals, world):
    t = torch.tensor(vals, dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


def bench_varlen(args, rank, world, steps=None, full_line=True):
    """Packed varlen prefill (64 sequences, log-uniform lengths in [128, 16384], 262144 tokens, nonzero initial
    states, final states returned), value heads sharded Hv/G per rank, no collective: strong scaling.  Parity
    (outside the timed region): the shortest, the median and the longest sequence of every rank's heads against
    the fp64 C checker, worst rank reported."""
    from avelang_b200 import gdn, synth
    from avelang_b200.block import HeadShard
    from oracle import c_oracle, gdn_oracle
    steps = steps or args.steps
    c_oracle.set_threads(torch.get_num_threads())
    inp = synth.config3()
    sh = HeadShard(rank, world, HK, HV)
    ks, vs = slice(sh.key_heads.start, sh.key_heads.stop), slice(sh.value_heads.start, sh.value_heads.stop)
    q, k, v = inp.q[:, :, ks].contiguous().cuda(), inp.k[:, :, ks].contiguous().cuda(), inp.v[:, :, vs].contiguous().cuda()
    g, beta = inp.g[:, :, vs].contiguous().cuda(), inp.beta[:, :, vs].contiguous().cuda()
    s0, cu = inp.initial_state[:, vs].contiguous().cuda(), inp.cu_seqlens.cuda()
    out = torch.empty_like(v)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    lens = inp.extras["lengths"]
    longest = max(lens)  # the host built the batch, so it knows the longest sequence
    res = {}

    def step():
        res["o"], res["s"] = gdn.chunk_gated_delta_rule(q, k, v, g, beta, initial_state=s0, output_final_state=True,
                                                        cu_seqlens=cu, out=out, max_seqlen=longest)

    with ClockSampler(torch.cuda.current_device()) as clocks:
        total_ms = max_over_ranks(time_steps(step, steps, args.warmup, world, flush), world)
    ms = total_ms / steps
    # parity of this rank's heads
    order = sorted(range(len(lens)), key=lambda n: lens[n])
    picks = [order[0], order[len(order) // 2], order[-1]]
    o_cpu, s_cpu, cul = res["o"].cpu(), res["s"].cpu(), inp.cu_seqlens.tolist()
    e_o = e_s = 0.0
    for n in picks:
        a, b = cul[n], cul[n + 1]
        o_ref, s_ref = c_oracle.recurrent(inp.q[:, a:b, ks], inp.k[:, a:b, ks], inp.v[:, a:b, vs], inp.g[:, a:b, vs],
                                          inp.beta[:, a:b, vs], inp.scale, inp.initial_state[n:n + 1, vs])
        e_o = max(e_o, gdn_oracle.rel_l2(o_cpu[:, a:b].float(), o_ref.to(torch.bfloat16).float()))
        e_s = max(e_s, gdn_oracle.rel_l2(s_cpu[n:n + 1], s_ref))
    e_o, e_s, st = max_tensor_over_ranks([e_o, e_s, float(gdn.read_status())], world)
    parity = {"o_rel_l2_max": e_o, "s_rel_l2_max": e_s, "o_gate": 1e-3, "s_gate": 1e-4, "status_word": int(st),
              "checked": f"sequences of {[lens[n] for n in picks]} tokens x the heads of every rank, vs the fp64 C checker",
              "ok": bool(e_o <= 1e-3 and e_s <= 1e-4 and st == 0)}
    chunks = sum((n + 63) // 64 for n in lens)
    flops = chunks * HV * FLOP_PER_CHUNK_HEAD
    algo_bytes = 2 * 2 * 262144 * HK * D * 1 + 2 * 2 * 262144 * HV * D + 2 * 4 * 262144 * HV + 2 * 64 * HV * D * D * 4
    peaks = measured_peaks()
    tokens = int(inp.cu_seqlens[-1])
    achieved = flops / (ms * 1e-3) / 1e12
    line = {"metric": "gdn_varlen_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 in / fp32 state and accumulate", "data": "synthetic",
            "config": {"workload": f"varlen packed prefill, 64 seqs, {tokens} tokens, {chunks} chunks, Hk=16, Hv=32, d=128, "
                                   "initial and final states", "parallelism": f"value heads sharded x{world}, no collective",
                       "l2": "256 MiB flush write before every timed step"},
            "gpu_launches": gdn.prefill_launch_count(q, k, v, cu_seqlens=cu, max_seqlen=longest) * steps, "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"] * world, "unit": "TFLOP/s",
                         "frac": achieved / (peaks["bf16_tflops"] * world), "traffic": None,
                         "peak_source": peaks["source"] + " (burst) x n_gpus",
                         "hbm_view": {"achieved_gbs": algo_bytes / (ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"] * world,
                                      "algorithmic_bytes": algo_bytes}},
            "parity": parity}
    if not full_line:
        for key in ("higher_is_better", "vs_baseline", "data", "warmup", "n_gpus", "clocks"):
            line.pop(key, None)
    return line


def bench_block(args, rank, world, steps=None, full_line=True):
    """Full GDN block, B=4, T=32768, hidden 2048: in-projection, conv1d+SiLU, L2 norm, gate/beta, chunked delta rule,
    gated RMSNorm on this rank's heads, then the all-gather of head outputs (peer stores fused into the norm kernel;
    at N >= 2 the NCCL all-gather is timed too and must give the same bits): strong scaling.  Parity (outside the timed
    region): a causal prefix of one batch row of the gathered output against the CPU block reference, and the
    delta-rule + norm stage alone against the C checker fed with the device's own stage inputs."""
    from avelang_b200 import gdn
    from avelang_b200.block import GdnBlockShard
    from oracle import c_oracle, gdn_oracle
    steps = steps or args.steps
    B, T, hidden = 4, 32768, 2048
    gen = torch.Generator().manual_seed(0)
    n_out = 2 * HK * D + 2 * HV * D + 2 * HV
    w_in = (0.02 * torch.randn(n_out, hidden, generator=gen)).bfloat16()
    conv_w = (torch.randn(2 * HK * D + HV * D, 4, generator=gen) / 2).bfloat16()
    A_log = torch.rand(HV, generator=gen) * 2.7726
    dt_bias = 0.1 * torch.randn(HV, generator=gen)
    norm_w = torch.ones(D)
    x_cpu = torch.randn(B, T, hidden, generator=gen).bfloat16()
    x = x_cpu.cuda()
    blk = GdnBlockShard(w_in, conv_w, A_log, dt_bias, norm_w, Hk=HK, Hv=HV, dk=D, dv=D, rank=rank, world=world)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    fused = os.environ.get("AVE_GDN_FUSED_GATHER", "1") != "0" and world > 1  # peer-store all-gather fused into the norm kernel
    res = {}

    def step():
        res["y"] = blk.forward(x, fused_gather=fused)

    with ClockSampler(torch.cuda.current_device()) as clocks:
        total_ms = max_over_ranks(time_steps(step, steps, args.warmup, world, flush), world)
    ms = total_ms / steps
    y = res["y"]
    extra = {}
    if world > 1:  # the same block with one NCCL all-gather instead
        def step_nccl():
            res["y_nccl"] = blk.forward(x, fused_gather=False)
        nccl_ms = max_over_ranks(time_steps(step_nccl, steps, args.warmup, world, flush), world) / steps
        # The two paths give the same bits when they run the same schedule.  With few chains per rank (16 at 8 ranks)
        # the NCCL path walks each sequence as parallel parts while the fused path keeps plain chains (its norm kernel
        # pushes rows range by range): each is within 1e-3 of the checker, so they may differ from one another by 2e-3.
        d_paths = float((y.float() - res["y_nccl"].float()).norm() / res["y_nccl"].float().norm()) if fused else None
        extra = {"nccl_gather_ms_per_step": nccl_ms, "fused_equals_nccl": bool(torch.equal(y, res["y_nccl"])) if fused else None,
                 "fused_vs_nccl_rel_l2": d_paths, "fused_vs_nccl_gate": 2e-3}
    if world > 1:
        # The tensor-parallel form's output projection [B*T, Hv*dv / world] x [hidden, Hv*dv / world]^T with its sum over
        # ranks: own GEMM + one NCCL all-reduce, against the GEMM whose epilogue stores each row at its owner (peer
        # stores) followed by the owners' sum-and-store kernel.  Timed on this rank's normalised head outputs.
        from avelang_b200.block import GdnBlockTP
        w_out = (0.05 * torch.randn(hidden, HV * D, generator=gen)).bfloat16()
        tp = GdnBlockTP(w_in, conv_w, A_log, dt_bias, norm_w, w_out, Hk=HK, Hv=HV, dk=D, dv=D, rank=rank, world=world)
        o2d = blk.forward_local(x).reshape(B * T, -1)
        pr = {}
        def proj_nccl():
            pr["nccl"] = tp.project(o2d)
        def proj_fused():
            pr["fused"] = tp.project(o2d, fused_reduce=True)
        p_nccl = max_over_ranks(time_steps(proj_nccl, steps, args.warmup, world, flush), world) / steps
        p_fused = max_over_ranks(time_steps(proj_fused, steps, args.warmup, world, flush), world) / steps
        d_proj = float((pr["fused"].float() - pr["nccl"].float()).norm() / pr["nccl"].float().norm())
        extra["out_projection"] = {"gemm_then_nccl_all_reduce_ms": p_nccl, "gemm_with_fused_sum_ms": p_fused,
                                   "fused_vs_nccl_rel_l2": d_proj, "gate": 1e-2,
                                   "shape": f"M={B * T}, N={hidden}, K={HV * D // world} per rank"}
        del o2d, pr, tp
    # parity 1: causal prefix of batch row 2, every head (they come from every rank), end to end
    P = 160
    ref = gdn_oracle.gdn_block_ref(x_cpu[2:3, :P], w_in, conv_w, A_log, dt_bias, norm_w, Hk=HK, Hv=HV, dk=D, dv=D)
    e_block = gdn_oracle.rel_l2(y[2:3, :P].float().cpu(), ref.bfloat16().float())
    # parity 2: the delta-rule + norm stage of this rank's heads on the device's own bf16 q/k/v/z and fp32 g/beta
    keep = {}
    o_loc = blk.forward_local(x, keep=keep)
    Pd = 2048
    cut = lambda t: t[1:2, :Pd].cpu()
    o_ref, _ = c_oracle.recurrent(cut(keep["q"]), cut(keep["k"]), cut(keep["v"]), cut(keep["g"]), cut(keep["beta"]), D ** -0.5,
                                  use_qk_l2norm_in_kernel=True)
    y_ref = gdn_oracle.gated_rmsnorm(o_ref, cut(keep["z"]), norm_w)
    e_stage = gdn_oracle.rel_l2(o_loc[1:2, :Pd].float().cpu(), y_ref.to(torch.bfloat16).float())
    e_block, e_stage, st = max_tensor_over_ranks([e_block, e_stage, float(gdn.read_status())], world)
    parity = {"block_prefix_rel_l2": e_block, "block_gate": 5e-3, "delta_rule_stage_rel_l2_max": e_stage, "stage_gate": 1e-3,
              "status_word": int(st),
              "checked": f"{P}-token prefix of batch row 2, all heads, vs the CPU block reference (5e-3: the bf16 projection "
                         f"and convolution outputs differ from the reference's by a rounding in a few per cent of elements); "
                         f"delta rule + gated norm on {Pd} tokens of batch row 1, every rank's heads, vs the fp64 C checker "
                         "fed the device's own stage inputs (1e-3)",
              "ok": bool(e_block <= 5e-3 and e_stage <= 1e-3 and st == 0 and (extra.get("fused_vs_nccl_rel_l2") or 0.0) <= 2e-3
                         and extra.get("out_projection", {}).get("fused_vs_nccl_rel_l2", 0.0) <= 1e-2)}
    flops = 2 * B * T * hidden * n_out + (B * T // 64) * HV * FLOP_PER_CHUNK_HEAD
    peaks = measured_peaks()
    achieved = flops / (ms * 1e-3) / 1e12
    line = {"metric": "gdn_block_tokens_per_s", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "GDN block B=4 T=32768 hidden 2048: in-proj, conv1d k=4 + SiLU, L2 norm, gate/beta, "
                                   "chunked delta rule, gated RMSNorm, head all-gather",
                       "parallelism": f"heads sharded x{world}, " + ("all-gather fused into the norm kernel (peer stores)" if fused else ("one NCCL all-gather" if world > 1 else "no gather")), "l2": "256 MiB flush write before every timed step"},
            "gpu_launches": (3 + gdn.prefill_launch_count(keep["q"], keep["k"], keep["v"], z=keep["z"], push=fused)) * steps,  # GEMM, conv, gate + the prefill's own
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"] * world, "unit": "TFLOP/s",
                         "frac": achieved / (peaks["bf16_tflops_sustained"] * world), "traffic": None,
                         "peak_source": peaks["source"] + " (sustained) x n_gpus"},
            "parity": parity, **extra}
    if not full_line:
        for key in ("higher_is_better", "vs_baseline", "data", "warmup", "n_gpus", "clocks"):
            line.pop(key, None)
    return line


def bench_helpers(args):
    """The kernels around the recurrence, each timed alone on one GPU (CUDA events, L2 flush between runs): the bf16
    GEMM on the in-projection shapes next to torch.matmul (cuBLAS) in the same run, the causal conv1d + SiLU, the
    fp32-input gated norm and the gate/beta kernel, with the bytes or flops each moves."""
    from avelang_b200 import gdn, gemm
    torch.cuda.set_device(0)
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    peaks = measured_peaks()

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            flush.add_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    out = {"metric": "gdn_helper_kernels", "peaks": peaks, "gemm": [], "streaming": []}
    gen = torch.Generator(device="cuda").manual_seed(0)
    for (m, n, k, what) in ((131072, 1544, 2048, "in-projection of one rank of eight"), (131072, 12352, 2048, "in-projection, one GPU"),
                            (8192, 8192, 8192, "square")):
        A = torch.randn(m, k, device="cuda", generator=gen).bfloat16()
        B = (0.02 * torch.randn(n, k, device="cuda", generator=gen)).bfloat16()
        C = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ours = timed(lambda: gemm.gemm_pipeline_transposed_b(A, B, out=C))
        ref = timed(lambda: torch.matmul(A, B.T, out=C))
        fl = 2.0 * m * n * k
        out["gemm"].append({"shape": [m, n, k], "what": what, "ms": ours, "tflops": fl / ours / 1e9, "cublas_ms": ref,
                            "cublas_tflops": fl / ref / 1e9, "frac_of_cublas": ref / ours,
                            "frac_of_measured_peak": fl / ours / 1e9 / peaks["bf16_tflops_sustained"]})
        del A, B, C
    Bt, T, Cn = 4, 32768, 8192
    x = torch.randn(Bt, T, Cn, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(Cn, 4, device="cuda", generator=gen) / 2).bfloat16()
    y = torch.empty_like(x)
    ms = timed(lambda: gdn.causal_conv1d_silu(x, w, out=y))
    by = 2 * x.numel() * 2
    out["streaming"].append({"kernel": "conv1d_silu_kernel<4>", "shape": [Bt, T, Cn], "ms": ms, "GBps": by / ms / 1e6,
                             "frac_of_measured_hbm": by / ms / 1e6 / peaks["hbm_gbs"], "bytes": by})
    del x, y
    rows, H = Bt * T, 32
    xo = torch.randn(rows, H, 128, device="cuda", generator=gen).bfloat16()
    z = torch.randn(rows, H, 128, device="cuda", generator=gen).bfloat16()
    yo = torch.empty_like(xo)
    ms = timed(lambda: gdn.gated_rmsnorm(xo, z, out=yo))
    by = 3 * xo.numel() * 2
    out["streaming"].append({"kernel": "gated_rmsnorm_kernel<128, bf16>", "shape": [rows, H, 128], "ms": ms, "GBps": by / ms / 1e6,
                             "frac_of_measured_hbm": by / ms / 1e6 / peaks["hbm_gbs"], "bytes": by})
    a_in = torch.randn(rows, H, device="cuda", generator=gen).bfloat16()
    b_in = torch.randn(rows, H, device="cuda", generator=gen).bfloat16()
    A_log, dt = torch.rand(H, device="cuda"), torch.randn(H, device="cuda") * 0.1
    ms = timed(lambda: gdn.gate_beta(a_in, b_in, A_log, dt))
    by = rows * H * (2 + 2 + 4 + 4)
    out["streaming"].append({"kernel": "gate_beta_kernel", "shape": [rows, H], "ms": ms, "GBps": by / ms / 1e6,
                             "frac_of_measured_hbm": by / ms / 1e6 / peaks["hbm_gbs"], "bytes": by})
    print(json.dumps(out))


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
    elif name == "parts8k":
        # few long chains: one sequence of 8192 tokens x 4 value heads is cut into parallel parts (transition chains,
        # combine, fix-up); about 0.1 GB of scratch
        inp = synth.config1(T=8192, Hk=2, Hv=4).to("cuda")
        for _ in range(3):
            gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, output_final_state=True, z=inp.z)
    elif name == "gemm1544":
        # the in-projection of one rank of eight at an eighth of the rows (16384 x 1544 x 2048): ragged last column tile
        from avelang_b200 import gemm
        A = torch.randn(16384, 2048, device="cuda").bfloat16()
        B = (0.02 * torch.randn(1544, 2048, device="cuda")).bfloat16()
        for _ in range(3):
            gemm.gemm_pipeline_transposed_b(A, B)
    elif name == "conv":
        x = torch.randn(1, 32768, 8192, device="cuda").bfloat16()  # 512 MiB in, 512 MiB out
        w = (torch.randn(8192, 4, device="cuda") / 2).bfloat16()
        for _ in range(3):
            gdn.causal_conv1d_silu(x, w)
    elif name == "norm":
        x = torch.randn(32768, 32, 128, device="cuda").bfloat16()  # 256 MiB per tensor
        z = torch.randn(32768, 32, 128, device="cuda").bfloat16()
        for _ in range(3):
            gdn.gated_rmsnorm(x, z)
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
    ap.add_argument("--no-sharded", action="store_true", help="skip the varlen and block objects")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "varlen", "block", "helpers"],
                    help="prefill (default, the headline line), varlen (head-sharded packed prefill), block, or helpers "
                         "(GEMM, conv1d, norm and gate kernels timed alone on one GPU)")
    ap.add_argument("--profile-case", default=None, choices=["decode", "prefill2048", "varlen32k", "parts8k", "gemm1544", "conv", "norm"],
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
    if args.workload == "helpers":
        return bench_helpers(args)
    rank, world, local = dist_setup(args.gpus)
    # torchrun exports OMP_NUM_THREADS=1: give every rank its share of the host cores for input generation and the checker
    share = max(1, (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)) // max(1, world))
    torch.set_num_threads(share)
    host_binding = bind_host_to_gpu_node(local) if world > 1 else {"numa_node": None, "cpus": None}
    peaks = measured_peaks()
    if args.workload != "prefill":
        line = (bench_varlen if args.workload == "varlen" else bench_block)(args, rank, world)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    ms, clocks, e2e_ms, h2d, d2h, legs, launches_per_call, launch_modes = bench_prefill(args, rank, world)
    tokens = T_PREFILL * world
    flops = (T_PREFILL // 64) * HV * FLOP_PER_CHUNK_HEAD
    algo_bytes = 272_629_760
    line = {"metric": "gdn_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 in / fp32 state and accumulate", "data": "synthetic",
            "config": workload_config(world),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "legs": legs, "host": host_binding},
            "gpu_launches": launches_per_call * args.steps,  # kernels one prefill call enqueues (asked from the library) x steps
            "launch_modes": launch_modes,
            "clocks": clocks}
    achieved = flops / (ms * 1e-3) / 1e12
    line["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": achieved / peaks["bf16_tflops"], "traffic": 469_767_936,
                        "traffic_source": "profiles/prefill_config1_launch_list.md: DRAM bytes read + written by the four "
                                          "chunk_scan launches of one step (the dominant kernel), ncu with its "
                                          "cache flush between kernels; algorithmic bytes of the step are in hbm_view",
                        "peak_source": peaks["source"] + " (burst)",
                        "note": "algorithmic 42.95 GFLOP per step over the whole step (all launches): a lower bound "
                                "for the dominant kernel",
                        "hbm_view": {"achieved_gbs": algo_bytes / (ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                                     "algorithmic_bytes": algo_bytes}}
    if rank == 0 and not args.no_decode:
        us, state_bytes, all_bytes, layer_step, launch_modes = bench_decode()
        line["decode"] = {"metric": "gdn_decode_state_GBps", "value": state_bytes / (us * 1e-6) / 1e9, "unit": "GB/s",
                          "us_per_step": us, "steps": 1000,
                          "config": {"workload": "256 seqs x 32 value heads, T=1, 512-slot fp32 pool [128x128], in place"},
                          "layer_step": layer_step, "launch_modes": launch_modes,
                          "note": "us_per_step is the faster of 1000 eager launches and 125 replays of an 8-step CUDA graph",
                          "roofline": {"bound": "hbm", "achieved": all_bytes / (us * 1e-6) / 1e9, "peak": peaks["hbm_gbs"],
                                       "unit": "GB/s", "frac": all_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"],
                                       "frac_of_nominal_8TBps": all_bytes / (us * 1e-6) / 8e12,
                                       "traffic": 1_021_515_264,  # dram read + write of one launch, ncu capture at full size
                                       "traffic_source": "profiles/decode_gdn_decode_kernel_config2.md",
                                       "peak_source": peaks["source"]}}
    if world > 1:
        barrier(world)
    if rank == 0 and world == 1 and not args.no_decode:
        line["backward"] = bench_backward()
    if rank == 0 and not args.no_cpu and world == 1:
        line["cpu_baseline"] = cpu_baseline()
    if not args.no_sharded:
        # the two sharded workloads over the same ranks, a few steps each, parity checked outside the timed regions
        sub = max(3, min(args.steps, 10))
        torch.cuda.empty_cache()
        line["varlen"] = bench_varlen(args, rank, world, steps=sub, full_line=False)
        torch.cuda.empty_cache()
        line["block"] = bench_block(args, rank, world, steps=max(3, min(args.steps, 5)), full_line=False)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
