#!/usr/bin/env python
"""Benchmark of the Mixture-of-Experts block: tokens/s and grouped-GEMM
fraction of the measured bf16 tensor peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one forward of the block over the workload's token batch. At N=1 the
workload is the bf16 prefill block (16384 tokens, d_model 1024, 8 experts,
d_ff 4096, top-2, uniform routing); the same line also carries the
decode-shaped calls of that block and the expert-parallel workload on this one
GPU. Under torchrun the default is the expert-parallel workload (65536 tokens,
d_model 2048, 64 experts, d_ff 1408, top-4, Zipf routing): tokens and experts
sharded over the ranks, strong scaling. Rank 0 prints one JSON line.

``--impl reference`` times the reference's own CPU implementation of the block on
this host's cores instead: its ``model.MOE`` class (from oracle/_ref, an
unmodified copy of the reference's model.py) where that class can express the
workload (two slots, integer expansion factor), else the CPU restatement in
oracle/moe_oracle.py (bit-identical to the class at two slots).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernels per step (GEGLU pass +
# down pass) from the ncu captures summarised under profiles/: a static figure, not measured by
# this run
NCU_TRAFFIC = {
    "c1_uniform": (429.7e6 + 405.7e6, "profiles/grouped_gemm_tc2_c1_uniform.md (static, ncu capture)"),
    "c2_t64": (204.8e6 + 3.8e6, "profiles/decode_spec_kernel_c2_t64.md (static, ncu capture)"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126e6
CPU_ARM_LIMIT_S = 240.0      # the whole --impl reference run should end within a few minutes


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            if "hbm_gbs" in d and "bf16_tflops" in d:
                return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed
    region runs (read-only queries)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def pipelined_e2e(m, x_host, out_host, aux_host, N, d, dt, dev, steps, warm=3):
    """End-to-end loop over three streams: every step copies its input from pinned host
    memory, runs the block and copies output and loss back; copy-in of step i+1, compute
    of step i and copy-out of step i-1 overlap, as a serving loop would. Returns the
    CUDA-event time of `steps` steps in ms (all results on the host when it ends)."""
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_comp = torch.cuda.current_stream(dev)
    x_bufs = [torch.empty(1, N, d, dtype=dt, device=dev) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = []

    def loop(n):
        with torch.no_grad():
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(in_free[b])          # compute of step i-2 has read this buffer
                    x_bufs[b].copy_(x_host.view(1, N, d), non_blocking=True)
                    in_ready[b].record(s_in)
                s_comp.wait_event(in_ready[b])
                o, aux = m(x_bufs[b])
                in_free[b].record(s_comp)
                done = torch.cuda.Event()
                done.record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    out_host.copy_(o.view(N, d), non_blocking=True)
                    aux_host.copy_(aux.view(1), non_blocking=True)
                    o.record_stream(s_out)
                    aux.record_stream(s_out)
                    fin = torch.cuda.Event()
                    fin.record(s_out)
                out_done.append(fin)
                if len(out_done) > 2:
                    out_done.pop(0).synchronize()       # bounded queue: step i-2 is on the host
                    _ = float(aux_host[0])
            for ev in out_done:
                ev.synchronize()
            out_done.clear()

    loop(warm)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loop(steps)
    torch.cuda.synchronize(dev)
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1)


def workload_config(wl):
    """The same keys in both arms, so that the two lines name one configuration."""
    return {"workload": wl.name, "tokens": wl.tokens, "d_model": wl.d_model,
            "n_experts": wl.n_experts, "d_ff": wl.d_ff, "top_k": wl.top_k, "routing": wl.gate_bias,
            "l2": "no flush: the working set of one step (expert weights, sorted rows, h) exceeds the "
                  "126 MB L2; decode-shaped calls rotate over copies of the weights instead"}


# ---------------------------------------------------------------------------
# CPU arm: the reference's own block on the host cores
# ---------------------------------------------------------------------------

def cpu_block(wl):
    """(kind, forward(x [N,d] fp32) -> None) for the workload. kind "reference": the
    reference's model.MOE from oracle/_ref; kind "port": oracle/moe_oracle.py."""
    from gemmallm_b200 import synthetic
    from oracle import make_ref, moe_oracle
    dt = synthetic.torch_dtype(wl.dtype)
    d, E, f, k = wl.d_model, wl.n_experts, wl.d_ff, wl.top_k
    why = None
    if k != 2 or f % d != 0:
        why = "the reference class has two slots and an integer expansion factor"
    elif not make_ref.available():
        why = "oracle/_ref/model.py is absent"
    if why is None:
        try:
            ref = make_ref.load()
            m = ref.MOE(d, num_experts=E, expansion_factor=f // d, device="cpu").eval()
            params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
                d, E, f, seed=0, gate_bias_kind=wl.gate_bias).items()}
            synthetic.load_into(m, params, torch.float32, "cpu")
            del params
            return "reference", (lambda x: m(x.view(1, *x.shape))), None
        except Exception as exc:       # import or construction failed on this box
            why = f"the reference module did not load here ({type(exc).__name__}: {exc})"
    if E > 16:
        w1, w2 = [], []
        for e in range(E):
            pe = synthetic.make_expert(d, f, e, 0)
            w1.append(synthetic.round_to(pe["w1"], dt))
            w2.append(synthetic.round_to(pe["w2"], dt))
        gate_w, gate_b = synthetic.make_gate(d, E, 0, wl.gate_bias)
        params = {"gate_w": synthetic.round_to(gate_w, dt), "gate_b": synthetic.round_to(gate_b, dt),
                  "w1": w1, "b1": torch.zeros(E, 2 * f), "w2": w2, "b2": torch.zeros(E, d)}
    else:
        params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
            d, E, f, seed=0, gate_bias_kind=wl.gate_bias).items()}
    return "port", (lambda x: moe_oracle.moe_forward(x, params, k)), why


def cpu_arm(wl, steps, warmup, limit_s):
    """Times the CPU block: fp32 on bf16-rounded values (the reference cannot run in bf16),
    all host threads. The sample is the whole token batch unless one step is so slow that
    steps + warmup of them would pass `limit_s`; then the first tokens of the batch, as many
    as fit. Returns (per-step seconds, cores, kind, sample text, tokens per step, note)."""
    from gemmallm_b200 import synthetic
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dt = synthetic.torch_dtype(wl.dtype)
    kind, fwd, why = cpu_block(wl)
    x_all = synthetic.round_to(synthetic.make_input(wl.tokens, wl.d_model, seed=1), dt)
    tokens = wl.tokens
    with torch.no_grad():
        t0 = time.perf_counter()
        fwd(x_all)
        first = time.perf_counter() - t0
        total_calls = steps + max(warmup - 1, 0)
        if first * total_calls > limit_s and tokens > 1024:
            tokens = max(1024, int(tokens * limit_s / (first * total_calls)) // 1024 * 1024)
        x = x_all[:tokens]
        for _ in range(max(warmup - 1, 0)):
            fwd(x)
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            fwd(x)
            times.append(time.perf_counter() - t0)
    sample = (f"all {tokens} tokens per step" if tokens == wl.tokens else
              f"first {tokens} of {wl.tokens} tokens per step (the whole batch would pass the time limit)")
    sample += ", fp32 on bf16-rounded values" if wl.dtype == "bf16" else ", fp32"
    return times, cores, kind, sample, tokens, why


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, cores, kind, sample, tokens, why = cpu_arm(wl, args.steps, args.warmup, CPU_ARM_LIMIT_S)
    total = sum(times)
    value = tokens * args.steps / total
    line = {
        "impl": "reference", "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": "strong" if (args.gpus > 1 and wl.name == "c4") else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(wl),
        "run": {"parallelism": "cpu", "threads": cores},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind,
                         "sample": sample, **({"why_port": why} if why else {})},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_record(wl, reps):
    times, cores, kind, sample, tokens, why = cpu_arm(wl, reps, 1, 30.0)
    times.sort()
    rec = {"value": tokens / times[len(times) // 2], "unit": "tokens/s", "cores": cores, "kind": kind,
           "sample": f"{sample}, median of {reps}"}
    if why:
        rec["why_port"] = why
    return rec


# ---------------------------------------------------------------------------
# our arm, one GPU (or token-sharded replicas)
# ---------------------------------------------------------------------------

def build_block(wl, dev, dt):
    from gemmallm_b200 import MOE, synthetic
    d, f, E, k = wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    m = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda").eval()
    if E > 16:
        # many experts: draw them one at a time (same rule as the expert-parallel ranks)
        m.to(device=dev, dtype=dt)
        gate_w, gate_b = synthetic.make_gate(d, E, 0, wl.gate_bias)
        with torch.no_grad():
            m.gate.weight.copy_(gate_w)
            m.gate.bias.copy_(gate_b)
            for e, ex in enumerate(m.experts):
                pe = synthetic.make_expert(d, f, e, 0)
                ex.gate_and_up.weight.copy_(pe["w1"])
                ex.down.weight.copy_(pe["w2"])
                ex.gate_and_up.bias.zero_()
                ex.down.bias.zero_()
    else:
        params = synthetic.make_params(d, E, f, seed=0, gate_bias_kind=wl.gate_bias)
        synthetic.load_into(m, params, dt, dev)
    return m


def clone_block(m, wl, dev, dt):
    from gemmallm_b200 import MOE
    r = MOE(wl.d_model, num_experts=wl.n_experts, d_ff=wl.d_ff, top_k=wl.top_k, device="cuda").eval()
    r.to(device=dev, dtype=dt)
    r.load_state_dict(m.state_dict())
    return r


def is_small_n(wl):
    from gemmallm_b200._cabi import lib
    return wl.dtype == "bf16" and wl.tokens * wl.top_k <= lib.moe_b200_decode_max_rows()


def is_mid_n(wl):
    return (wl.dtype == "bf16" and not is_small_n(wl) and wl.tokens * wl.top_k <= 4096
            and wl.tokens <= 2048 and wl.n_experts <= 32)


def streamed_bytes(m, wl, spec_all: bool):
    """Algorithmic bytes of one small-N call: weights of the distinct experts hit (all of them
    when the routing-independent kernel runs), router weights, x in, out."""
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    es = 2
    hit = int((m.last["cnt_slot"].sum(0) > 0).sum())
    wbytes = hit * (3 * d * f + 2 * f + d) * es
    touched = (E if spec_all else hit) * (3 * d * f + 2 * f + d) * es
    return hit, wbytes, wbytes + E * d * es + 2 * N * d * es, touched


def time_streaming(replicas, make_replica, wl, x, steps, graphs=True):
    """Device time per call of a small-N workload: the calls rotate over copies of the block so
    that no call finds its weights in L2, several calls per CUDA graph (as a decoder that
    captures all its layers would). Returns (ms per call, calls per graph, copies used)."""
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    m = replicas[0]
    with torch.no_grad():
        for _ in range(3):
            m(x)
    torch.cuda.synchronize()
    spec_all = N * k >= E and is_small_n(wl)
    _, _, _, touched = streamed_bytes(m, wl, spec_all)
    n_rep = max(1, -(-int(2 * L2_BYTES) // touched))
    while len(replicas) < n_rep:
        replicas.append(make_replica())
    use = replicas[:n_rep]
    with torch.no_grad():
        for r in use:
            for _ in range(3):
                r(x)
    torch.cuda.synchronize()
    per_graph = n_rep * max(1, 8 // n_rep)
    graph = None
    if graphs:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.no_grad(), torch.cuda.graph(graph):
                for i in range(per_graph):
                    use[i % n_rep](x)
        except Exception as exc:
            print(f"# CUDA graph capture failed ({exc}); timing eager calls", file=sys.stderr)
            torch.cuda.synchronize()
            graph = None

    def eager():
        with torch.no_grad():
            for i in range(per_graph):
                use[i % n_rep](x)

    step = graph.replay if graph is not None else eager
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    reps = max(1, steps // per_graph)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * per_graph), per_graph, n_rep, graph is not None


def decode_sweep(m, wl_main, dev, dt, hbm):
    """The decode-shaped calls of the same block (1, 8, 32, 64 tokens): whole call, CUDA-event
    time per call, algorithmic bytes over the measured HBM copy bandwidth."""
    from gemmallm_b200 import synthetic
    out = {}
    replicas = [m]
    for T in (1, 8, 32, 64):
        wl = synthetic.WORKLOADS[f"c2_t{T}"]
        if (wl.d_model, wl.d_ff, wl.n_experts, wl.top_k) != (wl_main.d_model, wl_main.d_ff,
                                                             wl_main.n_experts, wl_main.top_k):
            return None
        x = synthetic.make_input(T, wl.d_model, seed=1).to(dt).to(dev).view(1, T, wl.d_model)
        ms, per_graph, n_rep, graphed = time_streaming(
            replicas, lambda: clone_block(m, wl, dev, dt), wl, x, 400)
        for r in replicas:
            if r.device_status() != 0:
                raise RuntimeError(f"device status non-zero in the decode sweep at {T} tokens")
        hit, wbytes, nbytes, _ = streamed_bytes(replicas[0], wl, False)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[f"t{T}"] = {"us": ms * 1e3, "bytes": nbytes, "experts_hit": hit, "gbs": gbs,
                        "frac": gbs / hbm, "weight_copies_rotated": n_rep, "calls_per_graph": per_graph,
                        "cuda_graph": graphed}
    del replicas[1:]
    torch.cuda.empty_cache()
    return out


def run_ours(args, wl):
    import torch.distributed as dist
    from gemmallm_b200 import _cabi, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    dt = synthetic.torch_dtype(wl.dtype)
    es = 2 if wl.dtype == "bf16" else 4
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    m = build_block(wl, dev, dt)
    # each rank owns its own token batch (seed differs per rank)
    x_host = synthetic.make_input(N, d, seed=1 + rank).to(dt).pin_memory()
    x = x_host.to(dev).view(1, N, d)
    out_host = torch.empty(N, d, dtype=dt).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        return ms

    small_n, mid_n = is_small_n(wl), is_mid_n(wl)
    streaming = small_n or mid_n      # launch-bound from Python, bound by the weight stream on the GPU
    warm = max(args.warmup, 3)

    # ---- device-resident throughput -------------------------------------
    graphed, steps_per_graph, n_rep = False, 1, 1
    if streaming:
        barrier()
        with ClockSampler(local) as clocks:
            ms_step, steps_per_graph, n_rep, graphed = time_streaming(
                [m], lambda: clone_block(m, wl, dev, dt), wl, x, args.steps, graphs=not args.no_graph)
            barrier()
        ms_total = max_over_ranks(ms_step * args.steps)
    else:
        with torch.no_grad():
            for _ in range(warm):
                m(x)
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local) as clocks:
                ev0.record()
                for _ in range(args.steps):
                    m(x)
                ev1.record()
                barrier()
            ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    status = m.device_status()
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")
    ms_step = ms_total / args.steps
    value = N * world * args.steps / (ms_total * 1e-3)

    if args.quick:
        if rank == 0:
            print(json.dumps({"metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s",
                              "n_gpus": world, "steps": args.steps, "ms_per_step": ms_step,
                              "quick": True, "config": workload_config(wl)}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers in, host buffers out --------------------
    # Every step copies its input from pinned host memory, runs the block and
    # copies the output and the loss back. Large batches are pipelined over
    # three streams (copy-in of step i+1, compute of step i, copy-out of step
    # i-1 overlap, as a serving loop would); small-N calls replay one CUDA
    # graph per step and wait for it, since there latency is the point.
    aux_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    if streaming:
        x_dev = torch.empty(1, N, d, dtype=dt, device=dev)

        def e2e_step():
            x_dev.copy_(x_host.view(1, N, d), non_blocking=True)
            o, aux = m(x_dev)
            out_host.copy_(o.view(N, d), non_blocking=True)
            aux_host.copy_(aux.view(1), non_blocking=True)

        with torch.no_grad():
            for _ in range(2):
                e2e_step()
            torch.cuda.synchronize()
            run_e2e = e2e_step
            if not args.no_graph:
                try:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        e2e_step()
                    run_e2e = g.replay
                except Exception:
                    torch.cuda.synchronize()
            run_e2e()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                run_e2e()
                torch.cuda.current_stream().synchronize()   # output and loss are on the host now
                _loss = float(aux_host[0])
            e1.record()
            barrier()
            e2e_ms = max_over_ranks(e0.elapsed_time(e1))
        e2e_mode = "one CUDA graph per step, host waits for every step"
    else:
        barrier()
        e2e_ms = max_over_ranks(pipelined_e2e(m, x_host, out_host, aux_host, N, d, dt, dev, args.steps))
        barrier()
        e2e_mode = "three streams: copy-in, compute, copy-out of consecutive steps overlap"
    e2e_value = N * world * args.steps / (e2e_ms * 1e-3)

    # ---- per-stage times through the stage entry points --------------------
    launches_per_step = 3 if streaming else 5
    stage_ms = {}
    if rank == 0:
        stage_ms = time_stages(m, x.view(N, d), wl, dev, small_n, mid_n=mid_n)
    peaks, peak_kind = load_peaks()
    if rank == 0:
        flops = 6.0 * k * d * f * N
        t_gemm = stage_ms["experts"] * 1e-3
        achieved = flops / t_gemm / 1e12
        peak = float(peaks["bf16_tflops"])
        hbm = float(peaks["hbm_gbs"])
        stage_bytes = {
            "router": N * d * es + E * d * es + N * k * 8,
            "dispatch": N * d * es + N * k * d * es + N * k * 8,
            "combine": N * k * d * es + N * d * es + N * k * 8,
        }
        stage_bytes = {n: b for n, b in stage_bytes.items() if n in stage_ms}
        traffic, traffic_source = NCU_TRAFFIC.get(wl.name, (None, None))
        line = {
            "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic",
            "config": workload_config(wl),
            "run": {"parallelism": "single" if world == 1 else f"tokens sharded over {world} ranks, experts replicated",
                    "cuda_graph": graphed, "steps_per_graph": steps_per_graph,
                    "weight_copies_rotated": n_rep},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": N * d * es,
                    "d2h_bytes_per_step": N * d * es + 4, "ms_per_step": e2e_ms / args.steps,
                    "mode": e2e_mode},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"kernel": "grouped_gemm_tc2_kernel (GEGLU pass + down pass, CTA pairs)"
                                   if wl.dtype == "bf16" else "grouped_ffn_kernel<float> (CUDA cores)",
                         "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": f"{peak_kind} bf16 burst", "flops_per_step": flops,
                         "ms": stage_ms["experts"]},
            "stages_ms": stage_ms,
            "stages_hbm": {n: {"bytes": b, "gbs": b / (stage_ms[n] * 1e-3) / 1e9,
                               "frac": b / (stage_ms[n] * 1e-3) / 1e9 / hbm}
                           for n, b in stage_bytes.items()},
        }
        if streaming:
            hit, wbytes, nbytes_step, _ = streamed_bytes(m, wl, False)
            gbs_step = nbytes_step / (ms_step * 1e-3) / 1e9
            gbs_experts = wbytes / (stage_ms["experts"] * 1e-3) / 1e9
            line["roofline"] = {
                "kernel": ("decode_spec_kernel (GEGLU + split-K down tiles, one launch) / geglu_gemv + down_gemv"
                           if small_n else "decode_spec_kernel<SORTED> (GEGLU + split-K down tiles on sorted rows)"),
                "bound": "hbm", "achieved": gbs_experts, "peak": hbm, "unit": "GB/s",
                "frac": gbs_experts / hbm, "traffic": traffic, "traffic_source": traffic_source,
                "peak_source": f"{peak_kind} copy",
                "bytes_per_step": wbytes, "experts_hit": hit, "ms": stage_ms["experts"],
                "whole_step_gbs": gbs_step, "whole_step_frac": gbs_step / hbm}
            if small_n and N <= 8 and N * k < E:
                # one to eight tokens: the whole call is one kernel, timed by the step itself
                line["roofline"].update({
                    "kernel": "decode_tiny_kernel (routing, GEGLU, down product, weighted sum: one cooperative launch)",
                    "achieved": gbs_step, "frac": gbs_step / hbm, "bytes_per_step": nbytes_step,
                    "ms": ms_step})
                line["gpu_launches"] = args.steps
        if world == 1 and wl.name == "c1_uniform" and not args.no_extras:
            # the other single-GPU records of the default run: the decode-shaped calls of this
            # block, and the expert-parallel workload on this one GPU (the same-workload
            # denominator of the multi-GPU speed-ups)
            line["c2"] = decode_sweep(m, wl, dev, dt, hbm)
            line["around_the_block"] = around_the_block(m, x, dev)
            del m, x
            torch.cuda.empty_cache()
            line["c4_one_gpu"] = one_gpu_record(synthetic.WORKLOADS["c4"], dev, peak)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_record(wl, 3 if N > 256 else 20)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def around_the_block(m, x, dev, reps=20):
    """The block's callers on this workload, device-resident, ms per call: the LoRA branch
    (model.py:175-179,185-189: merged weights cached / re-merged after every parameter update) and
    the caller's LayerNorm (model.py:311-312,319) folded into the block or applied in front of it."""
    def timed(fn):
        with torch.no_grad():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(reps):
                fn()
            t1.record()
            torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps

    d = x.shape[-1]
    ln = torch.nn.LayerNorm(d).to(device=dev, dtype=x.dtype)
    with torch.no_grad():
        ln.weight.uniform_(0.5, 1.5)
        ln.bias.uniform_(-0.1, 0.1)

    def bump():
        # what an optimizer step does to the LoRA tensors: the cached merged weights are stale
        for ex in m.experts:
            ex.lora_down_b.weight.add_(0.0)
            ex.lora_gate_and_up_b.weight.add_(0.0)

    rec = {
        "plain_ms": timed(lambda: m(x, residual=x)),
        "lora_merged_cached_ms": timed(lambda: m(x, fine_tuning=True, residual=x)),
        "lora_remerged_every_call_ms": timed(lambda: (bump(), m(x, fine_tuning=True, residual=x))),
        "layernorm_folded_ms": timed(lambda: m(x, residual=x, norm=ln)),
        "layernorm_in_front_ms": timed(lambda: m(ln(x), residual=x)),
    }
    if m.device_status() != 0:
        raise RuntimeError("device status non-zero in the LoRA / LayerNorm timings")
    return rec


def one_gpu_record(wl, dev, peak, steps=10):
    """A workload's block on this one GPU, device-resident: ms per step, tokens/s and the
    grouped GEMMs' share of the tensor peak."""
    from gemmallm_b200 import synthetic
    dt = synthetic.torch_dtype(wl.dtype)
    N, d, f, k = wl.tokens, wl.d_model, wl.d_ff, wl.top_k
    m = build_block(wl, dev, dt)
    x = synthetic.make_input(N, d, seed=1).to(dt).to(dev).view(1, N, d)
    with torch.no_grad():
        for _ in range(3):
            m(x)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            m(x)
        t1.record()
        torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    if m.device_status() != 0:
        raise RuntimeError("device status non-zero")
    st = time_stages(m, x.view(N, d), wl, dev, reps=5)
    tf = 6.0 * k * d * f * N / (st["experts"] * 1e-3) / 1e12
    return {"workload": wl.name, "ms_per_step": ms, "tokens_per_s": N / (ms * 1e-3),
            "experts_ms": st["experts"], "experts_tflops": tf, "experts_frac": tf / peak}


# ---------------------------------------------------------------------------
# our arm, expert-parallel workload under torchrun
# ---------------------------------------------------------------------------

def ep_parity(m, x_host_f32, out, wl, rank, tokens=1024):
    """After the timed region: the first `tokens` tokens of this rank's last output against the
    CPU oracle under the kernel's own logits (tokens are independent, model.py:201)."""
    from gemmallm_b200 import synthetic
    from oracle import moe_oracle
    dt = synthetic.torch_dtype(wl.dtype)
    d, f, E, k = wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    n = min(tokens, x_host_f32.shape[0])
    w1, w2 = [], []
    for e in range(E):
        pe = synthetic.make_expert(d, f, e, 0)
        w1.append(synthetic.round_to(pe["w1"], dt))
        w2.append(synthetic.round_to(pe["w2"], dt))
    gate_w, gate_b = synthetic.make_gate(d, E, 0, wl.gate_bias)
    params = {"gate_w": synthetic.round_to(gate_w, dt), "gate_b": synthetic.round_to(gate_b, dt),
              "w1": w1, "b1": torch.zeros(E, 2 * f), "w2": w2, "b2": torch.zeros(E, d)}
    logits = m.last["logits"][:n].float().cpu()
    with torch.no_grad():
        o = moe_oracle.moe_forward(x_host_f32[:n], params, k, logits=logits)
    good = ~moe_oracle.tie_rows(o["probs"], k)
    idx_equal = bool(torch.equal(m.last["idx"][:n].cpu()[good].long(), o["idx"][good]))
    got = out.view(-1, d)[:n].float().cpu()
    err = float((got - o["out"])[good].abs().max())
    bound = 2e-2 * float(o["out"].abs().max())
    return idx_equal, err, bound


def run_ep(args, wl):
    """Expert-parallel workload under torchrun: tokens and experts sharded over
    the ranks, strong scaling (the token total is fixed)."""
    import torch.distributed as dist
    from gemmallm_b200 import _cabi, synthetic
    from gemmallm_b200._cabi import lib, check
    from gemmallm_b200.ep import ExpertParallelMOE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    dt = synthetic.torch_dtype(wl.dtype)
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    Nl = N // world
    placement = None
    if args.ep_placement == "lpt":
        # popularity prior from the router bias: softmax mass of the bias alone
        from gemmallm_b200.ep import lpt_placement
        prior = torch.softmax(synthetic.gate_bias(wl.gate_bias, E), 0).tolist()
        placement = lpt_placement(prior, world)
    replicate = None
    if args.ep_replicate > 0:
        # copies of the most popular experts (by the router-bias prior) on every rank
        prior = torch.softmax(synthetic.gate_bias(wl.gate_bias, E), 0)
        replicate = prior.topk(min(args.ep_replicate, E)).indices.tolist()
    m = ExpertParallelMOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda", placement=placement,
                          replicate=replicate).eval()
    m.to(device=dev, dtype=dt)
    gate_w, gate_b = synthetic.make_gate(d, E, 0, wl.gate_bias)
    with torch.no_grad():
        m.gate.weight.copy_(gate_w)
        m.gate.bias.copy_(gate_b)
        for e in sorted(set(m.local_ids)):
            p = synthetic.make_expert(d, f, e, 0)
            ex = m.experts[str(e)]
            ex.gate_and_up.weight.copy_(p["w1"])
            ex.down.weight.copy_(p["w2"])
            ex.gate_and_up.bias.zero_()
            ex.down.bias.zero_()
    x_f32 = synthetic.round_to(synthetic.make_input(Nl, d, seed=1 + rank), dt)
    x_host = x_f32.to(dt).pin_memory()
    x = x_host.to(dev).view(1, Nl, d)
    out_host = torch.empty(Nl, d, dtype=dt).pin_memory()
    aux_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            out, _aux = m(x)
        barrier()
        # One forward per CUDA graph: the call's hand-shake counter lives on the device, so the
        # same six launches replay unchanged and the host's share of a 0.7 ms step disappears.
        graph = None
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    out, _aux = m(x)
            except Exception as exc:
                print(f"# rank {rank}: CUDA graph capture failed ({exc}); timing eager calls", file=sys.stderr)
                torch.cuda.synchronize()
                graph = None
        # every rank must make the same calls: all replay, or none
        cap = torch.tensor([1.0 if graph is not None else 0.0], device=dev)
        dist.all_reduce(cap, op=dist.ReduceOp.MIN)
        if float(cap) == 0.0:
            graph = None

        def step():
            nonlocal out
            if graph is not None:
                graph.replay()
            else:
                out, _ = m(x)

        for _ in range(3):
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            ev0.record()
            for _ in range(args.steps):
                step()
            ev1.record()
            barrier()
        ms_total = max_over_ranks(ev0.elapsed_time(ev1))
        status = max_over_ranks(float(m.device_status()))
        if status != 0:
            raise RuntimeError(f"device status {status} after the timed region")
        if args.quick:
            if rank == 0:
                print(json.dumps({"metric": "moe_tokens_per_s", "value": N * args.steps / (ms_total * 1e-3),
                                  "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                                  "ms_per_step": ms_total / args.steps, "quick": True,
                                  "config": workload_config(wl)}), flush=True)
            dist.barrier()
            dist.destroy_process_group()
            return
        # parity of what was just timed, outside the timed region
        idx_equal, err, bound = ep_parity(m, x_f32, out, wl, rank)
        par = torch.tensor([1.0 if (idx_equal and err <= bound) else 0.0, 1.0 if idx_equal else 0.0,
                            err / bound], device=dev)
        pars = [torch.empty_like(par) for _ in range(world)]
        dist.all_gather(pars, par)
        # per-stage times (events recorded by the library at the stage boundaries)
        barrier()
        stages = m.time_stages(x, reps=10)
        st = torch.tensor([stages[n] for n in _cabi.EP_STAGES], device=dev)
        sts = [torch.empty_like(st) for _ in range(world)]
        dist.all_gather(sts, st)
        # the same exchange through NCCL all_to_all_single (host-side baseline)
        for _ in range(3):
            m.forward_nccl(x)
        nccl_ms = timed(lambda: m.forward_nccl(x), max(5, args.steps // 2)) / max(5, args.steps // 2)
        # end to end: pinned host input in, output and loss back, every step (pipelined)
        barrier()
        e2e_ms = max_over_ranks(pipelined_e2e(m, x_host, out_host, aux_host, Nl, d, dt, dev, args.steps))
        barrier()
        # grouped GEMMs alone on this rank's received rows
        rows = int(m.last["offsets_local"][-1])
        stt = m._state
        recv_x = stt["hdl"].buffer_ptrs[rank] + stt["symm_layout"]["recv_x"]
        hbuf = stt["ws_base"] + stt["ws_layout"]["h"]
        offs = stt["ws_base"] + stt["ws_layout"]["offsets_local"]
        stat = stt["ws_base"] + stt["ws_layout"]["status"]
        ybuf = torch.empty(max(rows, 1), d, dtype=dt, device=dev)
        s_ = torch.cuda.current_stream(dev).cuda_stream
        call = lambda: lib.moe_b200_experts(recv_x, offs, m._plan.base, rows, d, f, len(m.local_ids),
                                            _cabi.BF16, 0, hbuf, ybuf.data_ptr(), stat, s_)
        for _ in range(3):
            check(call(), "experts")
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(10):
            call()
        g1.record()
        torch.cuda.synchronize()
        gemm_ms = g0.elapsed_time(g1) / 10
    info = torch.tensor([float(rows), gemm_ms], device=dev)
    gathered = [torch.empty_like(info) for _ in range(world)]
    dist.all_gather(gathered, info)
    single, cpu_rec = None, None
    peaks, peak_kind = load_peaks()
    peak = float(peaks["bf16_tflops"])
    if rank == 0:
        # the same workload on this one GPU (all experts local, no exchange), for the speed-up
        del m
        torch.cuda.empty_cache()
        single = one_gpu_record(wl, dev, peak)
        if not args.no_cpu_baseline:
            cpu_rec = cpu_baseline_record(wl, 1)
    if rank == 0:
        es = 2
        per_rank = [{"rows": int(g[0]), "gemm_ms": float(g[1]),
                     "tflops": 6.0 * d * f * float(g[0]) / (float(g[1]) * 1e-3) / 1e12} for g in gathered]
        busiest = max(per_rank, key=lambda r: r["gemm_ms"])
        share = max(r["rows"] for r in per_rank) / float(N * k)
        ms_step = ms_total / args.steps
        ranks_ok = int(sum(float(p[0]) for p in pars))
        line = {
            "metric": "moe_tokens_per_s", "value": N * args.steps / (ms_total * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": workload_config(wl),
            "run": {"parallelism": f"ep{world}: tokens and experts sharded over {world} ranks, "
                                   f"{args.ep_placement} expert placement, {args.ep_replicate} hottest experts "
                                   "copied to every rank, peer-store all-to-all inside the kernels",
                    "cuda_graph": graph is not None},
            "e2e": {"value": N * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": Nl * d * es * world, "d2h_bytes_per_step": (Nl * d * es + 4) * world,
                    "ms_per_step": e2e_ms / args.steps,
                    "mode": "per rank three streams: copy-in, compute, copy-out of consecutive steps overlap"},
            "gpu_launches": 6 * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"kernel": "grouped_gemm_tc2_kernel (GEGLU pass + down pass) on the busiest rank",
                         "bound": "tensor", "achieved": busiest["tflops"], "peak": peak,
                         "unit": "TFLOP/s", "frac": busiest["tflops"] / peak, "traffic": None,
                         "peak_source": f"{peak_kind} bf16 burst", "ms": busiest["gemm_ms"]},
            "parity": {"checked": "first 1024 tokens of every rank's last timed output against the CPU "
                                  "oracle under the kernel's logits",
                       "idx_equal": all(float(p[1]) == 1.0 for p in pars),
                       "max_abs_over_bound": max(float(p[2]) for p in pars),
                       "bound": "2e-2 * max|reference|", "ranks_ok": ranks_ok},
            "stages_ms": {"rank0": {n: float(sts[0][i]) for i, n in enumerate(_cabi.EP_STAGES)},
                          "max_over_ranks": {n: max(float(s[i]) for s in sts)
                                             for i, n in enumerate(_cabi.EP_STAGES)}},
            "nccl_baseline": {"ms_per_step": nccl_ms, "tokens_per_s": N / (nccl_ms * 1e-3),
                              "what": "same router, expert and combine kernels; dispatch and return as "
                                      "torch.distributed all_to_all_single with host-side split sizes"},
            "ep": {"per_rank": per_rank, "max_rank_share_of_rows": share,
                   "balance_limited_speedup": 1.0 / share,
                   "gemm_ms_over_step_ms": busiest["gemm_ms"] / ms_step,
                   "same_workload_on_one_gpu": single,
                   "speedup_vs_one_gpu": (single["ms_per_step"] / ms_step) if single else None},
        }
        if cpu_rec:
            line["cpu_baseline"] = cpu_rec
        print(json.dumps(line), flush=True)
        if ranks_ok != world:
            print(f"# parity failed on {world - ranks_ok} rank(s)", file=sys.stderr)
    ok = torch.tensor([1.0 if (idx_equal and err <= bound) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if float(ok) != 1.0:
        sys.exit(1)


# ---------------------------------------------------------------------------
# the whole decoder forward with the block swapped in (workload "c3")
# ---------------------------------------------------------------------------

C3 = {"layers": 12, "vocab": 32000, "context": 64, "d_model": 1024, "factor": 4, "head_dim": 64,
      "q_heads": 16, "kv_heads": 1, "n_experts": 8, "batch": 512}


def build_decoder(device, swap: bool, dtype):
    """The reference's LLM (model.py:322-372, from oracle/_ref) with seeded N(0, 0.02^2) weights
    and zero biases; with `swap` every layer.moe is replaced by the new block through the strict
    state_dict."""
    from gemmallm_b200 import MOE
    from oracle import make_ref
    ref = make_ref.load()
    c = C3
    reset = torch.nn.Linear.reset_parameters
    torch.nn.Linear.reset_parameters = lambda self: None    # every Linear is overwritten below
    try:
        with torch.device(device):
            llm = ref.LLM(c["layers"], c["vocab"], c["context"], c["d_model"], expansion_factor=c["factor"],
                          head_dim=c["head_dim"], q_head=c["q_heads"], kv_head=c["kv_heads"], use_moe=True,
                          num_experts=c["n_experts"], device=str(device)).eval()
    finally:
        torch.nn.Linear.reset_parameters = reset
    g = torch.Generator(device=device).manual_seed(0)
    with torch.no_grad():
        for name, p in llm.named_parameters():
            if "pos_emb" in name or "norm" in name:
                continue
            if name.endswith(".bias"):
                p.zero_()
            else:
                p.copy_(torch.randn(p.shape, generator=g, device=device) * 0.02)
    if swap:
        for layer in llm.transformer:
            new = MOE(c["d_model"], num_experts=c["n_experts"], expansion_factor=c["factor"], device="cuda").eval()
            new.to(device)
            new.load_state_dict(layer.moe.state_dict(), strict=True)
            layer.moe = new
    return llm.to(dtype=dtype)


def decoder_config():
    c = C3
    return {"workload": "c3", "tokens": c["batch"] * c["context"], "d_model": c["d_model"],
            "n_experts": c["n_experts"], "d_ff": c["d_model"] * c["factor"], "top_k": 2, "routing": "zero",
            "layers": c["layers"], "vocab": c["vocab"], "context": c["context"],
            "l2": "no flush: one layer's working set exceeds the 126 MB L2"}


def run_decoder(args):
    """tokens/s of the reference's whole 12-layer decoder forward in bf16 with the new block in
    every layer; attention, norms and classifier are the reference's own torch code."""
    c = C3
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    dt = torch.bfloat16
    llm = build_decoder(dev, True, dt)
    ids = torch.randint(0, c["vocab"], (c["batch"], c["context"]), generator=torch.Generator().manual_seed(3))
    table = (torch.randn(c["vocab"], c["d_model"], generator=torch.Generator().manual_seed(2)) * 0.02)
    x_host = table[ids].to(dt).pin_memory()
    x = x_host.to(dev)
    mask = torch.triu(torch.full((c["context"], c["context"]), float("-inf"), device=dev, dtype=dt), 1)
    moe_events = []

    def pre(mod, a):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        moe_events.append([e, None])

    def post(mod, a, o):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        moe_events[-1][1] = e

    tokens = c["batch"] * c["context"]
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            logits, aux = llm(x.clone(), mask, False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(dev.index or 0) as clocks:
            e0.record()
            for _ in range(args.steps):
                logits, aux = llm(x.clone(), mask, False)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        # the block's share: events around every layer.moe call of a few more forwards
        handles = []
        for layer in llm.transformer:
            handles += [layer.moe.register_forward_pre_hook(pre), layer.moe.register_forward_hook(post)]
        for _ in range(3):
            llm(x.clone(), mask, False)
        torch.cuda.synchronize()
        for h in handles:
            h.remove()
        moe_ms = sum(a.elapsed_time(b) for a, b in moe_events) / 3
        # beyond the named configuration: the layers' attention replaced as well (fused RoPE /
        # scores / softmax / PV / head-gate kernel between the reference's Linears)
        from gemmallm_b200 import Attention
        for layer in llm.transformer:
            old = layer.mqa
            new = Attention(c["d_model"], c["head_dim"], c["q_heads"], c["kv_heads"], old.embedding).eval()
            new.load_state_dict(old.state_dict(), strict=True)
            layer.mqa = new.to(device=dev, dtype=dt)
        for _ in range(3):
            llm(x.clone(), mask, False)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(args.steps):
            llm(x.clone(), mask, False)
        a1.record()
        torch.cuda.synchronize()
        ms_att = a0.elapsed_time(a1) / args.steps
        # the whole layer replaced (model.py:278-321): the second LayerNorm folded into the block's
        # router and dispatch, the second skip connection into its combine
        from gemmallm_b200 import LLMLayer
        for i, layer in enumerate(llm.transformer):
            new = LLMLayer(c["d_model"], c["head_dim"], c["q_heads"], c["kv_heads"], layer.mqa.embedding,
                           expansion_factor=c["factor"], use_moe=True, num_experts=c["n_experts"],
                           device="cuda").eval()
            new.load_state_dict(layer.state_dict(), strict=True)
            llm.transformer[i] = new.to(device=dev, dtype=dt)
        for _ in range(3):
            llm(x.clone(), mask, False)
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(args.steps):
            llm(x.clone(), mask, False)
        b1.record()
        torch.cuda.synchronize()
        ms_layer = b0.elapsed_time(b1) / args.steps
        # end to end: embeddings from pinned host memory in, last-position logits and loss out
        out_host = torch.empty(c["batch"], c["vocab"], dtype=dt).pin_memory()
        aux_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            xin = x_host.to(dev, non_blocking=True)
            logits, aux = llm(xin, mask, False)
            out_host.copy_(logits[:, -1, :], non_blocking=True)
            aux_host.copy_(aux.float().view(1), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        t1.record()
        torch.cuda.synchronize()
        e2e_ms = t0.elapsed_time(t1) / args.steps
    status = max(layer.moe.device_status() for layer in llm.transformer)
    if status != 0:
        raise RuntimeError(f"device status {status}")
    peaks, peak_kind = load_peaks()
    flops = 6.0 * 2 * c["d_model"] * c["d_model"] * c["factor"] * tokens * c["layers"]
    line = {
        "metric": "moe_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decoder_config(),
        "run": {"what": "whole decoder forward (reference LLM, every layer.moe swapped for the new block)",
                "moe_ms_per_forward": moe_ms, "moe_share": moe_ms / ms,
                "with_new_attention_too": {"ms_per_step": ms_att, "tokens_per_s": tokens / (ms_att * 1e-3)},
                "with_the_whole_layer_replaced": {"ms_per_step": ms_layer,
                                                  "tokens_per_s": tokens / (ms_layer * 1e-3)},
                "moe_tflops_incl_router_dispatch_combine": flops / (moe_ms * 1e-3) / 1e12},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                "configuration": "every layer replaced by the new layer (block, attention, folded LayerNorm)",
                "h2d_bytes_per_step": tokens * c["d_model"] * 2,
                "d2h_bytes_per_step": c["batch"] * c["vocab"] * 2 + 4, "ms_per_step": e2e_ms,
                "mode": "embeddings from pinned host memory, last-position logits and loss back, host waits"},
        "gpu_launches": 5 * c["layers"] * args.steps,
        "clocks": clocks.summary(),
        "roofline": {"kernel": "grouped_gemm_tc2_kernel inside the 12 blocks (whole block timed)",
                     "bound": "tensor", "achieved": flops / (moe_ms * 1e-3) / 1e12,
                     "peak": float(peaks["bf16_tflops"]), "unit": "TFLOP/s",
                     "frac": flops / (moe_ms * 1e-3) / 1e12 / float(peaks["bf16_tflops"]), "traffic": None,
                     "peak_source": f"{peak_kind} bf16 burst"},
    }
    print(json.dumps(line), flush=True)


def run_decoder_reference(args):
    """The unmodified reference LLM (its own MoE) on the host cores, fp32: a bounded sample of
    16 sequences per step instead of 512."""
    c = C3
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    llm = build_decoder(torch.device("cpu"), False, torch.float32)
    batch = 16
    ids = torch.randint(0, c["vocab"], (batch, c["context"]), generator=torch.Generator().manual_seed(3))
    table = (torch.randn(c["vocab"], c["d_model"], generator=torch.Generator().manual_seed(2)) * 0.02)
    x = table[ids]
    mask = torch.triu(torch.full((c["context"], c["context"]), float("-inf")), 1)
    with torch.no_grad():
        for _ in range(max(1, min(args.warmup, 2))):
            llm(x.clone(), mask, False)
        times = []
        for _ in range(args.steps):
            t0 = time.perf_counter()
            llm(x.clone(), mask, False)
            times.append(time.perf_counter() - t0)
    value = batch * c["context"] * args.steps / sum(times)
    line = {"impl": "reference", "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * sum(times) / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": decoder_config(),
            "run": {"parallelism": "cpu", "threads": cores},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "reference",
                             "sample": f"{batch} of {c['batch']} sequences per step, whole decoder forward, fp32"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# training step of the block (reference train.py:136-142 around model.py:200-276):
# forward in training mode, loss = sum(out * g) + 0.01 * load_balancing_loss, backward
# ---------------------------------------------------------------------------

TRAIN_DROPOUT = 0.1     # the reference's default dropout_ratio (model.py:155,193)


def train_config(wl):
    c = workload_config(wl)
    c["workload"] = wl.name + "_train"
    c["dropout"] = TRAIN_DROPOUT
    c["step"] = "forward in training mode + backward for the input and every parameter; no optimizer"
    return c


def run_train(args, wl):
    """One step = training-mode forward (dropout on h) plus the whole backward pass of the block at
    the workload's shape, device-resident; e2e adds the host copies of the input and of the
    input gradient. flops: 6kdfN forward, 12kdfN backward."""
    from gemmallm_b200 import synthetic
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dt = synthetic.torch_dtype(wl.dtype)
    N, d, f, E, k = wl.tokens, wl.d_model, wl.d_ff, wl.n_experts, wl.top_k
    m = build_block(wl, dev, dt)
    for ex in m.experts:
        ex.dropout.p = TRAIN_DROPOUT
    m.train()
    x = synthetic.make_input(N, d, seed=1).to(dt).to(dev).view(1, N, d).requires_grad_(True)
    g = (torch.randn(N, d, generator=torch.Generator().manual_seed(5)) * 0.01).to(dt).to(dev).view(1, N, d)
    params = [p for p in m.parameters() if p.requires_grad]

    def step():
        out, aux = m(x)
        loss = (out.float() * g.float()).sum() + 0.01 * aux
        loss.backward()
        for p in params:
            p.grad = None
        gx, x.grad = x.grad, None
        return gx, loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if m.device_status() != 0:
        raise RuntimeError("device status non-zero after the warm-up")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / args.steps
    # end to end: input from pinned host memory, input gradient and loss back to the host
    x_host = synthetic.make_input(N, d, seed=1).to(dt).pin_memory()
    gx_host = torch.empty(N, d, dtype=dt).pin_memory()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        with torch.no_grad():
            x.view(N, d).copy_(x_host, non_blocking=True)
        gx, loss = step()
        gx_host.copy_(gx.view(N, d), non_blocking=True)
        _ = float(loss)
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / args.steps
    peaks, peak_kind = load_peaks()
    flops = 18.0 * k * d * f * N
    peak = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    es = 2
    line = {
        "metric": "moe_train_tokens_per_s", "value": N / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic", "config": train_config(wl),
        "run": {"parallelism": "single", "cuda_graph": False},
        "e2e": {"value": N / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": N * d * es,
                "d2h_bytes_per_step": N * d * es + 4, "ms_per_step": e2e_ms,
                "mode": "input copied in, input gradient and loss copied out, every step, one stream"},
        "gpu_launches": 26 * args.steps,   # the library's kernels per step (launch list in profiles/)
        "clocks": clocks.summary(),
        "roofline": {"kernel": "whole step: six grouped_gemm_tc2_kernel launches (two forward, four backward) "
                               "plus router, dispatch, combine, their backward kernels and the transposes",
                     "bound": "tensor", "achieved": flops / (ms_step * 1e-3) / 1e12, "peak": peak,
                     "unit": "TFLOP/s", "frac": flops / (ms_step * 1e-3) / 1e12 / peak, "traffic": None,
                     "peak_source": f"{peak_kind} bf16 sustained (the step is a seconds-long loop of GEMMs)",
                     "flops_per_step": flops},
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = train_reference_record(wl, 3)
    print(json.dumps(line), flush=True)


def cpu_train_step(wl, tokens):
    """The reference class (oracle/_ref) in training mode on the host cores: forward, the same
    loss, backward. Returns (kind, step function)."""
    from gemmallm_b200 import synthetic
    from oracle import make_ref
    dt = synthetic.torch_dtype(wl.dtype)
    d, E, f, k = wl.d_model, wl.n_experts, wl.d_ff, wl.top_k
    ref = make_ref.load()
    m = ref.MOE(d, num_experts=E, expansion_factor=f // d, dropout_ratio=TRAIN_DROPOUT, device="cpu")
    params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
        d, E, f, seed=0, gate_bias_kind=wl.gate_bias).items()}
    synthetic.load_into(m, params, torch.float32, "cpu")
    m.train()
    x = synthetic.round_to(synthetic.make_input(wl.tokens, d, seed=1), dt)[:tokens].clone().requires_grad_(True)
    g = torch.randn(tokens, d, generator=torch.Generator().manual_seed(5)) * 0.01

    def step():
        out, aux = m(x.view(1, tokens, d))
        loss = (out.view(tokens, d) * g).sum() + 0.01 * aux
        loss.backward()
        m.zero_grad(set_to_none=True)
        x.grad = None
    return step


def train_reference_times(wl, steps, warmup, limit_s):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tokens = wl.tokens
    step = cpu_train_step(wl, tokens)
    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    calls = steps + max(warmup - 1, 0)
    if first * calls > limit_s and tokens > 1024:
        tokens = max(1024, int(tokens * limit_s / (first * calls)) // 1024 * 1024)
        step = cpu_train_step(wl, tokens)
        step()
    for _ in range(max(warmup - 1, 0)):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sample = (f"all {tokens} tokens per step" if tokens == wl.tokens else
              f"first {tokens} of {wl.tokens} tokens per step (the whole batch would pass the time limit)")
    return times, cores, sample + ", fp32 on bf16-rounded values, forward + backward", tokens


def train_reference_record(wl, reps):
    times, cores, sample, tokens = train_reference_times(wl, reps, 1, 30.0)
    times.sort()
    return {"value": tokens / times[len(times) // 2], "unit": "tokens/s", "cores": cores,
            "kind": "reference", "sample": f"{sample}, median of {reps}"}


def run_train_reference(args, wl):
    times, cores, sample, tokens = train_reference_times(wl, args.steps, args.warmup, CPU_ARM_LIMIT_S)
    total = sum(times)
    value = tokens * args.steps / total
    line = {
        "impl": "reference", "metric": "moe_train_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": train_config(wl),
        "run": {"parallelism": "cpu", "threads": cores},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_stages(m, x2d, wl, dev, small_n: bool = False, reps: int = 20, mid_n: bool = False):
    """CUDA-event time of each stage, called through its own C-ABI entry point
    on the buffers of the module's workspace, on the current stream."""
    from gemmallm_b200 import _cabi
    from gemmallm_b200._cabi import lib, check
    N, d = x2d.shape
    f, E, k = wl.d_ff, wl.n_experts, wl.top_k
    code = _cabi.BF16 if wl.dtype == "bf16" else _cabi.F32
    buf, base, nbytes, lay = m._ws
    p = {n: base + off for n, off in lay.items()}
    plan = m._plan.base
    s = torch.cuda.current_stream(dev).cuda_stream
    out = torch.empty_like(x2d)
    gw, gb = m.gate.weight, m.gate.bias
    calls = {
        "router": lambda: lib.moe_b200_router(x2d.data_ptr(), gw.data_ptr(), gb.data_ptr(), N, d, E,
                                              k, code, p["logits"], p["idx"], p["w"],
                                              p["psum_part"], p["status"], s),
        "dispatch": lambda: lib.moe_b200_dispatch(x2d.data_ptr(), p["idx"], N, d, E, k, code,
                                                  p["scratch"], p["cnt_slot"], p["offsets"],
                                                  p["row_of"], p["perm"], p["psum_part"], p["psum"],
                                                  p["aux"], p["status"], s),
        "experts": lambda: lib.moe_b200_experts(p["perm"], p["offsets"], plan, N * k, d, f, E, code,
                                                0, p["h"], p["y"], p["status"], s),
        "combine": lambda: lib.moe_b200_combine(p["y"], p["row_of"], p["w"], None, N, d, k, code,
                                                out.data_ptr(), s),
    }
    if small_n:
        # the small-N path replaces router + dispatch by one single-block launch
        front = lambda: lib.moe_b200_front_small(
            x2d.data_ptr(), gw.data_ptr(), gb.data_ptr(), N, d, E, k, code, p["logits"], p["idx"],
            p["w"], p["cnt_slot"], p["offsets"], p["row_of"], p["perm"], p["psum"], p["aux"], s)
        if front() == 0:
            del calls["router"], calls["dispatch"]
            calls = {"front": front, **calls}
        splits = lib.moe_b200_decode_splits(f)
        ready = p["status"] + 4 * _cabi.READY_OFFSET
        calls["experts"] = lambda: lib.moe_b200_experts_decode_fused(
            p["perm"], p["offsets"], plan, N * k, d, f, E, p["h"], p["part"], ready, p["status"], s)
        if N * k >= E and N <= 128 and E <= 32:
            # the kernel the forward uses when most experts are hit (timed here without its overlap
            # with the routing kernel); "experts_sorted" is the kernel for a few hit experts
            calls["experts_sorted"] = calls["experts"]
            calls["experts"] = lambda: lib.moe_b200_experts_decode_spec(
                x2d.data_ptr(), p["idx"], p["offsets"], plan, N, k, d, f, E, p["h"], p["part"], ready,
                p["status"], s)
        calls["experts_gemv"] = lambda: lib.moe_b200_experts_gemv(
            p["perm"], p["offsets"], plan, N * k, d, f, E, p["h"], p["part"], s)
        if "experts_sorted" not in calls:
            # a row or two per expert: the forward uses the matrix-vector kernels
            calls["experts_fused"], calls["experts"] = calls["experts"], calls["experts_gemv"]
        calls["combine"] = lambda: lib.moe_b200_combine_decode(
            p["part"], splits, N * k, p["row_of"], p["idx"], p["w"], plan, E, None, N, d, k,
            out.data_ptr(), s)
    if mid_n:
        # single-launch front (blocks share the routing), streaming kernel on the sorted rows,
        # the small-N combine
        ks = lib.moe_b200_rows_splits(N * k, d, f, E)
        ready = p["status"] + 4 * _cabi.READY_OFFSET
        counter = ready + 4 * (_cabi.READY_INTS - 4)
        calls = {
            "front": lambda: lib.moe_b200_front_small_split(
                x2d.data_ptr(), gw.data_ptr(), gb.data_ptr(), N, d, E, k, code, p["logits"], p["idx"],
                p["w"], p["cnt_slot"], p["offsets"], p["row_of"], p["perm"], p["psum"], p["aux"],
                p["scratch"], counter, p["status"], s),
            "experts": lambda: lib.moe_b200_experts_rows(
                p["perm"], p["offsets"], plan, N * k, d, f, E, ks, p["h"], p["part"], ready,
                p["status"], s),
            "combine": lambda: lib.moe_b200_combine_decode(
                p["part"], ks, N * k, p["row_of"], p["idx"], p["w"], plan, E, None, N, d, k,
                out.data_ptr(), s),
        }
    res = {}
    for name, fn in calls.items():
        for _ in range(3):
            check(fn(), name)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / reps
    # the stage calls above share the workspace's status region with the forward: leave it clean
    m._view("status", torch.int32, (_cabi.READY_OFFSET + _cabi.READY_INTS,)).zero_()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    help="default: c1_uniform on one GPU, c4 (expert-parallel) on several; c3 = the whole "
                         "12-layer decoder forward with the block swapped in (one GPU); c1_uniform_train = "
                         "training-mode forward + backward of the block (one GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="one GPU, default workload: skip the decode-shaped sweep and the "
                         "expert-parallel workload on this GPU")
    ap.add_argument("--ep-placement", default="strided", choices=["strided", "lpt"])
    ap.add_argument("--ep-replicate", type=int, default=16,
                    help="expert-parallel: copy the N most popular experts (by the router-bias prior) "
                         "to every rank, on top of the even sharding; 0 = no copies")
    ap.add_argument("--no-graph", action="store_true", help="small-N workloads: time eager calls")
    ap.add_argument("--quick", action="store_true",
                    help="device-resident loop only (for profiler captures): no end-to-end leg, "
                         "no per-stage timing, no CPU baseline; prints a reduced line")
    args = ap.parse_args()
    from gemmallm_b200 import synthetic
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload is None:
        args.workload = "c1_uniform" if world == 1 else "c4"
    if args.workload == "c3":
        if int(os.environ.get("RANK", "0")) == 0:
            run_decoder_reference(args) if args.impl == "reference" else run_decoder(args)
        return
    if args.workload.endswith("_train"):
        if int(os.environ.get("RANK", "0")) == 0:
            wl = synthetic.WORKLOADS[args.workload[:-len("_train")]]
            run_train_reference(args, wl) if args.impl == "reference" else run_train(args, wl)
        return
    wl = synthetic.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    elif world > 1 and wl.name == "c4":
        run_ep(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
