#!/usr/bin/env python
"""Benchmark of the Mixture-of-Experts block: tokens/s and grouped-GEMM
fraction of the measured bf16 tensor peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one forward of the block over the workload's token batch. At N=1 the
workload is the bf16 prefill block (16384 tokens, d_model 1024, 8 experts,
d_ff 4096, top-2, uniform routing). Under torchrun every rank runs the same
block on its own token batch (tokens sharded, no data-path collective; weak
scaling). Rank 0 prints one JSON line.

``--impl reference`` times the CPU restatement of the reference block
(oracle/moe_oracle.py, bit-identical to the reference class at k=2) on this
host's cores instead.
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

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernels per step, from the ncu
# captures summarised under profiles/ (GEGLU pass + down pass)
NCU_TRAFFIC_BYTES = {"c1_uniform": 429.7e6 + 405.7e6, "c2_t64": 204.8e6 + 3.8e6}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
CPU_SAMPLE_TOKENS = 4096
L2_BYTES = 126e6


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


def workload_config(wl, extra):
    cfg = {"workload": wl.name, "tokens": wl.tokens, "d_model": wl.d_model,
           "n_experts": wl.n_experts, "d_ff": wl.d_ff, "top_k": wl.top_k, "routing": wl.gate_bias}
    cfg.update(extra)
    return cfg


def cpu_baseline(wl, tokens, repeats, warmup):
    """Oracle (port of the reference block) on the host cores, fp32 on
    bf16-rounded values: the reference cannot run in bf16."""
    from gemmallm_b200 import synthetic
    from oracle import moe_oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dt = synthetic.torch_dtype(wl.dtype)
    params = {n: synthetic.round_to(t, dt) for n, t in synthetic.make_params(
        wl.d_model, wl.n_experts, wl.d_ff, seed=0, gate_bias_kind=wl.gate_bias).items()}
    x = synthetic.round_to(synthetic.make_input(tokens, wl.d_model, seed=1), dt)
    with torch.no_grad():
        for _ in range(warmup):
            moe_oracle.moe_forward(x, params, wl.top_k)
        times = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            moe_oracle.moe_forward(x, params, wl.top_k)
            times.append(time.perf_counter() - t0)
    return times, cores


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = min(wl.tokens, CPU_SAMPLE_TOKENS)
    times, cores = cpu_baseline(wl, tokens, args.steps, args.warmup)
    total = sum(times)
    value = tokens * args.steps / total
    sample = f"first {tokens} of {wl.tokens} tokens per step, fp32 on bf16-rounded values"
    line = {
        "impl": "reference", "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(wl, {"parallelism": "cpu"}),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, wl):
    import torch.distributed as dist
    from gemmallm_b200 import MOE, _cabi, synthetic
    from gemmallm_b200._cabi import lib, check

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
        del params
    m.flags = getattr(args, "flags", 0)
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

    small_n = wl.dtype == "bf16" and N * k <= lib.moe_b200_decode_max_rows()
    # between the decode and the prefill sizes: the streaming kernels on sorted rows
    mid_n = (wl.dtype == "bf16" and not small_n and N * k <= 4096 and N <= 2048 and E <= 32
             and not (getattr(args, "flags", 0) & _cabi.FLAG_NO_ROWS_PATH))
    streaming = small_n or mid_n      # launch-bound from Python, bound by the weight stream on the GPU

    def capture(fn):
        """Small-N calls are launch-bound from Python: replay them as a CUDA graph."""
        if not streaming or args.no_graph:
            return None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g
        except Exception as exc:  # capture unsupported: time eager calls instead
            print(f"# CUDA graph capture failed ({exc}); timing eager calls", file=sys.stderr)
            torch.cuda.synchronize()
            return None

    # ---- device-resident throughput -------------------------------------
    replicas, steps_per_graph = [m], 1
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            m(x)
        torch.cuda.synchronize()
        if streaming and not args.no_graph:
            # A small-N step touches only the weights of the experts it hits, which can be less
            # than the L2: rotate over copies of the block so that no step finds its weights
            # cached by the step before, and put several steps into one graph, as a decoder
            # that captures all its layers would (the gap between two graph launches is not
            # the block's).
            hit = int((m.last["cnt_slot"].sum(0) > 0).sum())
            if N * k >= 2 * E and small_n:
                hit = E      # the routing-independent kernel streams every expert
            touched = hit * (3 * d * f + 2 * f + d) * es
            n_rep = max(1, -(-int(2 * L2_BYTES) // touched))
            for _ in range(n_rep - 1):
                r = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda").eval()
                r.to(device=dev, dtype=dt)
                r.load_state_dict(m.state_dict())
                r.flags = m.flags
                replicas.append(r)
            for r in replicas:
                for _ in range(3):
                    r(x)
            torch.cuda.synchronize()
            steps_per_graph = n_rep * max(1, 8 // n_rep)
        graph = capture(lambda: [replicas[i % len(replicas)](x) for i in range(steps_per_graph)])
        graph1 = capture(lambda: m(x)) if steps_per_graph > 1 else graph
        if graph is None:
            steps_per_graph = 1
        step = graph.replay if graph is not None else (lambda: m(x))
        step1 = graph1.replay if graph1 is not None else (lambda: m(x))
        for _ in range(3):
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            ev0.record()
            for _ in range(args.steps // steps_per_graph):
                step()
            for _ in range(args.steps % steps_per_graph):
                step1()
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
                              "quick": True, "config": workload_config(wl, {})}), flush=True)
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
            e2e_graph = capture(e2e_step)
            run_e2e = e2e_graph.replay if e2e_graph is not None else e2e_step
            run_e2e()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                run_e2e()
                torch.cuda.current_stream().synchronize()   # output and loss are on the host now
                loss = float(aux_host[0])
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
    two_pass = bool(m.flags & _cabi.FLAG_DECODE_TWO_PASS)
    stage_ms, launches_per_step = {}, ((4 if two_pass else 3) if small_n else (3 if mid_n else 5))
    if rank == 0:
        stage_ms = time_stages(m, x.view(N, d), wl, dev, small_n, mid_n=mid_n)
    peaks, peak_kind = load_peaks()
    line = None
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
        line = {
            "metric": "moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic",
            "config": workload_config(wl, {
                "parallelism": "single" if world == 1 else f"tokens sharded over {world} ranks, experts replicated",
                "l2": ("working set per step (expert weights streamed once per step) exceeds the 126 MB L2"
                       if len(replicas) == 1 else
                       f"{len(replicas)} copies of the block's weights used in rotation: the weights one step "
                       "touches were evicted by the steps in between (together over twice the 126 MB L2)"),
                "cuda_graph": graph is not None, "steps_per_graph": steps_per_graph}),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": N * d * es,
                    "d2h_bytes_per_step": N * d * es + 4, "ms_per_step": e2e_ms / args.steps,
                    "mode": e2e_mode},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"kernel": "grouped_gemm_tc2_kernel (GEGLU pass + down pass, CTA pairs)",
                         "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                         "peak_source": f"{peak_kind} bf16 burst", "flops_per_step": flops,
                         "ms": stage_ms["experts"]},
            "stages_ms": stage_ms,
            "stages_hbm": {n: {"bytes": b, "gbs": b / (stage_ms[n] * 1e-3) / 1e9,
                               "frac": b / (stage_ms[n] * 1e-3) / 1e9 / hbm}
                           for n, b in stage_bytes.items()},
        }
        if streaming:
            # weight streaming: bytes of the distinct experts hit, plus router weights, x in, out
            hit = int((m.last["cnt_slot"].sum(0) > 0).sum())
            wbytes = hit * (3 * d * f + 2 * f + d) * es
            nbytes_step = wbytes + E * d * es + 2 * N * d * es
            gbs_step = nbytes_step / (ms_step * 1e-3) / 1e9
            gbs_experts = wbytes / (stage_ms["experts"] * 1e-3) / 1e9
            line["roofline"] = {
                "kernel": ("decode_spec_kernel / decode_fused_kernel (GEGLU + split-K down tiles, one launch)"
                           if small_n else "decode_spec_kernel<SORTED> (GEGLU + split-K down tiles on sorted rows)"),
                "bound": "hbm", "achieved": gbs_experts, "peak": hbm, "unit": "GB/s",
                "frac": gbs_experts / hbm, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                "peak_source": f"{peak_kind} copy",
                "bytes_per_step": wbytes, "experts_hit": hit, "ms": stage_ms["experts"],
                "whole_step_gbs": gbs_step, "whole_step_frac": gbs_step / hbm}
        if world == 1 and not args.no_cpu_baseline:
            tokens = min(N, CPU_SAMPLE_TOKENS)
            times, cores = cpu_baseline(wl, tokens, 3 if N > 256 else 20, 1)
            times.sort()
            line["cpu_baseline"] = {
                "value": tokens / times[len(times) // 2], "unit": "tokens/s", "cores": cores,
                "kind": "port",
                "sample": f"first {tokens} of {N} tokens, median of 3, fp32 on bf16-rounded values"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    m.flags = args.ep_flags
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
    x_host = synthetic.make_input(Nl, d, seed=1 + rank).to(dt).pin_memory()
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

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
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
        status = max_over_ranks(float(m.device_status()))
        if status != 0:
            raise RuntimeError(f"device status {status} after the timed region")
        # end to end: pinned host input in, output and loss back, every step (pipelined)
        barrier()
        e2e_ms = max_over_ranks(pipelined_e2e(m, x_host, out_host, aux_host, Nl, d, dt, dev, args.steps))
        barrier()
        # grouped GEMMs alone on this rank's received rows
        rows = int(m.last["offsets_local"][-1])
        st = m._state
        recv_x = st["hdl"].buffer_ptrs[rank] + st["symm_layout"]["recv_x"]
        hbuf = st["ws_base"] + st["ws_layout"]["h"]
        offs = st["ws_base"] + st["ws_layout"]["offsets_local"]
        stat = st["ws_base"] + st["ws_layout"]["status"]
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
    single = None
    if rank == 0 and not args.quick:
        # the same workload on this one GPU (all experts local, no exchange), for the speed-up
        from gemmallm_b200 import MOE
        del m
        torch.cuda.empty_cache()
        m1 = MOE(d, num_experts=E, d_ff=f, top_k=k, device="cuda").eval()
        m1.to(device=dev, dtype=dt)
        with torch.no_grad():
            m1.gate.weight.copy_(gate_w)
            m1.gate.bias.copy_(gate_b)
            for e, ex in enumerate(m1.experts):
                pe = synthetic.make_expert(d, f, e, 0)
                ex.gate_and_up.weight.copy_(pe["w1"])
                ex.down.weight.copy_(pe["w2"])
                ex.gate_and_up.bias.zero_()
                ex.down.bias.zero_()
            x1 = synthetic.make_input(N, d, seed=1).to(dt).to(dev).view(1, N, d)
            for _ in range(3):
                m1(x1)
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(10):
                m1(x1)
            t1.record()
            torch.cuda.synchronize()
            single = t0.elapsed_time(t1) / 10
        del m1, x1
    if rank == 0:
        peaks, peak_kind = load_peaks()
        peak = float(peaks["bf16_tflops"])
        es = 2
        per_rank = [{"rows": int(g[0]), "gemm_ms": float(g[1]),
                     "tflops": 6.0 * d * f * float(g[0]) / (float(g[1]) * 1e-3) / 1e12} for g in gathered]
        busiest = max(per_rank, key=lambda r: r["gemm_ms"])
        share = max(r["rows"] for r in per_rank) / float(N * k)
        ms_step = ms_total / args.steps
        line = {
            "metric": "moe_tokens_per_s", "value": N * args.steps / (ms_total * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": workload_config(wl, {
                "parallelism": f"ep{world}: tokens and experts sharded over {world} ranks, "
                               f"{args.ep_placement} expert placement, {args.ep_replicate} hottest experts copied to every rank, "
                               "peer-store all-to-all",
                "l2": "per-rank working set (received rows, h, owned expert weights) exceeds the 126 MB L2"}),
            "e2e": {"value": N * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": Nl * d * es * world, "d2h_bytes_per_step": (Nl * d * es + 4) * world,
                    "ms_per_step": e2e_ms / args.steps,
                    "mode": "per rank three streams: copy-in, compute, copy-out of consecutive steps overlap"},
            "gpu_launches": 9 * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"kernel": "grouped_gemm_tc2_kernel (GEGLU pass + down pass) on the busiest rank",
                         "bound": "tensor", "achieved": busiest["tflops"], "peak": peak,
                         "unit": "TFLOP/s", "frac": busiest["tflops"] / peak, "traffic": None,
                         "peak_source": f"{peak_kind} bf16 burst", "ms": busiest["gemm_ms"]},
            "ep": {"per_rank": per_rank, "max_rank_share_of_rows": share,
                   "balance_limited_speedup": 1.0 / share,
                   "gemm_ms_over_step_ms": busiest["gemm_ms"] / ms_step,
                   "same_workload_on_one_gpu_ms_per_step": single,
                   "speedup_vs_one_gpu": (single / ms_step) if single else None},
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


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
                                                m.flags, p["h"], p["y"], p["status"], s),
        "combine": lambda: lib.moe_b200_combine(p["y"], p["row_of"], p["w"], None, N, d, k, code,
                                                out.data_ptr(), s),
    }
    if small_n:
        # the small-N path replaces router + dispatch by one single-block launch
        if lib.moe_b200_front_small(x2d.data_ptr(), gw.data_ptr(), gb.data_ptr(), N, d, E, k, code,
                                    p["logits"], p["idx"], p["w"], p["cnt_slot"], p["offsets"],
                                    p["row_of"], p["perm"], p["psum"], p["aux"], s) == 0:
            del calls["router"], calls["dispatch"]
            calls = {"front": lambda: lib.moe_b200_front_small(
                x2d.data_ptr(), gw.data_ptr(), gb.data_ptr(), N, d, E, k, code, p["logits"], p["idx"],
                p["w"], p["cnt_slot"], p["offsets"], p["row_of"], p["perm"], p["psum"], p["aux"], s),
                **calls}
        splits = lib.moe_b200_decode_splits(f)
        ready = p["status"] + 4 * _cabi.READY_OFFSET
        calls["experts"] = lambda: lib.moe_b200_experts_decode_fused(
            p["perm"], p["offsets"], plan, N * k, d, f, E, p["h"], p["part"], ready, p["status"], s)
        if N * k >= 2 * E and N <= 128 and E <= 32 and not (m.flags & (_cabi.FLAG_DECODE_NO_SPEC | _cabi.FLAG_DECODE_TWO_PASS)):
            # the kernel the forward uses when most experts are hit (timed here without its overlap
            # with the routing kernel); "experts_sorted" is the kernel for a few hit experts
            calls["experts_sorted"] = calls["experts"]
            calls["experts"] = lambda: lib.moe_b200_experts_decode_spec(
                x2d.data_ptr(), p["idx"], p["offsets"], plan, N, k, d, f, E, p["h"], p["part"], ready,
                p["status"], s)
        calls["experts_two_pass"] = lambda: lib.moe_b200_experts_decode(
            p["perm"], p["offsets"], plan, N * k, d, f, E, p["h"], p["part"], p["status"], s)
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
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    help="default: c1_uniform on one GPU, c4 (expert-parallel) on several")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-placement", default="strided", choices=["strided", "lpt"])
    ap.add_argument("--ep-replicate", type=int, default=16,
                    help="expert-parallel: copy the N most popular experts (by the router-bias prior) "
                         "to every rank, on top of the even sharding; 0 = no copies")
    ap.add_argument("--ep-flags", type=int, default=0, help="flags for moe_b200_ep_forward")
    ap.add_argument("--flags", type=int, default=0, help="flags for moe_b200_forward (one GPU)")
    ap.add_argument("--no-graph", action="store_true", help="small-N workloads: time eager calls")
    ap.add_argument("--quick", action="store_true",
                    help="device-resident loop only (for profiler captures): no end-to-end leg, "
                         "no per-stage timing, no CPU baseline; prints a reduced line")
    args = ap.parse_args()
    from gemmallm_b200 import synthetic
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload is None:
        args.workload = "c1_uniform" if world == 1 else "c4"
    wl = synthetic.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    elif world > 1 and wl.name == "c4":
        run_ep(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
