#!/usr/bin/env python3
"""Benchmark of the optimizer-step engine: fused AdamW + global-norm clip + bf16 shadow.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

One "step" is one pass of the hot path over one parameter set: the gradient-norm
reduction and the fused update (clip coefficient folded in, bf16 shadow written in the
same pass) — two kernel launches. At one GPU the workload is the Llama-style 1.3B
parameter set; at N > 1 it is the Llama-3-8B-shaped set sharded ZeRO-1 style
(reduce-scatter of gradients, clip, shard update, all-gather of bf16 shadows).

Prints ONE JSON line. `value` is parameters updated per second with everything resident
in HBM; `e2e` is the same step driven through the C ABI's host-buffer entry point, with
the gradients copied from page-locked host memory and the norm read back inside the
timed region; `roofline` rates the update kernel against the measured HBM copy
bandwidth; `cpu_baseline` is the CPU restatement of the reference's host optimizer timed
on this machine's cores on a bounded sample of the same workload.

`--impl reference` times that CPU path alone (the reference is Go and cannot be built
in this image, so its arithmetic is run from the C restatement under oracle/).
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

METRIC = "fused AdamW+clip+bf16-shadow step throughput"
UNIT = "Gparams/s"
BYTES_UPDATE = 30   # R p,g,m,v (16) + W p,m,v (12) + W bf16 (2)
BYTES_NORM = 4      # R g
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (MEASURED_PEAKS.json absent)"


# DRAM bytes per parameter of one launch, from the ncu captures summarised under profiles/
# (oe_adamw_fused_gpt110m_ncu_full.md, oe_grad_sumsq_gpt110m_ncu_full.md): dram__bytes_read.sum +
# dram__bytes_write.sum over 109,630,464 parameters. Traffic grows in proportion to the parameter
# count, so the figure is scaled to the launch that is timed.
NCU_TRAFFIC_BYTES_PER_PARAM = {"oe_adamw_fused_bytes_per_param": 29.50, "oe_grad_sumsq_bytes_per_param": 4.03}


def ncu_traffic_per_param():
    return NCU_TRAFFIC_BYTES_PER_PARAM


def bind_to_gpu_numa_node(gpu_index: int):
    """Pins this process to the CPUs of the NUMA node the GPU hangs off, so that the page-locked
    staging memory it allocates next (first touch) and the threads that feed the copies are local to
    the GPU's PCIe root: what a host feeding eight GPUs at once has to do to keep every link busy.
    Returns a short description for the JSON line, or None when the topology cannot be read."""
    try:
        import torch
        props = torch.cuda.get_device_properties(gpu_index)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return {"gpu": gpu_index, "pci": bus, "numa_node": node, "cpus": len(allowed)}
    except Exception:
        return None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------
# CPU path (the reference's host optimizer, restated in C under oracle/)
# ---------------------------------------------------------------------------------------
def _host_available_bytes() -> int:
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        try:
            return os.sysconf("SC_AVPHYS_PAGES") * os.sysconf("SC_PAGE_SIZE")
        except Exception:
            return 0


def _synthetic(n: int, std: float, block):
    """n float32 values of the given spread: one seeded block of normals repeated (the CPU path's speed
    does not depend on the values, and drawing 1.3 B fresh normals per array would take longer than the
    timed steps)."""
    import numpy as np
    out = np.empty(n, np.float32)
    scaled = (block * np.float32(std)).astype(np.float32)
    for a in range(0, n, scaled.size):
        k = min(scaled.size, n - a)
        out[a:a + k] = scaled[:k]
    return out


def cpu_reference_run(ps, sample_params: int, steps: int, warmup: int, cores: int):
    """Times clip (serial float64 sum + in-place scale) and AdamW (per-tensor worker split)
    on the leading tensors of the workload up to sample_params elements (all of it when that
    many fit)."""
    import numpy as np

    from gograd_b200 import paramsets
    from oracle import oracle
    sample = paramsets.scaled(ps, sample_params)
    rng = np.random.default_rng(ps.grad_seed)
    block = rng.standard_normal(1 << 24, dtype=np.float32)
    params = [_synthetic(s.numel, 0.02, block) for s in sample.params]
    grads0 = [_synthetic(s.numel, ps.grad_std, block[::-1]) for s in sample.params]
    wd = sample.groups[0].weight_decay
    opt = oracle.OracleAdamW(params, lr=ps.hparams["lr"], weight_decay=wd, beta1=ps.hparams["beta1"],
                             beta2=ps.hparams["beta2"], eps=ps.hparams["eps"], max_procs=cores)
    n = sum(s.numel for s in sample.params)
    grads = [np.empty_like(g) for g in grads0]
    times = []
    for it in range(warmup + steps):
        for dst, src in zip(grads, grads0):   # fresh gradients; the copy is outside the timed region
            np.copyto(dst, src)
        t0 = time.perf_counter()
        if ps.max_norm > 0:
            oracle.clip_grad_norm(grads, ps.max_norm)
        opt.step(grads)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    whole = n == ps.numel
    return {"value": n / sec / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": (f"the whole {ps.key} set" if whole else f"{len(sample.params)} leading tensors of {ps.key}") +
                      f" = {n} params, {steps} steps after {warmup} warm-up; "
                      "C restatement of the Go host optimizer (AdamW split over min(cores, n/65536) workers per tensor, "
                      "clip single-threaded, as the reference)",
            "ms_per_step_sample": sec * 1e3}, n, sec


def run_reference_arm(args):
    """The reference's CPU implementation of the path on this host's cores: the configured number
    of steps and warm-up steps, on the whole parameter set when the host can hold it (20 bytes per
    parameter: p, g, m, v and the per-step fresh copy of g) and a step stays within seconds, else on
    the leading tensors that fit, which config.note then says."""
    from gograd_b200 import paramsets
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    key = args.workload if args.workload != "auto" else ("llama1b" if args.gpus == 1 else "llama8b")
    ps = paramsets.get(key)
    cores = os.cpu_count() or 1
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    available = _host_available_bytes()
    by_memory = int(available * 0.7) // 20
    # about 0.6 Gparams/s on 16 cores: 2e9 parameters keep a step near three seconds, so that
    # steps + warm-up of the default run end within a few minutes
    by_time = 2_000_000_000
    limit = args.reference_sample_params or min(by_memory, by_time)
    limit = max(limit, 1)
    note = ("the reference is Go (no toolchain in this image): CPU host path restated in C, all host threads; "
            f"host memory available {available / 1e9:.0f} GB")
    if limit < ps.numel:
        note += (f"; the {ps.numel}-parameter set is timed on its leading tensors up to {limit} parameters "
                 "(host memory or step-time bound) and reported per parameter")
    base, n, sec = cpu_reference_run(ps, limit, steps, warmup, cores)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": key, "params_total": ps.numel, "params_in_sample": n, "note": note},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------
# engine arm, one GPU
# ---------------------------------------------------------------------------------------
def run_single(args):
    import torch

    import gograd_b200 as eng
    from gograd_b200 import paramsets, workload
    from gograd_b200.engine import OE_WRITE_SHADOW

    key = args.workload if args.workload != "auto" else "llama1b"
    ps = paramsets.get(key)
    torch.cuda.set_device(0)
    eng.init(0)
    state = workload.materialize(ps, "cuda:0")
    plan = eng.Plan(state.descs(), 0, args.chunk)
    if args.variant:
        plan.set_variant(args.variant)
    if args.step_grid == "units":
        plan.set_tuning(eng.engine.OE_TUNE_STEP_GRID, 1)
    n_params = state.numel
    hp = ps.hparams
    flags = OE_WRITE_SHADOW if ps.bf16_shadow else 0
    stream = torch.cuda.current_stream()
    step_no = [0]

    is_sgd = ps.optimizer == "sgd"
    bytes_update = (20 if hp.get("momentum", 0) > 0 else 12) if is_sgd else 28
    bytes_update += 2 if ps.bf16_shadow else 0

    def hparams():
        step_no[0] += 1
        if is_sgd:
            return eng.SGDHParams(hp["lr"], hp["momentum"], hp["dampening"], ps.max_norm, flags)
        b1, b2 = workload.bias_corrections(hp["beta1"], hp["beta2"], step_no[0])
        return eng.AdamWHParams(hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], b1, b2, ps.max_norm, flags)

    def one_step(events=None):
        if events is not None:
            events[0].record(stream)
        if ps.max_norm > 0:
            plan.grad_norm(0, stream)
        if events is not None:
            events[1].record(stream)
        if is_sgd:
            plan.sgd_step(hparams(), stream)
        else:
            plan.adamw_step(hparams(), stream)
        if events is not None:
            events[2].record(stream)

    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()

    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    eng.launch_count_reset()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for k in range(args.steps):
        one_step(ev[k])
    stop.record(stream)
    torch.cuda.synchronize()
    launches = eng.launch_count()
    total_ms = start.elapsed_time(stop)
    ms_per_step = total_ms / args.steps
    norm_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    upd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    norm_value, _ = plan.read_norm(stream)

    # ---- optional: the same step captured once in a CUDA graph and replayed ----------------
    graph_info = None
    if args.graph:
        step_dev = torch.full((1,), step_no[0], dtype=torch.int32, device="cuda:0")
        lr_dev = torch.full((1,), hp["lr"], dtype=torch.float32, device="cuda:0")
        def captured_step():
            if ps.max_norm > 0:
                plan.grad_norm(0)
            if is_sgd:
                plan.sgd_step(eng.SGDHParams(hp["lr"], hp["momentum"], hp["dampening"], ps.max_norm, flags,
                                             step_dev=step_dev.data_ptr(), lr_dev=lr_dev.data_ptr()))
            else:
                plan.adamw_step(eng.AdamWHParams(hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], max_norm=ps.max_norm,
                                                 flags=flags, step_dev=step_dev.data_ptr(), lr_dev=lr_dev.data_ptr()))

        def replay_ms(steps_per_graph):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(steps_per_graph):
                    captured_step()
            replays = max(1, args.steps // steps_per_graph)
            for _ in range(args.warmup):
                g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(replays):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / (replays * steps_per_graph)

        one = replay_ms(1)
        graph_info = {"ms_per_step": one, "value": n_params / (one * 1e-3) / 1e9,
                      "note": "one captured step (device step counter and learning rate) replayed"}
        if args.graph_steps > 1:
            # several steps per graph: the host's cost of launching a graph is shared, what is
            # left is the device-side time of a step
            many = replay_ms(args.graph_steps)
            graph_info["steps_per_graph"] = args.graph_steps
            graph_info["ms_per_step_many"] = many
            graph_info["value_many"] = n_params / (many * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point -------------------------------
    e2e = None
    if not args.no_e2e and not is_sgd:
        try:
            host_grads = [torch.empty(t.numel(), dtype=torch.float32).pin_memory() for t in state.g]
            for hg, g in zip(host_grads, state.g):
                hg.copy_(g)
            torch.cuda.synchronize()
            e2e_steps = max(3, min(args.steps, 10))
            plan.adamw_step_from_host(hparams(), host_grads, stream)  # warm-up
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                plan.adamw_step_from_host(hparams(), host_grads, stream)
            dt = (time.perf_counter() - t0) / e2e_steps
            e2e = {"value": n_params / dt / 1e9, "unit": UNIT, "h2d_bytes_per_step": 4 * n_params,
                   "d2h_bytes_per_step": 32, "ms_per_step": dt * 1e3, "steps": e2e_steps,
                   "api": "oe_adamw_step_from_host (gradients from page-locked host memory, norm read back, stream "
                          "synchronised every step)"}
            del host_grads
        except Exception as exc:  # pinned allocation can fail on a small host
            e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 4 * n_params, "d2h_bytes_per_step": 32,
                   "error": str(exc)[:200]}
    clocks = sampler.stop()

    peak, peak_kind = measured_peak()
    BYTES_UPDATE, BYTES_NORM = bytes_update, (4 if ps.max_norm > 0 else 0)
    achieved = BYTES_UPDATE * n_params / (upd_ms * 1e-3) / 1e9
    traffic = ncu_traffic_per_param().get("oe_adamw_fused_bytes_per_param") if (not is_sgd and ps.bf16_shadow) else None
    roofline = {"bound": "hbm", "kernel": "oe_sgd_fused" if is_sgd else "oe_adamw_fused", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": peak_kind,
                "traffic": None if traffic is None else traffic * n_params,
                "traffic_source": None if traffic is None else
                "not measured in this run: dram__bytes_read.sum + dram__bytes_write.sum per parameter from the ncu capture "
                "summarised in profiles/oe_adamw_fused_gpt110m_ncu_full.md (109.6 M-parameter set), scaled by the parameter count",
                "algorithmic_bytes_per_launch": BYTES_UPDATE * n_params, "kernel_ms": upd_ms,
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "norm_kernel": {"kernel": "oe_grad_sumsq", "kernel_ms": norm_ms,
                                "achieved": BYTES_NORM * n_params / (norm_ms * 1e-3) / 1e9,
                                "frac": BYTES_NORM * n_params / (norm_ms * 1e-3) / 1e9 / peak},
                "whole_step": {"bytes_per_param": BYTES_UPDATE + BYTES_NORM,
                               "achieved": (BYTES_UPDATE + BYTES_NORM) * n_params / (ms_per_step * 1e-3) / 1e9,
                               "frac": (BYTES_UPDATE + BYTES_NORM) * n_params / (ms_per_step * 1e-3) / 1e9 / peak}}

    cpu_baseline = None
    if not args.no_cpu_baseline:
        cpu_baseline, _, _ = cpu_reference_run(ps, args.cpu_sample_params, 5, 1, os.cpu_count() or 1)

    line = {
        "metric": METRIC if key == "llama1b" else f"fused {ps.optimizer} step throughput ({key})",
        "value": n_params / (ms_per_step * 1e-3) / 1e9, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": key, "title": ps.title, "params": n_params, "tensors": len(ps.params),
                   "optimizer": ps.optimizer, "max_norm": ps.max_norm, "bf16_shadow": ps.bf16_shadow,
                   "chunk_elems": plan.info(5), "grid_update": plan.info(3), "grid_norm": plan.info(4),
                   "variant": args.variant or "default",
                   "l2": "inputs larger than L2: %.1f GB of p/g/m/v/shadow per step" % ((18 * n_params) / 1e9),
                   "grad_norm": norm_value},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
        "gpu_launches": launches,
    }
    if graph_info:
        line["graph_replay"] = graph_info
    print(json.dumps(line))
    plan.close()
    return 0


def run_secondary(args):
    """Times the other kernels of the path on one large synthetic tensor set (CUDA events, median):
    SGD update, in-place clip, stand-alone bf16 cast, gradient zeroing, the allocation-free norm."""
    import torch

    import gograd_b200 as eng
    from gograd_b200 import _lib, paramsets, workload

    ps = paramsets.get(args.workload if args.workload != "auto" else "llama1b")
    torch.cuda.set_device(0)
    eng.init(0)
    state = workload.materialize(ps, "cuda:0")
    n = state.numel
    stream = torch.cuda.current_stream()
    peak, peak_kind = measured_peak()

    def timed(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in ev:
            a.record(stream)
            fn()
            b.record(stream)
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev)

    out = {}

    def record(name, bytes_per_param, ms):
        gbs = bytes_per_param * n / (ms * 1e-3) / 1e9
        out[name] = {"bytes_per_param": bytes_per_param, "ms": ms, "GB/s": gbs, "frac_of_peak": gbs / peak}

    flags1 = [torch.zeros(1, device="cuda:0") for _ in state.p]
    descs = [eng.TensorDesc(state.p[i], state.g[i], state.s1[i], flags1[i], state.shadow[i]) for i in range(len(state.p))]
    plan = eng.Plan(descs, 0, args.chunk)
    if args.step_grid == "units":
        plan.set_tuning(eng.engine.OE_TUNE_STEP_GRID, 1)
    record("oe_sgd_fused momentum (20 B)", 20, timed(lambda: plan.sgd_step(eng.SGDHParams(1e-3, 0.9), stream)))
    record("oe_sgd_fused momentum + shadow (22 B)", 22,
           timed(lambda: plan.sgd_step(eng.SGDHParams(1e-3, 0.9, flags=eng.engine.OE_WRITE_SHADOW), stream)))
    plain = eng.Plan([eng.TensorDesc(state.p[i], state.g[i]) for i in range(len(state.p))], 0, args.chunk)
    if args.step_grid == "units":
        plain.set_tuning(eng.engine.OE_TUNE_STEP_GRID, 1)
    record("oe_sgd_fused plain (12 B)", 12, timed(lambda: plain.sgd_step(eng.SGDHParams(1e-3), stream)))
    plain.grad_norm(0, stream)
    # Halving max_norm on every call keeps the norm above it, so the scale kernel really rewrites
    # the gradients each time it is timed.
    limit = [1.0]

    def clip_harder():
        limit[0] *= 0.5
        plain.clip_grad_norm(limit[0], 0, stream)

    record("oe_grad_sumsq + oe_scale_grads, clipping (4 + 8 B)", 12, timed(clip_harder))
    record("oe_grad_sumsq + oe_scale_grads, not clipping (4 + 0 B)", 4, timed(lambda: plain.clip_grad_norm(1e30, 0, stream)))
    record("oe_zero_grads (4 B)", 4, timed(lambda: plain.zero_grads(stream)))
    big = max(range(len(state.p)), key=lambda i: state.p[i].numel())
    src, dst = state.p[big], state.shadow[big]
    lib = _lib.lib()
    s_int = int(stream.cuda_stream)
    norm_out = torch.zeros(1, device="cuda:0")

    def record_n(name, bytes_per_elem, elems, ms):
        gbs = bytes_per_elem * elems / (ms * 1e-3) / 1e9
        out[name] = {"bytes_per_param": bytes_per_elem, "elements": elems, "ms": ms, "GB/s": gbs, "frac_of_peak": gbs / peak}

    # the two per-buffer entry points at three sizes: one tensor (a 50-70 us launch, ramp and tail
    # included), every tensor of the set back to back, and one buffer that streams for a millisecond
    record_n("oe_cast_bf16 (6 B), one %d-element tensor" % src.numel(), 6, src.numel(),
             timed(lambda: eng.cast_bf16(src, dst, stream)))

    def cast_all():
        for a, b in zip(state.p, state.shadow):
            eng.cast_bf16(a, b, stream)

    record_n("oe_cast_bf16 (6 B), all %d tensors back to back" % len(state.p), 6, n, timed(cast_all, iters=5, warm=2))
    record_n("oe_grad_norm_static (4 B), one %d-element tensor" % src.numel(), 4, src.numel(),
             timed(lambda: _lib.check(lib.oe_grad_norm_static(0, src.data_ptr(), src.numel(), norm_out.data_ptr(), s_int))))

    def norm_all():
        for a in state.g:
            _lib.check(lib.oe_grad_norm_static(0, a.data_ptr(), a.numel(), norm_out.data_ptr(), s_int))

    record_n("oe_grad_norm_static (4 B), all %d tensors back to back" % len(state.g), 4, n, timed(norm_all, iters=5, warm=2))
    long_elems = 1 << 30
    long_src = torch.empty(long_elems, dtype=torch.float32, device="cuda:0").normal_(0.0, 1e-3)
    long_dst = torch.empty(long_elems, dtype=torch.bfloat16, device="cuda:0")
    record_n("oe_cast_bf16 (6 B), one 2^30-element buffer", 6, long_elems, timed(lambda: eng.cast_bf16(long_src, long_dst, stream)))
    record_n("oe_grad_norm_static (4 B), one 2^30-element buffer", 4, long_elems,
             timed(lambda: _lib.check(lib.oe_grad_norm_static(0, long_src.data_ptr(), long_elems, norm_out.data_ptr(), s_int))))
    record_n("oe_grad_sumsq (4 B), the plan's norm over the whole set, for comparison", 4, n, timed(lambda: plain.grad_norm(0, stream)))
    print(json.dumps({"secondary_kernels": out, "params": n, "workload": ps.key, "peak_GBs": peak, "peak_kind": peak_kind}))
    return 0


def run_buffer_kernels(args):
    """The two per-buffer entry points (oe_cast_bf16, oe_grad_norm_static) on ONE buffer of
    --buffer-elems fp32 elements: a small, self-contained case (for a profiler capture, say)."""
    import torch

    import gograd_b200 as eng
    from gograd_b200 import _lib

    torch.cuda.set_device(0)
    eng.init(0)
    n = args.buffer_elems
    stream = torch.cuda.current_stream()
    s_int = int(stream.cuda_stream)
    peak, peak_kind = measured_peak()
    src = torch.empty(n, dtype=torch.float32, device="cuda:0").normal_(0.0, 1e-3)
    dst = torch.empty(n, dtype=torch.bfloat16, device="cuda:0")
    norm_out = torch.zeros(1, device="cuda:0")
    lib = _lib.lib()

    def timed(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in ev:
            a.record(stream)
            fn()
            b.record(stream)
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev)

    out = {}
    for name, bytes_per, fn in (
            ("oe_cast_bf16", 6, lambda: eng.cast_bf16(src, dst, stream)),
            ("oe_grad_norm_static", 4, lambda: _lib.check(lib.oe_grad_norm_static(0, src.data_ptr(), n, norm_out.data_ptr(), s_int)))):
        ms = timed(fn, iters=args.steps, warm=args.warmup)
        gbs = bytes_per * n / (ms * 1e-3) / 1e9
        out[name] = {"bytes_per_element": bytes_per, "ms": ms, "GB/s": gbs, "frac_of_peak": gbs / peak}
    ok = bool(torch.equal(dst.view(torch.int16), src.to(torch.bfloat16).view(torch.int16)))
    want = float(src.double().pow(2).sum().sqrt().item())
    print(json.dumps({"buffer_kernels": out, "elements": n, "cast_equals_rne": ok,
                      "norm_rel_err_vs_float64": abs(float(norm_out.item()) - want) / want, "peak_GBs": peak, "peak_kind": peak_kind}))
    return 0 if ok else 3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--variant", default="")
    ap.add_argument("--chunk", type=int, default=0)
    ap.add_argument("--step-grid", default="persistent", choices=["persistent", "units"],
                    help="N = 1: grid of the update launch (a persistent grid, or one CTA per work unit in table order)")
    ap.add_argument("--comm", default="abi", choices=["peer", "abi", "nccl"],
                    help="N > 1: fused peer-memory kernels ordered by tiny NCCL all-reduces (peer) or by the library's own "
                         "bounded exchanges, one C call per step (abi); or NCCL reduce-scatter / all-gather around the "
                         "single-GPU kernels (nccl)")
    ap.add_argument("--multicast", action="store_true", help="N > 1: shadow stores through the NVLink multicast mapping")
    ap.add_argument("--push-order", default="ascending", choices=["ascending", "rotated"])
    ap.add_argument("--reduce-first", default="rank0", choices=["rank0", "rotated"])
    ap.add_argument("--reduce-grid", type=int, default=0)
    ap.add_argument("--update-grid", type=int, default=0)
    ap.add_argument("--push-warp-rotate", default="", choices=["", "on", "off"])
    ap.add_argument("--ce-pull-sources", type=int, default=None,
                    help="N > 1, --comm abi: peers whose gradient range a copy stages before the pull kernel (default: the library's choice; 0 = none)")
    ap.add_argument("--ce-push-targets", type=int, default=None,
                    help="N > 1, --comm abi: ranks served by a shadow copy after the update kernel (default: the library's choice; 0 = none)")
    ap.add_argument("--staging-readers", action="store_true",
                    help="N > 1, --comm abi: the staged gradient ranges are read by the reducing rank instead of written by their owners")
    ap.add_argument("--sweep", action="store_true",
                    help="N > 1: time the two peer kernels over every launch-shape knob instead of the step")
    ap.add_argument("--no-parity-check", action="store_true", help="N > 1: skip the oracle check of one step before the warm-up")
    ap.add_argument("--secondary", action="store_true", help="time the other kernels of the path instead of the step")
    ap.add_argument("--buffer-elems", type=int, default=0,
                    help="time only the per-buffer entry points (bf16 cast, allocation-free norm) on one buffer of this many elements")
    ap.add_argument("--graph", action="store_true", help="also time the step captured in a CUDA graph and replayed")
    ap.add_argument("--graph-steps", type=int, default=1,
                    help="with --graph: also capture this many steps in one graph (shares the host's graph-launch cost)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-params", type=int, default=120_000_000)
    ap.add_argument("--reference-sample-params", type=int, default=0,
                    help="--impl reference: parameters timed per step (0 = the whole set when host memory and step time allow)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.buffer_elems > 0:
        return run_buffer_kernels(args)
    if args.secondary:
        return run_secondary(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        import bench_zero1
        return bench_zero1.run(args)
    return run_single(args)


if __name__ == "__main__":
    sys.exit(main())
