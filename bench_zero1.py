"""bench.py's N > 1 arm: the sharded AdamW + clip + bf16-shadow step on N GPUs of one node.

Before the warm-up every run checks the step it is about to time: one real step of the full-size
optimizer on the seeded per-rank gradients, compared on a fixed set of windows (both ends of every
rank's shard, i.e. both sides of every shard boundary) with the CPU oracle — see `parity_check`.
The JSON line carries the verdict and the process exits non-zero when it fails."""
from __future__ import annotations

import json
import os
import statistics
import time

# Peer-copy bandwidth per direction per GPU measured on this pool with one copy-engine copy at a time.
# It is a constant typed in here, not measured in the run: the line labels it so, and reports the
# fraction of the nominal 900 GB/s beside it.
NVLINK_PEER_GBS = 770.0
NVLINK_NOMINAL_GBS = 900.0


def run(args) -> int:
    import torch
    import torch.distributed as dist

    from gograd_b200 import paramsets
    from gograd_b200.zero1 import Zero1AdamW
    import bench as B  # the root script: constants, clock sampler, peak lookup, CPU baseline

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    # stdout carries exactly one JSON line: whatever libraries print on file descriptor 1 while the
    # ranks run (NCCL's version banner, for one) is sent to stderr until the line is written.
    import sys
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    key = args.workload if args.workload != "auto" else "llama8b"
    ps = paramsets.get(key)
    hp = ps.hparams
    group_of = [(ps.group_of(s.group).lr_scale, ps.group_of(s.group).weight_decay) for s in ps.params]
    comm = getattr(args, "comm", "peer") or "peer"
    opt = Zero1AdamW([s.numel for s in ps.params], group_of, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                     ps.max_norm, local, comm=comm, chunk_elems=args.chunk, multicast=args.multicast,
                     push_order=args.push_order, exchange_timeout_ms=30000,
                     ce_pull_sources=getattr(args, "ce_pull_sources", None) if comm == "abi" else None,
                     ce_push_targets=getattr(args, "ce_push_targets", None) if comm == "abi" else None,
                     staging_writers=not getattr(args, "staging_readers", False))
    ce_pull, ce_push = opt.ctx.copy_engine_use() if opt.ctx is not None else (0, 0)
    staged_by = "owners" if (opt.ctx is not None and opt.ctx.staging_written_by_owners()) else "reader"
    tuning = apply_tuning(opt, args)
    n_params = ps.numel
    gen = torch.Generator(device=f"cuda:{local}").manual_seed(ps.grad_seed * 1000 + rank)
    opt.grad_flat.normal_(0.0, ps.grad_std, generator=gen)   # per-rank gradients, seeded by rank
    opt.zero_padding()
    opt.master.normal_(0.0, 0.02, generator=gen)
    stream = torch.cuda.current_stream()

    link = measure_link_peaks(opt, torch, dist) if comm != "nccl" else None
    parity = None if args.no_parity_check else parity_check(opt, torch, dist)
    if args.sweep:
        records = launch_shape_sweep(opt, torch, dist)
        if rank == 0:
            sys.stdout.flush()
            os.dup2(real_stdout, 1)
            print(json.dumps({"launch_shape_sweep": records, "link_peaks": link, "n_gpus": world, "workload": key, "comm": comm,
                              "multicast_shadow_stores": bool(args.multicast), "parity_check": parity}), flush=True)
            os.dup2(2, 1)
        opt.close()
        dist.destroy_process_group()
        return 0 if (parity is None or parity["ok"]) else 3

    for _ in range(args.warmup):
        opt.step()
    torch.cuda.synchronize()
    opt.exchange_status()   # abi path: raises if a rank missed an exchange
    dist.barrier()

    sampler = B.ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    from gograd_b200.engine import launch_count, launch_count_reset
    launch_count_reset()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(args.steps):
        opt.step()
    stop.record(stream)
    torch.cuda.synchronize()
    opt.exchange_status()
    dist.barrier()
    launches = launch_count()
    elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed.item()) / args.steps
    norm_value = opt.grad_norm()

    # ---- per-phase timing (separate short loop, events around each phase, max over ranks) ----
    phases = phase_times(opt, torch, dist, 3)

    # ---- end to end: gradients come from page-locked host memory every step -------------------
    e2e = None
    if not args.no_e2e:
        try:
            numa = B.bind_to_gpu_numa_node(local)   # before the page-locked allocation: first touch decides the node
            stage_elems = 1 << 28  # 1 GiB staging buffer, reused for every range of the gradient buffer
            stage = torch.empty(stage_elems, dtype=torch.float32).pin_memory()
            stage.normal_(0.0, ps.grad_std)
            used = opt.layout.used
            e2e_steps = 2

            def host_step():
                pos = 0
                while pos < used:
                    n = min(stage_elems, used - pos)
                    opt.grad_flat[pos:pos + n].copy_(stage[:n], non_blocking=True)
                    pos += n
                opt.step()
                return opt.grad_norm()   # device -> host read of the step's result, synchronises

            host_step()
            dist.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                host_step()
            torch.cuda.synchronize()
            dt = torch.tensor([(time.perf_counter() - t0) / e2e_steps], dtype=torch.float64, device=f"cuda:{local}")
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            e2e = {"value": n_params / float(dt.item()) / 1e9, "unit": B.UNIT, "h2d_bytes_per_step": 4 * used * world,
                   "d2h_bytes_per_step": 32 * world, "ms_per_step": float(dt.item()) * 1e3, "steps": e2e_steps,
                   "api": "Zero1AdamW.step after copying every rank's full fp32 gradient buffer from page-locked host "
                          "memory (1 GiB staging buffer reused per range), norm read back",
                   "numa_binding_rank0": numa}
            del stage
        except Exception as exc:
            e2e = {"value": None, "unit": B.UNIT, "error": str(exc)[:200]}
    clocks = sampler.stop() if rank == 0 else None

    cpu_baseline = None
    if rank == 0 and not args.no_cpu_baseline:
        # the reference's CPU path on this host's cores, on a bounded sample of the same parameter set
        cpu_baseline, _, _ = B.cpu_reference_run(ps, args.cpu_sample_params, 3, 1, os.cpu_count() or 1)
    dist.barrier()

    if rank == 0:
        peak, peak_kind = B.measured_peak()
        shard = opt.layout.shard_len
        pull_remote = 4.0 * shard * (world - 1)          # bytes this rank pulls over NVLink in the reduce kernel
        push_remote = 2.0 * shard * (world - 1)          # bytes it stores into peers' shadows in the update kernel
        k1, k2 = phases.get("reduce_ms"), phases.get("update_ms")
        # the link rates this box gave the two access patterns a moment ago, with nothing else riding on them
        read_peak = link["reads_GBs"] if link else None
        store_peak = link["stores_GBs"] if link else None
        copy_peak = max(link["ring_copy_GBs"], link.get("ring_copy_write_GBs", 0.0)) if link else None
        # With copies carrying part of a phase, the phase is rated against the better of the two rates the
        # fabric gave a moment ago: SM-issued accesses to every peer at once, or one copy between neighbours.
        reduce_peak = max(read_peak, copy_peak) if (read_peak and ce_pull) else read_peak
        push_peak = max(store_peak, copy_peak) if (store_peak and ce_push) else store_peak
        nvlink_ms = (pull_remote + push_remote) / (NVLINK_PEER_GBS * 1e9) * 1e3
        hbm_ms = ((4.0 * world + 4.0) + 30.0) * shard / (peak * 1e9) * 1e3
        # The update cannot start before the global norm is known, i.e. before every rank's reduction is
        # over, so the two phases cannot overlap: the reduction at link rate (or its own HBM traffic, if
        # that takes longer) followed by the update at HBM rate (or its remote stores at link rate).
        reduce_floor = max(pull_remote / (NVLINK_PEER_GBS * 1e9), (4.0 * world + 4.0) * shard / (peak * 1e9)) * 1e3
        update_floor = max(30.0 * shard / (peak * 1e9), push_remote / (NVLINK_PEER_GBS * 1e9)) * 1e3
        roofline = {
            "bound": "nvlink",
            "kernel": ("ncclReduceScatter" if comm == "nccl" else
                       "%d staged peer copies + oe_peer_reduce_sumsq (pull reduce-scatter + norm)" % ce_pull if ce_pull else
                       "oe_peer_reduce_sumsq (pull reduce-scatter + norm)"),
            "achieved": pull_remote / (k1 * 1e-3) / 1e9 if k1 else None, "peak": reduce_peak or NVLINK_PEER_GBS, "unit": "GB/s",
            "frac": (pull_remote / (k1 * 1e-3) / 1e9 / (reduce_peak or NVLINK_PEER_GBS)) if k1 else None,
            "peak_kind": ("measured in this run: the better of every rank reading its shard of every peer's gradient buffer at "
                          "the same time (oe_link_probe_reads) and every rank copying from, or to, its neighbour at the same time") if (reduce_peak and ce_pull) else
                         ("measured in this run: every rank reading its shard of every peer's gradient buffer at the same time, "
                          "nothing stored (oe_link_probe_reads)") if read_peak else
                         "builder constant: 770 GB/s, a one-at-a-time copy-engine peer copy measured on this pool "
                         "(not measured in this run)",
            "frac_of_770_builder_constant": (pull_remote / (k1 * 1e-3) / 1e9 / NVLINK_PEER_GBS) if k1 else None,
            "link_peaks": link,
            "frac_of_nominal_900GBs": (pull_remote / (k1 * 1e-3) / 1e9 / NVLINK_NOMINAL_GBS) if k1 else None,
            "traffic": None,
            "traffic_source": "none: the bytes that cross NVLink are not DRAM traffic of this GPU; ncu is not run on "
                              "multi-rank commands",
            "algorithmic_bytes_per_launch": pull_remote, "kernel_ms": k1,
            "update_kernel": {"kernel": ("oe_adamw_fused + ncclAllGather" if comm == "nccl" else
                                         "oe_adamw_fused_peers + %d shadow copies" % ce_push if ce_push else "oe_adamw_fused_peers"),
                              "kernel_ms": k2, "remote_store_bytes": push_remote,
                              "nvlink_achieved": push_remote / (k2 * 1e-3) / 1e9 if k2 else None,
                              "nvlink_peak_measured": push_peak,
                              "nvlink_frac_of_measured": push_remote / (k2 * 1e-3) / 1e9 / push_peak if (k2 and push_peak) else None,
                              "nvlink_frac_of_770_builder_constant": push_remote / (k2 * 1e-3) / 1e9 / NVLINK_PEER_GBS if k2 else None,
                              "nvlink_frac_of_nominal_900GBs": push_remote / (k2 * 1e-3) / 1e9 / NVLINK_NOMINAL_GBS if k2 else None,
                              "hbm_bytes": 30.0 * shard,
                              "hbm_achieved": 30.0 * shard / (k2 * 1e-3) / 1e9 if k2 else None, "hbm_peak": peak},
            "step_floor_ms": {"nvlink": nvlink_ms, "hbm": hbm_ms, "reduce_then_update": reduce_floor + update_floor,
                              "reduce_then_update_at_measured_link_rates":
                                  (max(pull_remote / (reduce_peak * 1e9), (4.0 * world + 4.0) * shard / (peak * 1e9)) +
                                   max(30.0 * shard / (peak * 1e9), push_remote / (push_peak * 1e9))) * 1e3
                                  if (reduce_peak and push_peak) else None},
            "step_frac_of_floor": max(nvlink_ms, hbm_ms) / ms_per_step,
            "step_frac_of_serial_floor": (reduce_floor + update_floor) / ms_per_step,
            "phases_ms": phases,
        }
        line = {
            "metric": B.METRIC, "value": n_params / (ms_per_step * 1e-3) / 1e9, "unit": B.UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": key, "title": ps.title, "params": n_params, "tensors": len(ps.params),
                       "optimizer": "adamw", "max_norm": ps.max_norm, "bf16_shadow": True, "sharding": f"zero1 x{world}",
                       "comm": comm, "multicast_shadow_stores": bool(args.multicast), "push_order": args.push_order,
                       "tuning": tuning, "copy_engine": {"staged_pull_sources": ce_pull, "shadow_copy_targets": ce_push, "staged_by": staged_by},
                       "shard_elems": shard, "grad_reduce": "mean, ascending rank order",
                       "l2": "inputs larger than L2: %.1f GB per rank" % ((6.0 * opt.layout.total + 12.0 * shard) / 1e9),
                       "grad_norm": norm_value},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks, "gpu_launches": launches,
            "parity_check": parity,
        }
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    opt.close()
    dist.destroy_process_group()
    return 0 if (parity is None or parity["ok"]) else 3


def apply_tuning(opt, args):
    """Launch-shape knobs of the peer kernels from the command line (none changes a result)."""
    from gograd_b200 import engine as E
    chosen = {}
    if opt.comm == "nccl":
        return chosen
    if args.reduce_grid:
        opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_GRID, args.reduce_grid)
        chosen["reduce_grid"] = args.reduce_grid
    if args.update_grid:
        opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_GRID, args.update_grid)
        chosen["update_grid"] = args.update_grid
    if args.reduce_first == "rotated":
        opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_FIRST, (opt.rank + 1) % opt.world)
        chosen["reduce_first"] = "rank+1"
    if args.push_warp_rotate:
        opt.plan.set_tuning(E.OE_TUNE_PEER_PUSH_WARP_ROTATE, {"on": 1, "off": 2}[args.push_warp_rotate])
        chosen["push_warp_rotate"] = args.push_warp_rotate
    return chosen


def measure_link_peaks(opt, torch, dist, iters: int = 3):
    """What the NVLink fabric of this box gives the step's two access patterns when nothing else rides on them,
    all ranks at once (a barrier before each launch, max over ranks): every load of the pull-reduce with no store,
    and bf16 stores to every peer's shadow in the update's launch shape with no update around them. The store
    probe writes zeros over ranges the next step rewrites, so it runs before anything is checked or timed."""
    world = opt.world
    if world < 2:
        return None
    dev = opt.master.device
    stream = torch.cuda.current_stream()
    shard = opt.layout.shard_len

    def timed(fn):
        vals = []
        for _ in range(iters + 1):          # the first launch warms up
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            torch.cuda.synchronize()
            vals.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(vals[1:])], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    r = timed(lambda: opt.plan.link_probe_reads(opt.grad_bases, opt.lo, shard))
    w = timed(lambda: opt.plan.link_probe_stores(opt.shadow_flat.data_ptr() + 2 * opt.lo, opt.shadow_deltas, shard))
    # and what a copy gets when every rank copies from the rank after it at the same time (one reader and one
    # writer per GPU): this rank's shard range of the next rank's gradient buffer into a scratch tensor
    scratch = torch.empty(shard, dtype=torch.float32, device=dev)
    source = opt.grad_bases[(opt.rank + 1) % world] + 4 * opt.lo
    c = timed(lambda: engine_copy(opt, scratch.data_ptr(), source, 4 * shard))
    del scratch
    out = {"reads_GBs": 4.0 * shard * (world - 1) / r / 1e6, "reads_ms": r,
           "stores_GBs": 2.0 * shard * (world - 1) / w / 1e6, "stores_ms": w,
           "ring_copy_GBs": 4.0 * shard / c / 1e6, "ring_copy_ms": c,
           "how": "oe_link_probe_reads / oe_link_probe_stores / one oe_memcpy_d2d from the next rank (and, where the ranks' "
                  "staging is shared, one into the next rank's staging), on every rank at once, median of %d, max over ranks" % iters}
    if opt.staging_bases:
        # the same copy the other way: this rank's gradient range for the next rank, written into that rank's staging
        nxt = (opt.rank + 1) % world
        cw = timed(lambda: engine_copy(opt, opt.staging_bases[nxt], opt.grad_flat.data_ptr() + 4 * shard * nxt, 4 * shard))
        out["ring_copy_write_GBs"], out["ring_copy_write_ms"] = 4.0 * shard / cw / 1e6, cw
    return out


def engine_copy(opt, dst: int, src: int, nbytes: int) -> None:
    from gograd_b200 import engine as E
    E.check(E.lib().oe_memcpy_d2d(opt.device, dst, src, nbytes, E._stream(None)))


def launch_shape_sweep(opt, torch, dist, iters: int = 3):
    """Times the two peer kernels of the step over every launch-shape knob the library exposes
    (grid sizes, first-issued source rank, store order), one kernel at a time with a barrier before
    each launch, max over ranks. A diagnostic for a new machine; no knob changes a result."""
    from gograd_b200 import engine as E
    from gograd_b200.engine import OE_PARTIAL_ONLY, OE_WRITE_SHADOW
    world, rank = opt.world, opt.rank
    dev = opt.master.device
    stream = torch.cuda.current_stream()
    shard = opt.layout.shard_len
    pull_bytes, push_bytes = 4.0 * shard * (world - 1), 2.0 * shard * (world - 1)
    own = opt.grad_flat[opt.lo:opt.hi]
    records = []

    def timed(fn):
        vals = []
        for _ in range(iters):
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            torch.cuda.synchronize()
            vals.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(vals)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def pull():
        opt.plan.peer_reduce_grads(opt.grad_bases, opt.lo, shard, own.data_ptr(), 1.0 / world, OE_PARTIAL_ONLY)

    for grid in (0, 148, 74):
        for first in ("rank0", "rank+1", "rank+1+warp"):
            opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_GRID, grid)
            opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_FIRST, (rank + 1) % world if first != "rank0" else 0)
            opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_WARP_ROTATE, 1 if first == "rank+1+warp" else 0)
            ms = timed(pull)
            records.append({"kernel": "oe_peer_reduce_sumsq", "grid": grid or "default", "first_source": first, "ms": ms,
                            "pulled_GBs": pull_bytes / ms / 1e6})
    opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_GRID, 0)
    opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_FIRST, 0)
    opt.plan.set_tuning(E.OE_TUNE_PEER_REDUCE_WARP_ROTATE, 0)
    # a norm for the updates that follow
    if opt.comm == "abi":
        opt.ctx.exchange(0)
        pull()
        opt.ctx.exchange(1)
    else:
        pull()
        dist.all_reduce(opt.sumsq)
        opt.plan.norm_finalize()
    opt.step_count += 1
    hp = opt._hparams(OE_WRITE_SHADOW)
    keep_order = opt.push_order
    if opt.multicast:
        for grid in (0, 148, 74):
            opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_GRID, grid)
            ms = timed(lambda: opt.plan.adamw_step_multicast(hp, opt.shadow_deltas, opt.mc_delta))
            records.append({"kernel": "oe_adamw_fused_peers (multimem.st)", "grid": grid or "default", "ms": ms,
                            "received_GBs": push_bytes / ms / 1e6})
    else:
        # grid 0 and warp rotation 0 are "the library's choice"; the sweep pins both (296 = the persistent grid)
        shapes = [(4, g, "ascending", w) for g in (296, 222, 148, 111, 74, 37) for w in (2, 1)] + \
                 [(4, g, "rotated", w) for g in (296, 148) for w in (2, 1)] + \
                 [(2, g, "ascending", w) for g in (444, 296, 148) for w in (2, 1)]
        for vectors, grid, order, warp_rotate in shapes:
            opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_VECTORS, vectors)
            opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_GRID, grid)
            opt.plan.set_tuning(E.OE_TUNE_PEER_PUSH_WARP_ROTATE, warp_rotate)
            opt.push_order = order
            ms = timed(lambda: opt.plan.adamw_step_peers(hp, opt._push_deltas()))
            records.append({"kernel": "oe_adamw_fused_peers", "vectors_in_flight": vectors, "grid": grid,
                            "store_order": order, "warp_rotate": warp_rotate == 1, "ms": ms,
                            "pushed_GBs": push_bytes / ms / 1e6})
        opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_VECTORS, 0)
        opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_GRID, 0)
        opt.plan.set_tuning(E.OE_TUNE_PEER_PUSH_WARP_ROTATE, 0)
        ms = timed(lambda: opt.plan.adamw_step_peers(hp, opt._push_deltas()))
        records.append({"kernel": "oe_adamw_fused_peers", "shape": "the library's choice for %d ranks" % world, "ms": ms,
                        "pushed_GBs": push_bytes / ms / 1e6})
    opt.plan.set_tuning(E.OE_TUNE_PEER_UPDATE_GRID, 0)
    opt.plan.set_tuning(E.OE_TUNE_PEER_PUSH_WARP_ROTATE, 0)
    opt.push_order = keep_order
    if opt.comm == "abi":
        opt.ctx.exchange(2)
        records.append({"kernel": "oe_rank_exchange", "ms": timed(lambda: opt.ctx.exchange(0))})
        opt.ctx.exchange(1)
        opt.ctx.exchange(2)
        opt.exchange_status()
    return records


def parity_check(opt, torch, dist, window: int = 65536):
    """One real step of the optimizer that is about to be timed, checked against the CPU oracle.

    Windows: the first and the last `window` elements of every rank's shard, so both sides of every
    shard boundary are covered and every rank owns some of them. Compared, on every window:
      (a) the reduced gradient the owner holds after the step with the mean of the N ranks' gradients
          added on the host in ascending rank order in float32 (bit for bit, except on the NCCL path,
          whose order is NCCL's: 1e-6 of the window's largest magnitude there);
      (b) the owner's p, m, v with the oracle's AdamW fed that mean and the clip coefficient of the
          step's own norm (bit for bit / 1e-6 relative on the NCCL path);
      (c) every rank's bf16 shadow with round-to-nearest-even of the owner's master (bit for bit);
      (d) the global norm with an independent float64 reduction of the reduced gradient (1e-6 relative).
    Returns the verdict (identical on every rank); the caller exits non-zero when ok is false."""
    import numpy as np

    from oracle import oracle
    L, world, rank = opt.layout, opt.world, opt.rank
    exact = opt.comm != "nccl"
    windows = []
    for r in range(world):
        lo, hi = L.shard_range(r)
        w = min(window, hi - lo)
        for a, b in ((lo, lo + w), (hi - w, hi)):
            if (a, b) not in windows:
                windows.append((a, b))
    mine = [(a, b) for a, b in windows if L.owner_of(a) == rank]

    torch.cuda.synchronize()
    pre = {"g": {w: opt.grad_flat[w[0]:w[1]].cpu().numpy() for w in windows},
           "p": {w: opt.master[w[0] - opt.lo:w[1] - opt.lo].cpu().numpy() for w in mine},
           "m": {w: opt.m[w[0] - opt.lo:w[1] - opt.lo].cpu().numpy() for w in mine},
           "v": {w: opt.v[w[0] - opt.lo:w[1] - opt.lo].cpu().numpy() for w in mine}}
    everyone = [None] * world
    dist.all_gather_object(everyone, pre["g"])

    opt.step()
    torch.cuda.synchronize()
    opt.exchange_status()
    norm = float(opt.grad_norm())

    problems, max_ulp, checked = [], 0, 0

    def ulps(got, want):
        from_bits = lambda x: np.where(x < 0, -(x & 0x7FFFFFFF), x)
        a = from_bits(np.ascontiguousarray(got, np.float32).view(np.int32).astype(np.int64))
        b = from_bits(np.ascontiguousarray(want, np.float32).view(np.int32).astype(np.int64))
        return int(np.max(np.abs(a - b))) if a.size else 0

    def compare(what, got, want, w):
        nonlocal max_ulp
        if exact:
            d = ulps(got, want)
            max_ulp = max(max_ulp, d)
            if d != 0:
                problems.append(f"{what} of window {w}: {d} ulp from the oracle")
        else:
            scale = float(np.max(np.abs(want))) or 1.0
            err = float(np.max(np.abs(got.astype(np.float64) - want) / (np.abs(want) + scale)))
            if err > 2e-6:
                problems.append(f"{what} of window {w}: relative error {err:.3g}")

    # (d) the norm against an independent float64 reduction of what the owners now hold
    total = torch.zeros(1, dtype=torch.float64, device=opt.master.device)
    own = opt.grad_flat[opt.lo:opt.hi]
    for a in range(0, own.numel(), 1 << 26):
        total += own[a:a + (1 << 26)].double().pow(2).sum()
    dist.all_reduce(total)
    want_norm = float(np.float32(np.sqrt(float(total.item()))))
    norm_err = abs(norm - want_norm) / want_norm
    if not norm_err <= 1e-6:
        problems.append(f"global norm {norm} against the float64 reduction {want_norm}: {norm_err:.3g}")

    coef = oracle.clip_coefficient(norm, opt.max_norm)
    bc1, bc2 = opt.bias_corrections()
    post_master = {}
    for w in mine:
        a, b = w
        # (a) fixed-order mean on the host
        acc = everyone[0][w].copy()
        for r in range(1, world):
            acc = (acc + everyone[r][w]).astype(np.float32)
        mean = (acc * np.float32(1.0 / world)).astype(np.float32)
        compare("reduced gradient", opt.grad_flat[a:b].cpu().numpy(), mean, w)
        got = {k: t[a - opt.lo:b - opt.lo].cpu().numpy() for k, t in (("p", opt.master), ("m", opt.m), ("v", opt.v))}
        post_master[w] = got["p"]
        # (b) the oracle's update, tensor piece by tensor piece (groups differ per tensor); padding is skipped
        for pc in opt.my_pieces:
            x, y = max(a, pc.flat_offset), min(b, pc.flat_offset + pc.length)
            if x >= y:
                continue
            sl = slice(x - a, y - a)
            # the NCCL path's reduction order is NCCL's own: its update is checked on the gradient it produced
            g = mean[sl].copy() if exact else opt.grad_flat[x:y].cpu().numpy().copy()
            oracle.scale_(g, float(coef))
            scale, decay = opt.group_of[pc.tensor]
            step, dec = oracle.C.c_float(), oracle.C.c_float()
            oracle.lib().oracle_adamw_group_scale(opt.lr, scale, decay, step, dec)
            p, m, v = (np.ascontiguousarray(pre[k][w][sl]).copy() for k in ("p", "m", "v"))
            oracle.lib().oracle_adamw_update(oracle._ptr(p), oracle._ptr(g), oracle._ptr(m), oracle._ptr(v), p.size,
                                             opt.beta1, opt.beta2, opt.eps, step.value, dec.value, bc1, bc2)
            for k, want in (("p", p), ("m", m), ("v", v)):
                compare(k, got[k][sl], want, (x, y))
            checked += y - x
    # (c) every rank's shadow against RNE of the owner's master
    masters = [None] * world
    dist.all_gather_object(masters, post_master)
    for owner_windows in masters:
        for (a, b), master in owner_windows.items():
            shadow = opt.shadow_flat[a:b].view(torch.int16).cpu().numpy().view(np.uint16)
            want = oracle.f32_to_bf16(master)
            keep = np.zeros(b - a, bool)
            for r in range(world):
                for pc in L.pieces(r):
                    x, y = max(a, pc.flat_offset), min(b, pc.flat_offset + pc.length)
                    if x < y:
                        keep[x - a:y - a] = True
            if not np.array_equal(shadow[keep], want[keep]):
                problems.append(f"bf16 shadow of window {(a, b)} on rank {rank} differs from RNE of the owner's master")
    verdicts = [None] * world
    dist.all_gather_object(verdicts, (problems, max_ulp, checked))
    all_problems = [f"rank {r}: {p}" for r, (ps_, _, _) in enumerate(verdicts) for p in ps_]
    return {"ok": not all_problems, "windows": len(windows), "window_elems": window,
            "elements_checked": int(sum(v[2] for v in verdicts)), "max_ulp": int(max(v[1] for v in verdicts)),
            "bit_exact_required": exact, "norm": norm, "norm_rel_err_vs_float64": norm_err,
            "checks": ["reduced gradient = ascending-rank-order fp32 mean", "p/m/v = oracle AdamW with the step's clip coefficient",
                       "every rank's bf16 shadow = RNE(owner's master)", "global norm vs float64 reduction <= 1e-6"],
            "problems": all_problems[:8]}


def phase_times(opt, torch, dist, iters: int):
    """Times the phases of the peer path one by one (a barrier before each, max over ranks)."""
    from gograd_b200.engine import OE_PARTIAL_ONLY, OE_WRITE_SHADOW
    dev = opt.master.device
    stream = torch.cuda.current_stream()
    out = {}

    def timed(fn):
        vals = []
        for _ in range(iters):
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            torch.cuda.synchronize()
            vals.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(vals)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    own = opt.grad_flat[opt.lo:opt.hi]
    if opt.comm == "abi":
        out["reduce_ms"] = timed(opt.ctx.reduce)          # staged copies (if the context uses them) + pull kernel
    elif opt.comm != "nccl":
        out["reduce_ms"] = timed(lambda: opt.plan.peer_reduce_grads(opt.grad_bases, opt.lo, opt.layout.shard_len,
                                                                    own.data_ptr(), 1.0 / opt.world, OE_PARTIAL_ONLY))
    else:
        out["reduce_ms"] = timed(lambda: dist.reduce_scatter_tensor(own, opt.grad_flat, op=dist.ReduceOp.AVG))
        out["norm_ms"] = timed(lambda: opt.plan.grad_norm(OE_PARTIAL_ONLY))
    if opt.comm == "abi":
        out["exchange_ms"] = timed(lambda: opt.ctx.exchange(0))   # one of the three bounded exchanges of a step
        opt.ctx.exchange(1)                                        # totals the partial sums into the norm
    else:
        out["allreduce_8B_ms"] = timed(lambda: dist.all_reduce(opt.sumsq))
        opt.plan.norm_finalize()
    opt.step_count += 1
    hp = opt._hparams(OE_WRITE_SHADOW)
    if opt.comm == "nccl":
        out["update_ms"] = timed(lambda: opt.plan.adamw_step(hp))
        out["allgather_ms"] = timed(lambda: dist.all_gather_into_tensor(opt.shadow_flat, opt.shadow_flat[opt.lo:opt.hi]))
    elif opt.comm == "abi":
        out["update_ms"] = timed(lambda: opt.ctx.adamw_update(hp))   # fused update + shadow stores, then shadow copies
    elif opt.multicast:
        out["update_ms"] = timed(lambda: opt.plan.adamw_step_multicast(hp, opt.shadow_deltas, opt.mc_delta))
    else:
        out["update_ms"] = timed(lambda: opt.plan.adamw_step_peers(hp, opt._push_deltas()))
    if opt.comm == "abi":
        opt.ctx.exchange(2)
        opt.exchange_status()
    return out
