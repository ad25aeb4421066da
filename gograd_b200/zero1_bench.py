"""bench.py's N > 1 arm: the sharded AdamW + clip + bf16-shadow step on N GPUs of one node."""
from __future__ import annotations

import json
import os
import statistics
import time

NVLINK_PEER_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool


def run(args) -> int:
    import torch
    import torch.distributed as dist

    from . import paramsets
    from .zero1 import Zero1AdamW
    import bench as B  # the root script: constants, clock sampler, peak lookup

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
                     ps.max_norm, local, comm=comm, chunk_elems=args.chunk)
    n_params = ps.numel
    gen = torch.Generator(device=f"cuda:{local}").manual_seed(ps.grad_seed * 1000 + rank)
    opt.grad_flat.normal_(0.0, ps.grad_std, generator=gen)   # per-rank gradients, seeded by rank
    opt.zero_padding()
    opt.master.normal_(0.0, 0.02, generator=gen)
    stream = torch.cuda.current_stream()

    for _ in range(args.warmup):
        opt.step()
    torch.cuda.synchronize()
    dist.barrier()

    sampler = B.ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    from .engine import launch_count, launch_count_reset
    launch_count_reset()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(args.steps):
        opt.step()
    stop.record(stream)
    torch.cuda.synchronize()
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
                          "memory (1 GiB staging buffer reused per range), norm read back"}
            del stage
        except Exception as exc:
            e2e = {"value": None, "unit": B.UNIT, "error": str(exc)[:200]}
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peak, peak_kind = B.measured_peak()
        shard = opt.layout.shard_len
        pull_remote = 4.0 * shard * (world - 1)          # bytes this rank pulls over NVLink in the reduce kernel
        push_remote = 2.0 * shard * (world - 1)          # bytes it stores into peers' shadows in the update kernel
        k1, k2 = phases.get("reduce_ms"), phases.get("update_ms")
        nvlink_ms = (pull_remote + push_remote) / (NVLINK_PEER_GBS * 1e9) * 1e3
        hbm_ms = ((4.0 * world + 4.0) + 30.0) * shard / (peak * 1e9) * 1e3
        # The update cannot start before the global norm is known, i.e. before every rank's reduction is
        # over, so the two phases cannot overlap: the reduction at link rate (or its own HBM traffic, if
        # that takes longer) followed by the update at HBM rate (or its remote stores at link rate).
        reduce_floor = max(pull_remote / (NVLINK_PEER_GBS * 1e9), (4.0 * world + 4.0) * shard / (peak * 1e9)) * 1e3
        update_floor = max(30.0 * shard / (peak * 1e9), push_remote / (NVLINK_PEER_GBS * 1e9)) * 1e3
        roofline = {
            "bound": "nvlink", "kernel": "oe_peer_reduce_sumsq (pull reduce-scatter + norm)" if comm == "peer" else "ncclReduceScatter",
            "achieved": pull_remote / (k1 * 1e-3) / 1e9 if k1 else None, "peak": NVLINK_PEER_GBS, "unit": "GB/s",
            "frac": (pull_remote / (k1 * 1e-3) / 1e9 / NVLINK_PEER_GBS) if k1 else None,
            "peak_kind": "measured peer-copy bandwidth per direction per GPU (nominal 900)",
            "traffic": None, "algorithmic_bytes_per_launch": pull_remote, "kernel_ms": k1,
            "update_kernel": {"kernel": "oe_adamw_fused_peers" if comm == "peer" else "oe_adamw_fused + ncclAllGather",
                              "kernel_ms": k2, "remote_store_bytes": push_remote,
                              "nvlink_achieved": push_remote / (k2 * 1e-3) / 1e9 if k2 else None,
                              "hbm_bytes": 30.0 * shard,
                              "hbm_achieved": 30.0 * shard / (k2 * 1e-3) / 1e9 if k2 else None, "hbm_peak": peak},
            "step_floor_ms": {"nvlink": nvlink_ms, "hbm": hbm_ms, "reduce_then_update": reduce_floor + update_floor},
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
                       "comm": comm, "shard_elems": shard, "grad_reduce": "mean, ascending rank order",
                       "l2": "inputs larger than L2: %.1f GB per rank" % ((6.0 * opt.layout.total + 12.0 * shard) / 1e9),
                       "grad_norm": norm_value},
            "roofline": roofline, "cpu_baseline": None, "e2e": e2e, "clocks": clocks, "gpu_launches": launches,
        }
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    opt.close()
    dist.destroy_process_group()
    return 0


def phase_times(opt, torch, dist, iters: int):
    """Times the phases of the peer path one by one (a barrier before each, max over ranks)."""
    from .engine import OE_PARTIAL_ONLY, OE_WRITE_SHADOW
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
    if opt.comm == "peer":
        out["reduce_ms"] = timed(lambda: opt.plan.peer_reduce_grads(opt.grad_bases, opt.lo, opt.layout.shard_len,
                                                                    own.data_ptr(), 1.0 / opt.world, OE_PARTIAL_ONLY))
    else:
        out["reduce_ms"] = timed(lambda: dist.reduce_scatter_tensor(own, opt.grad_flat, op=dist.ReduceOp.AVG))
        out["norm_ms"] = timed(lambda: opt.plan.grad_norm(OE_PARTIAL_ONLY))
    out["allreduce_8B_ms"] = timed(lambda: dist.all_reduce(opt.sumsq))
    opt.plan.norm_finalize()
    opt.step_count += 1
    hp = opt._hparams(OE_WRITE_SHADOW)
    if opt.comm == "peer":
        out["update_ms"] = timed(lambda: opt.plan.adamw_step_peers(hp, opt.shadow_deltas))
    else:
        out["update_ms"] = timed(lambda: opt.plan.adamw_step(hp))
        out["allgather_ms"] = timed(lambda: dist.all_gather_into_tensor(opt.shadow_flat, opt.shadow_flat[opt.lo:opt.hi]))
    return out
