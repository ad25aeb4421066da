"""The sharded step's kernels on the GPU.

One GPU: the ranks are emulated as separate buffers on the same device (the peer kernels
never wait on one another, so running the ranks one after the other is exact). Two or more
GPUs: real ranks over NCCL with CUDA-IPC peer mappings, both data paths, against the oracle.
"""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

NUMELS = [5000, 3, 4097, 12, 70001, 8192]
GROUPS = [(1.0, 0.1), (1.0, 0.0), (0.5, 0.1), (1.0, 0.0), (1.0, 0.1), (2.0, 0.05)]
HP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, max_norm=0.01)


def _grads(rank, step):
    rng = np.random.default_rng(1000 * step + rank)
    return [rng.normal(0, 1e-3, n).astype(np.float32) for n in NUMELS]


def _weights():
    rng = np.random.default_rng(77)
    return [rng.normal(0, 0.02, n).astype(np.float32) for n in NUMELS]


def _oracle_run(world, steps):
    """Unsharded oracle on the fixed-order mean: (((g0+g1)+g2)+...) * float32(1/world)."""
    from oracle import oracle
    groups = [oracle.Group(f"g{i}", [i], s, d) for i, (s, d) in enumerate(GROUPS)]
    ref = oracle.OracleAdamW([w.copy() for w in _weights()], lr=HP["lr"], groups=groups, beta1=HP["beta1"],
                             beta2=HP["beta2"], eps=HP["eps"])
    norms = []
    for step in range(1, steps + 1):
        per_rank = [_grads(r, step) for r in range(world)]
        mean = []
        for i in range(len(NUMELS)):
            acc = per_rank[0][i].copy()
            for r in range(1, world):
                acc = (acc + per_rank[r][i]).astype(np.float32)
            mean.append((acc * np.float32(1.0 / world)).astype(np.float32))
        norm, _ = oracle.clip_grad_norm(mean, HP["max_norm"])
        norms.append(float(norm))
        ref.step(mean)
    return ref, norms


@pytest.mark.parametrize("world,tuned", [(2, False), (3, False), (8, False), (3, True), (8, True)])
def test_peer_kernels_with_emulated_ranks(world, tuned):
    """tuned: every launch-shape knob of the peer kernels away from its default (first-issued rank,
    small grids, warp-rotated and rank-rotated store order); no result may change."""
    import gograd_b200 as eng
    from gograd_b200.engine import OE_PARTIAL_ONLY, OE_WRITE_SHADOW
    from gograd_b200.workload import bias_corrections
    from gograd_b200.zero1 import ShardLayout, _RawCuda
    from oracle import oracle

    eng.init(0)
    L = ShardLayout(NUMELS, world)
    G = [torch.zeros(L.total, device="cuda") for _ in range(world)]
    S = [torch.full((L.total,), -1, dtype=torch.int16, device="cuda") for _ in range(world)]
    weights = np.zeros(L.total, np.float32)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = w
    P, M, V, plans, records = [], [], [], [], []
    for r in range(world):
        lo, hi = L.shard_range(r)
        P.append(torch.from_numpy(weights[lo:hi].copy()).cuda())
        M.append(torch.zeros(L.shard_len, device="cuda"))
        V.append(torch.zeros(L.shard_len, device="cuda"))
        descs = []
        for pc in L.pieces(r):
            a, b = pc.flat_offset, pc.flat_offset + pc.length
            descs.append(eng.TensorDesc(P[r][a - lo:b - lo], G[r][a:b], M[r][a - lo:b - lo], V[r][a - lo:b - lo],
                                        S[r][a:b], *GROUPS[pc.tensor]))
        plans.append(eng.Plan(descs))
        records.append(torch.as_tensor(_RawCuda(plans[r].norm_address(), (1,), "<f8"), device="cuda"))
        if tuned:
            from gograd_b200.engine import (OE_TUNE_PEER_PUSH_WARP_ROTATE, OE_TUNE_PEER_REDUCE_FIRST,
                                            OE_TUNE_PEER_REDUCE_GRID, OE_TUNE_PEER_UPDATE_GRID,
                                            OE_TUNE_PEER_UPDATE_VECTORS, OE_TUNE_PEER_REDUCE_WARP_ROTATE)
            plans[r].set_tuning(OE_TUNE_PEER_REDUCE_WARP_ROTATE, 1)
            plans[r].set_tuning(OE_TUNE_PEER_UPDATE_VECTORS, 2 if world == 8 else 8)   # the other two built shapes
            plans[r].set_tuning(OE_TUNE_PEER_REDUCE_FIRST, (r + 1) % world)
            plans[r].set_tuning(OE_TUNE_PEER_REDUCE_GRID, 3)
            plans[r].set_tuning(OE_TUNE_PEER_UPDATE_GRID, 5)
            plans[r].set_tuning(OE_TUNE_PEER_PUSH_WARP_ROTATE, 1)
    steps = 2
    ref, want_norms = _oracle_run(world, steps)
    for step in range(1, steps + 1):
        for r in range(world):
            G[r].zero_()
            for o, g in zip(L.offsets, _grads(r, step)):
                G[r][o:o + g.size] = torch.from_numpy(g).cuda()
        bases = [g.data_ptr() for g in G]
        for r in range(world):
            lo, hi = L.shard_range(r)
            plans[r].peer_reduce_grads(bases, lo, L.shard_len, G[r][lo:hi].data_ptr(), 1.0 / world, OE_PARTIAL_ONLY)
        total = sum(float(rec.item()) for rec in records)     # what the 8-byte all-reduce does
        for r in range(world):
            records[r].fill_(total)
            plans[r].norm_finalize()
            norm, _ = plans[r].read_norm()
            assert abs(norm - want_norms[step - 1]) <= 1e-6 * want_norms[step - 1]
            b1, b2 = bias_corrections(HP["beta1"], HP["beta2"], step)
            hp = eng.AdamWHParams(HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], b1, b2, HP["max_norm"], OE_WRITE_SHADOW)
            deltas = [S[k].data_ptr() - S[r].data_ptr() for k in range(world)]
            if tuned:   # stores issued starting after this rank, ending with it
                deltas = [deltas[(r + 1 + j) % world] for j in range(world)]
            plans[r].adamw_step_peers(hp, deltas)
    torch.cuda.synchronize()
    flat = {k: np.zeros(L.total, np.float32) for k in "pmv"}
    for r in range(world):
        lo, hi = L.shard_range(r)
        flat["p"][lo:hi], flat["m"][lo:hi], flat["v"][lo:hi] = P[r].cpu().numpy(), M[r].cpu().numpy(), V[r].cpu().numpy()
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat["p"][o:o + n], ref.params[i]), f"p[{i}] world {world}"
        assert np.array_equal(flat["m"][o:o + n], ref.m[i]) and np.array_equal(flat["v"][o:o + n], ref.v[i])
        want = oracle.f32_to_bf16(ref.params[i]).view(np.int16)
        for r in range(world):
            assert np.array_equal(S[r][o:o + n].cpu().numpy(), want), f"shadow[{i}] on rank {r}"
    # padding of every shadow buffer was never written
    for r in range(world):
        got = S[r].cpu().numpy()
        for a, b in L.padding_ranges():
            assert np.all(got[a:b] == -1)
    for p in plans:
        p.close()


def _comm_options(spec, world):
    """"peer", "nccl", "abi", optionally "+mc" (multicast shadow stores), "+rot" (rotated store order) and "+ce"
    (copies stage all peers' gradients but one, two with two ranks, and carry the shadow to the last ranks of
    the ring: the library would not choose that for shards this small, so it is asked for)."""
    parts = spec.split("+")
    options = dict(comm=parts[0], multicast="mc" in parts[1:], push_order="rotated" if "rot" in parts[1:] else "ascending")
    if "ce" in parts[1:] or "cew" in parts[1:]:   # "cew": the staged ranges are written by their owners
        options.update(ce_pull_sources=1 if world == 2 else world - 2, ce_push_targets=1 if world <= 4 else world - 4,
                       staging_writers="cew" in parts[1:])
    return options


def _rank_main(rank, world, port, comm, queue):
    import torch.distributed as dist
    from gograd_b200.zero1 import Zero1AdamW
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    opt = Zero1AdamW(NUMELS, GROUPS, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], rank,
                     exchange_timeout_ms=20000, **_comm_options(comm, world))
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())
    norms = []
    for step in (1, 2):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))
        opt.step()
        norms.append(opt.grad_norm())
    torch.cuda.synchronize()
    assert opt.exchange_status() == 0
    queue.put((rank, opt.lo, opt.master.cpu().numpy(), opt.m.cpu().numpy(), opt.v.cpu().numpy(),
               opt.shadow_flat.view(torch.int16).cpu().numpy(), norms))
    opt.close()
    dist.destroy_process_group()


def _run_real_ranks(world, comm):
    import torch.multiprocessing as mp
    from gograd_b200.zero1 import ShardLayout
    from oracle import oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, comm, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    ref, want_norms = _oracle_run(world, 2)
    L = ShardLayout(NUMELS, world)
    flat = {k: np.zeros(L.total, np.float32) for k in "pmv"}
    for rank, lo, master, m, v, shadow, norms in results:
        flat["p"][lo:lo + master.size], flat["m"][lo:lo + m.size], flat["v"][lo:lo + v.size] = master, m, v
        for a, b in zip(norms, want_norms):
            assert abs(a - b) <= 1e-6 * b
    return ref, L, flat, results, oracle


@pytest.mark.parametrize("comm", ["peer", "nccl", "abi", "peer+rot", "abi+mc", "abi+ce", "abi+cew"])
def test_two_real_ranks(comm):
    """Two ranks: every path is bit-identical to the oracle (a two-term sum has one order). "abi" runs
    the whole step through oe_zero1_adamw_step with the library's own exchanges between the ranks;
    "+mc" sends the shadow through the NVLink multicast mapping."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ref, L, flat, results, oracle = _run_real_ranks(2, comm)
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat["p"][o:o + n], ref.params[i]), f"p[{i}] ({comm})"
        assert np.array_equal(flat["m"][o:o + n], ref.m[i]) and np.array_equal(flat["v"][o:o + n], ref.v[i])
        want = oracle.f32_to_bf16(ref.params[i]).view(np.int16)
        for rank, lo, master, m, v, shadow, norms in results:
            assert np.array_equal(shadow[o:o + n], want), f"rank {rank} shadow[{i}] ({comm})"


@pytest.mark.parametrize("comm", ["peer", "nccl", "abi", "abi+mc", "abi+ce", "abi+cew"])
def test_all_real_ranks_of_the_box(comm):
    """Every GPU of the box as a rank (4 or 8): the peer path adds in ascending rank order and stays
    bit-identical to the oracle; NCCL's order is its own, so that path is held to the stated
    tolerances (1e-6 relative after the first steps) and its shadows to RNE of its own master."""
    world = torch.cuda.device_count()
    if world < 3:
        pytest.skip("needs more than two GPUs")
    world = 8 if world >= 8 else 4 if world >= 4 else world
    ref, L, flat, results, oracle = _run_real_ranks(world, comm)
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        if comm != "nccl":
            assert np.array_equal(flat["p"][o:o + n], ref.params[i]), f"p[{i}] world {world}"
            assert np.array_equal(flat["m"][o:o + n], ref.m[i]) and np.array_equal(flat["v"][o:o + n], ref.v[i])
        else:
            for key, want in (("p", ref.params[i]), ("m", ref.m[i]), ("v", ref.v[i])):
                got = flat[key][o:o + n].astype(np.float64)
                scale = float(np.max(np.abs(want))) or 1.0
                assert np.max(np.abs(got - want) / (np.abs(want) + scale)) <= 2e-6, f"{key}[{i}] world {world}"
        own = oracle.f32_to_bf16(flat["p"][o:o + n]).view(np.int16)
        for rank, lo, master, m, v, shadow, norms in results:
            assert np.array_equal(shadow[o:o + n], own), f"rank {rank} shadow[{i}] ({comm})"


SGD_HP = dict(lr=0.05, momentum=0.9, dampening=0.0, nesterov=True, maximize=False, max_norm=0.01)


def _oracle_sgd_run(world, steps):
    """Unsharded oracle SGD on the fixed-order mean, clipped in place first."""
    from oracle import oracle
    groups = [oracle.Group(f"g{i}", [i], s, d) for i, (s, d) in enumerate(GROUPS)]
    ref = oracle.OracleSGD([w.copy() for w in _weights()], lr=SGD_HP["lr"], momentum=SGD_HP["momentum"],
                           dampening=SGD_HP["dampening"], nesterov=SGD_HP["nesterov"], maximize=SGD_HP["maximize"],
                           groups=groups)
    for step in range(1, steps + 1):
        per_rank = [_grads(r, step) for r in range(world)]
        mean = []
        for i in range(len(NUMELS)):
            acc = per_rank[0][i].copy()
            for r in range(1, world):
                acc = (acc + per_rank[r][i]).astype(np.float32)
            mean.append((acc * np.float32(1.0 / world)).astype(np.float32))
        oracle.clip_grad_norm(mean, SGD_HP["max_norm"])
        ref.step(mean)
    return ref


def test_sgd_peer_kernel_with_emulated_ranks():
    """oe_sgd_step_peers on one GPU: two "ranks" as separate buffers, each updating its shard of the flat
    layout and storing bf16 into both shadow buffers; p, momentum buffers and shadows equal the
    unsharded oracle, every piece's init flag is set after the first step."""
    import gograd_b200 as eng
    from gograd_b200.engine import OE_NESTEROV, OE_PARTIAL_ONLY, OE_WRITE_SHADOW
    from gograd_b200.zero1 import ShardLayout, _RawCuda
    from oracle import oracle

    eng.init(0)
    world, steps = 2, 3
    L = ShardLayout(NUMELS, world)
    G = [torch.zeros(L.total, device="cuda") for _ in range(world)]
    S = [torch.full((L.total,), -1, dtype=torch.int16, device="cuda") for _ in range(world)]
    weights = np.zeros(L.total, np.float32)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = w
    P, B, F, plans, records = [], [], [], [], []
    for r in range(world):
        lo, hi = L.shard_range(r)
        pieces = L.pieces(r)
        P.append(torch.from_numpy(weights[lo:hi].copy()).cuda())
        B.append(torch.zeros(L.shard_len, device="cuda"))
        F.append(torch.zeros(len(pieces), device="cuda"))
        descs = []
        for k, pc in enumerate(pieces):
            a, b = pc.flat_offset, pc.flat_offset + pc.length
            descs.append(eng.TensorDesc(P[r][a - lo:b - lo], G[r][a:b], B[r][a - lo:b - lo], F[r][k:k + 1], S[r][a:b],
                                        *GROUPS[pc.tensor]))
        plans.append(eng.Plan(descs))
        records.append(torch.as_tensor(_RawCuda(plans[r].norm_address(), (1,), "<f8"), device="cuda"))
    ref = _oracle_sgd_run(world, steps)
    for step in range(1, steps + 1):
        for r in range(world):
            G[r].zero_()
            for o, g in zip(L.offsets, _grads(r, step)):
                G[r][o:o + g.size] = torch.from_numpy(g).cuda()
        bases = [g.data_ptr() for g in G]
        for r in range(world):
            lo, hi = L.shard_range(r)
            plans[r].peer_reduce_grads(bases, lo, L.shard_len, G[r][lo:hi].data_ptr(), 1.0 / world, OE_PARTIAL_ONLY)
        total = sum(float(rec.item()) for rec in records)
        for r in range(world):
            records[r].fill_(total)
            plans[r].norm_finalize()
            hp = eng.SGDHParams(SGD_HP["lr"], SGD_HP["momentum"], SGD_HP["dampening"], SGD_HP["max_norm"],
                                OE_WRITE_SHADOW | OE_NESTEROV)
            plans[r].sgd_step_peers(hp, [S[k].data_ptr() - S[r].data_ptr() for k in range(world)])
        if step == 1:
            assert all(bool((f == 1).all()) for f in F)
    torch.cuda.synchronize()
    flat_p, flat_b = np.zeros(L.total, np.float32), np.zeros(L.total, np.float32)
    for r in range(world):
        lo, hi = L.shard_range(r)
        flat_p[lo:hi], flat_b[lo:hi] = P[r].cpu().numpy(), B[r].cpu().numpy()
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat_p[o:o + n], ref.params[i]), f"p[{i}]"
        assert np.array_equal(flat_b[o:o + n], ref.buffers[i]), f"buffer[{i}]"
        want = oracle.f32_to_bf16(ref.params[i]).view(np.int16)
        for r in range(world):
            assert np.array_equal(S[r][o:o + n].cpu().numpy(), want), f"shadow[{i}] on rank {r}"
    for p in plans:
        p.close()


def _sgd_rank_main(rank, world, port, comm, queue):
    import torch.distributed as dist
    from gograd_b200.zero1 import Zero1SGD
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    options = _comm_options(comm, world)
    opt = Zero1SGD(NUMELS, GROUPS, SGD_HP["lr"], SGD_HP["momentum"], SGD_HP["dampening"], SGD_HP["nesterov"],
                   SGD_HP["maximize"], SGD_HP["max_norm"], rank, options.pop("comm"), **options)
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())
    for step in (1, 2, 3):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))
        opt.step()
    torch.cuda.synchronize()
    queue.put((rank, opt.lo, opt.master.cpu().numpy(), opt.buffer.cpu().numpy(),
               opt.shadow_flat.view(torch.int16).cpu().numpy()))
    opt.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("comm", ["peer", "nccl", "abi", "abi+ce"])
def test_two_real_ranks_sgd(comm):
    """The sharded SGD over two real ranks, both data paths, bit-identical to the unsharded oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gograd_b200.zero1 import ShardLayout
    from oracle import oracle
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_sgd_rank_main, args=(r, world, port, comm, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    ref = _oracle_sgd_run(world, 3)
    L = ShardLayout(NUMELS, world)
    flat_p, flat_b = np.zeros(L.total, np.float32), np.zeros(L.total, np.float32)
    for rank, lo, master, buffer, shadow in results:
        flat_p[lo:lo + master.size], flat_b[lo:lo + buffer.size] = master, buffer
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat_p[o:o + n], ref.params[i]), f"p[{i}] ({comm})"
        assert np.array_equal(flat_b[o:o + n], ref.buffers[i]), f"buffer[{i}] ({comm})"
        want = oracle.f32_to_bf16(ref.params[i]).view(np.int16)
        for rank, lo, master, buffer, shadow in results:
            assert np.array_equal(shadow[o:o + n], want), f"rank {rank} shadow[{i}] ({comm})"


def _saving_rank_main(rank, world, port, out_dir, queue):
    import torch.distributed as dist
    from gograd_b200.zero1 import Zero1AdamW
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    opt = Zero1AdamW(NUMELS, GROUPS, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], rank, comm="peer")
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())
    for step in (1, 2):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))
        opt.step()
    names = [f"t{i}" for i in range(len(NUMELS))]
    shapes = [[n] for n in NUMELS]
    opt.save_state(os.path.join(out_dir, "streamed.safetensors"), names, shapes)
    opt.save_state(os.path.join(out_dir, "gathered.safetensors"), names, shapes, streaming=False)
    torch.cuda.synchronize()
    queue.put((rank, opt.lo, opt.m.cpu().numpy(), opt.v.cpu().numpy()))
    opt.close()
    dist.destroy_process_group()


def test_two_real_ranks_stream_their_state_into_one_file(tmp_path):
    """Two ranks, tensors straddling the shard boundary: the streamed file (owners send their pieces
    to rank 0 entry by entry) equals the gathered one byte for byte and holds every rank's moments."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gograd_b200 import autograd as ag
    from gograd_b200.zero1 import ShardLayout
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_saving_rank_main, args=(r, world, port, str(tmp_path), queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    streamed = open(tmp_path / "streamed.safetensors", "rb").read()
    assert streamed == open(tmp_path / "gathered.safetensors", "rb").read()
    L = ShardLayout(NUMELS, world)
    flat_m, flat_v = np.zeros(L.total, np.float32), np.zeros(L.total, np.float32)
    for rank, lo, m, v in results:
        flat_m[lo:lo + m.size], flat_v[lo:lo + v.size] = m, v
    d = ag.safetensors_describe(str(tmp_path / "streamed.safetensors"))
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert d["entries"][f"m.{i}"]["shape"] == [n]
        for key, flat in (("m", flat_m), ("v", flat_v)):
            want = flat[o:o + n].astype(np.float64)
            assert abs(d["entries"][f"{key}.{i}"]["sum"] - float(want.sum())) <= 1e-9 * float(np.abs(want).sum()) + 1e-30


def _leaving_rank_main(rank, world, port, queue):
    """Rank 1 leaves after step 1, between steps: every rank has synchronised its device and met
    the others in the store first, so nothing of the leaving rank is in flight anywhere."""
    from datetime import timedelta

    import torch.distributed as dist
    from gograd_b200.zero1 import PeerLiveness, RankLost, Zero1AdamW
    os.environ["NCCL_NVLS_ENABLE"] = "0"          # plain peer transport only; no switch-side objects
    torch.cuda.set_device(rank)
    store = dist.TCPStore("127.0.0.1", port, is_master=False, timeout=timedelta(seconds=60))
    dist.init_process_group("nccl", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    opt = Zero1AdamW(NUMELS, GROUPS, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], rank, comm="peer")
    opt.liveness = PeerLiveness(store, rank, world, timeout_s=2.0)
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())

    def load(step):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))

    load(1)
    opt.step()
    torch.cuda.synchronize()
    store.set(f"idle/{rank}", "1")
    store.wait([f"idle/{r}" for r in range(world)], timedelta(seconds=60))   # every device is idle now
    if rank == 1:
        result = "left between steps"
    else:
        before = [t.clone() for t in (opt.master, opt.m, opt.v, opt.shadow_flat.view(torch.int16))]
        load(2)
        try:
            opt.step()
            result = "stepped"
        except RankLost as e:
            torch.cuda.synchronize()               # the context still answers
            after = (opt.master, opt.m, opt.v, opt.shadow_flat.view(torch.int16))
            same = all(bool(torch.equal(a, b)) for a, b in zip(before, after))
            result = (e.missing, e.step, opt.step_count, same)
    if rank == 0:
        opt.close()                                # the survivor cleans up: local, no collective, no barrier
        opt.close()                                # and a second call does nothing
        result = result + (len(opt._imported),)
    queue.put((rank, result))
    queue.close()
    queue.join_thread()
    os._exit(0)                                    # the leaving rank never calls close(); no communicator teardown


def test_a_rank_that_left_is_found_before_the_next_launch():
    """Two real ranks on the peer path. Rank 1 exits between steps with nothing in flight; rank 0's
    next step starts with the roll call, which names rank 1 within its limit and launches nothing:
    the step counter, the shard of p/m/v and the shadow keep their values and the device still works."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from datetime import timedelta

    import torch.distributed as dist
    import torch.multiprocessing as mp
    world = 2
    server = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False, timeout=timedelta(seconds=60))
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_leaving_rank_main, args=(r, world, server.port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results[1] == "left between steps"
    assert results[0] == ([1], 2, 1, True, 0), results


def test_sharded_state_file_loads_into_unsharded_adamw_and_back(tmp_path):
    """The sharded optimizer writes its gathered moments in the reference's per-tensor layout
    ("gograd-adamw": m.<i>, v.<i>, configuration metadata). The unsharded host-mirror AdamW loads that
    file and both continue bit for bit; the file the unsharded optimizer writes loads back into a
    sharded one. One rank on one GPU is enough to exercise the layout code."""
    import torch.distributed as dist
    from gograd_b200 import autograd as ag
    from gograd_b200.zero1 import Zero1AdamW

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        names = [f"t{i}" for i in range(len(NUMELS))]
        shapes = [[n] for n in NUMELS]
        groups = [(1.0, 0.1)] * len(NUMELS)
        z = Zero1AdamW(NUMELS, groups, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], 0, comm="peer")
        L = z.layout
        weights = torch.zeros(L.total)
        for o, w in zip(L.offsets, _weights()):
            weights[o:o + w.size] = torch.from_numpy(w)
        z.load_master(weights.cuda())

        def sharded_step(opt, step):
            opt.grad_flat.zero_()
            for view, g in zip(opt.grads, _grads(0, step)):
                view.copy_(torch.from_numpy(g))
            opt.step()

        for step in (1, 2):
            sharded_step(z, step)
        path = str(tmp_path / "sharded.safetensors")
        z.save_state(path, names, shapes)                       # streamed, entry by entry
        gathered = str(tmp_path / "gathered.safetensors")
        z.save_state(gathered, names, shapes, streaming=False)  # all of m and v in host memory first
        assert open(path, "rb").read() == open(gathered, "rb").read()
        d = ag.safetensors_describe(path)
        assert d["metadata"]["format"] == "gograd-adamw" and d["metadata"]["step_count"] == "2"
        assert sorted(d["entries"]) == sorted([f"m.{i}" for i in range(len(NUMELS))] + [f"v.{i}" for i in range(len(NUMELS))])
        # unsharded optimizer over the same weights
        torch.cuda.synchronize()
        flat = z.master.cpu().numpy()
        params = [ag.Parameter(n, ag.Tensor(flat[o:o + k])) for n, o, k in zip(names, L.offsets, NUMELS)]
        u = ag.NewAdamW(params, 1.0, 0.1)
        u.LoadSafeTensors(path)
        assert u.StepCount == 2 and u.LearningRate() == np.float32(HP["lr"])
        sharded_step(z, 3)
        for p, g in zip(params, _grads(0, 3)):
            p.Value.set_grad(g)
        u.StepClipped(HP["max_norm"])
        torch.cuda.synchronize()
        flat = z.master.cpu().numpy()
        for p, o, k in zip(params, L.offsets, NUMELS):
            assert np.array_equal(p.Value.to_host(), flat[o:o + k]), p.Name
        # and back: the unsharded file into a fresh sharded optimizer
        back = str(tmp_path / "unsharded.safetensors")
        u.SaveSafeTensors(back)
        z2 = Zero1AdamW(NUMELS, groups, 9.0, 0.5, 0.5, 1e-3, HP["max_norm"], 0, comm="nccl")
        z2.load_master(z.master.new_zeros(L.total).index_copy_(0, torch.arange(L.shard_len, device="cuda"), z.master))
        z2.load_state(back, names, shapes)
        assert z2.step_count == 3 and np.float32(z2.lr) == np.float32(HP["lr"]) and np.float32(z2.beta2) == np.float32(HP["beta2"])
        assert torch.equal(z2.m, z.m) and torch.equal(z2.v, z.v)
        sharded_step(z, 4)
        sharded_step(z2, 4)
        torch.cuda.synchronize()
        assert torch.equal(z2.master, z.master) and torch.equal(z2.shadow_flat, z.shadow_flat)
        with pytest.raises(ValueError, match="name or shape"):
            z2.load_state(back, names[::-1], shapes)
        z.close()
        z2.close()
    finally:
        dist.destroy_process_group()


def test_chunk_range_steps_and_accumulated_norm_equal_whole_launches():
    """Piecewise forms of the two sharded-step kernels, on one GPU: the update over consecutive ranges of
    work units equals one launch over the plan, and a shard reduced range by range with
    OE_ACCUMULATE leaves the same reduced values and a sum of squares equal up to summation order."""
    import gograd_b200 as eng
    from gograd_b200.engine import OE_ACCUMULATE, OE_PARTIAL_ONLY, OE_WRITE_SHADOW
    from gograd_b200.workload import bias_corrections

    eng.init(0)
    rng = np.random.default_rng(4)
    sizes = [20000, 5, 4097, 12289]
    state = {}
    for tag in ("whole", "ranged"):
        r = np.random.default_rng(4)
        state[tag] = [[torch.from_numpy(r.normal(0, s, n).astype(np.float32)).cuda() for s in (.02, .01)] +
                      [torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"),
                       torch.zeros(n, dtype=torch.int16, device="cuda")] for n in sizes]
    plans = {tag: eng.Plan([eng.TensorDesc(p, g, m, v, sh, 1.0, 0.1) for p, g, m, v, sh in state[tag]])
             for tag in state}
    b1, b2 = bias_corrections(0.9, 0.999, 1)
    hp = eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, b1, b2, 0.0, OE_WRITE_SHADOW)
    plans["whole"].adamw_step(hp)
    total = plans["ranged"].n_chunks
    unit = plans["ranged"].info(5)      # the work-unit size the library chose for a set this small
    assert unit in (1024, 2048, 4096) and total == sum(-(-n // unit) for n in sizes)
    for first, count in ((0, 2), (2, 0), (2, 3), (5, total - 5)):
        plans["ranged"].adamw_step_chunks(hp, first, count)
    with pytest.raises(eng.engine.EngineError):
        plans["ranged"].adamw_step_chunks(hp, total, 1)
    for a, b in zip(state["whole"], state["ranged"]):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    # reduction of a flat buffer in three ranges against one launch (two "ranks" on one device)
    n = 3 * 8192
    g0 = torch.from_numpy(rng.normal(0, 1e-2, n).astype(np.float32)).cuda()
    g1 = torch.from_numpy(rng.normal(0, 1e-2, n).astype(np.float32)).cuda()
    out_whole, out_ranged = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    plan = plans["whole"]
    plan.peer_reduce_grads([g0.data_ptr(), g1.data_ptr()], 0, n, out_whole.data_ptr(), 0.5, OE_PARTIAL_ONLY)
    _, whole_sq = plan.read_norm()
    for k in range(3):
        plan.peer_reduce_grads([g0.data_ptr(), g1.data_ptr()], k * 8192, 8192, out_ranged.data_ptr() + 4 * k * 8192, 0.5,
                               OE_PARTIAL_ONLY | (OE_ACCUMULATE if k else 0))
    _, ranged_sq = plan.read_norm()
    assert torch.equal(out_whole, out_ranged)
    assert abs(ranged_sq - whole_sq) <= 1e-12 * whole_sq
    want = ((g0 + g1) * 0.5).double().pow(2).sum().item()
    assert abs(whole_sq - want) <= 1e-12 * want
    for p in plans.values():
        p.close()


def _single_rank_group():
    import torch.distributed as dist
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    return dist


def test_one_rank_through_the_library_alone():
    """comm="abi" with a world of one on one GPU: oe_zero1_adamw_step enqueues exchange, pull-reduce,
    exchange with the norm, update, exchange — five launches per step, no collective — and the result
    is the unsharded oracle's, bit for bit. The exchanges of a single rank meet only themselves."""
    import gograd_b200 as eng
    from gograd_b200.zero1 import Zero1AdamW
    from oracle import oracle
    dist = _single_rank_group()
    try:
        opt = Zero1AdamW(NUMELS, GROUPS, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], 0, comm="abi")
        L = opt.layout
        weights = torch.zeros(L.total)
        for o, w in zip(L.offsets, _weights()):
            weights[o:o + w.size] = torch.from_numpy(w)
        opt.load_master(weights.cuda())
        ref, want_norms = _oracle_run(1, 2)
        eng.launch_count_reset()
        for step in (1, 2):
            opt.grad_flat.zero_()
            for view, g in zip(opt.grads, _grads(0, step)):
                view.copy_(torch.from_numpy(g))
            opt.step()
            assert abs(opt.grad_norm() - want_norms[step - 1]) <= 1e-6 * want_norms[step - 1]
        assert opt.exchange_status() == 0
        assert eng.launch_count() == 10 and eng.launch_count("oe_rank_exchange") == 6
        p, m, v = opt.master.cpu().numpy(), opt.m.cpu().numpy(), opt.v.cpu().numpy()
        shadow = opt.shadow_flat.view(torch.int16).cpu().numpy()
        for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
            assert np.array_equal(p[o:o + n], ref.params[i]) and np.array_equal(m[o:o + n], ref.m[i])
            assert np.array_equal(v[o:o + n], ref.v[i])
            assert np.array_equal(shadow[o:o + n], oracle.f32_to_bf16(ref.params[i]).view(np.int16))
        opt.close()
        opt.close()
    finally:
        dist.destroy_process_group()


def test_an_exchange_gives_up_and_the_step_does_nothing():
    """One GPU, a step of two ranks of which the second never arrives: its exchange area is a local
    buffer that nothing writes. The first exchange's wait runs out after its limit (50 ms here), the
    kernel records the missing rank in the status word and RETURNS; the pull-reduce, the update and
    the later exchanges of that step see the word and do nothing, so master weights, moments and
    shadow keep their values. Nothing hangs and the device still answers."""
    import time

    import gograd_b200 as eng
    from gograd_b200.engine import OE_WRITE_SHADOW, OE_ZERO1_SYNC_BYTES, EngineError, Zero1Context
    from gograd_b200.workload import bias_corrections
    eng.init(0)
    n = 3 * 4096
    rng = np.random.default_rng(5)
    mine, absent = (torch.from_numpy(rng.normal(0, 1e-3, 2 * n).astype(np.float32)).cuda() for _ in range(2))
    p = torch.from_numpy(rng.normal(0, .02, n).astype(np.float32)).cuda()
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    shadows = [torch.full((2 * n,), -1, dtype=torch.int16, device="cuda") for _ in range(2)]
    sync = [torch.zeros(OE_ZERO1_SYNC_BYTES // 4, dtype=torch.int32, device="cuda") for _ in range(2)]
    plan = eng.Plan([eng.TensorDesc(p, mine[:n], m, v, shadows[0][:n], 1.0, 0.1)])
    ctx = Zero1Context(plan, 0, 2, 0, n, [mine.data_ptr(), absent.data_ptr()],
                       [0, shadows[1].data_ptr() - shadows[0].data_ptr()], [s.data_ptr() for s in sync], timeout_ms=50)
    before = [t.clone() for t in (p, m, v, mine, shadows[0], shadows[1])]
    b1, b2 = bias_corrections(0.9, 0.999, 1)
    t0 = time.perf_counter()
    ctx.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, b1, b2, 1.0, OE_WRITE_SHADOW))
    with pytest.raises(EngineError) as err:
        ctx.status()
    waited = time.perf_counter() - t0
    assert err.value.code == -6 and "rank 1" in err.value.message            # OE_ERR_DEVICE, names the rank
    word = ctx.status_word()
    assert word & 1 and (word >> 8) & 0xff == 0 and (word >> 16) & 0xff == 1  # timed out at exchange 0, rank 1 missing
    assert 0.04 <= waited < 5.0, waited
    for a, b in zip(before, (p, m, v, mine, shadows[0], shadows[1])):
        assert torch.equal(a, b)
    # the area of this rank shows its own arrival; the absent rank's area received this rank's announcement
    assert int(sync[0][0].item()) == 1 and int(sync[0][1].item()) == 0 and int(sync[1][0].item()) == 1
    # the device still works and the word is sticky: a second step is skipped at once
    ctx.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, b1, b2, 1.0, OE_WRITE_SHADOW))
    t1 = time.perf_counter()
    assert ctx.status_word() == word and time.perf_counter() - t1 < 0.04
    assert torch.equal(before[0], p)
    plan.grad_norm()
    assert plan.read_norm()[0] > 0
    ctx.close()
    plan.close()


def test_sharded_sgd_state_file_loads_into_unsharded_sgd_and_back(tmp_path):
    """The sharded SGD writes its momentum buffers in the reference's per-tensor layout ("gograd-sgd":
    buffer.<i> only for initialised parameters, the flags in the metadata). The unsharded host-mirror
    SGD loads that file and both continue bit for bit; the file the unsharded optimizer writes loads
    back into a fresh sharded one; a file saved before the first step has no buffer entry at all."""
    from gograd_b200 import autograd as ag
    from gograd_b200.zero1 import Zero1SGD
    dist = _single_rank_group()
    try:
        names = [f"t{i}" for i in range(len(NUMELS))]
        shapes = [[n] for n in NUMELS]
        groups = [(1.0, 5e-4)] * len(NUMELS)
        hp = dict(lr=0.05, momentum=0.9, dampening=0.0, nesterov=True, maximize=False)

        def make(comm="peer", **over):
            c = dict(hp, **over)
            return Zero1SGD(NUMELS, groups, c["lr"], c["momentum"], c["dampening"], c["nesterov"], c["maximize"],
                            HP["max_norm"], 0, comm)

        z = make()
        L = z.layout
        weights = torch.zeros(L.total)
        for o, w in zip(L.offsets, _weights()):
            weights[o:o + w.size] = torch.from_numpy(w)
        z.load_master(weights.cuda())

        def sharded_step(opt, step):
            opt.grad_flat.zero_()
            for view, g in zip(opt.grads, _grads(0, step)):
                view.copy_(torch.from_numpy(g))
            opt.step()

        empty = str(tmp_path / "before_first_step.safetensors")
        z.save_state(empty, names, shapes)
        d = ag.safetensors_describe(empty)
        assert d["entries"] == {} and d["metadata"]["format"] == "gograd-sgd" and d["metadata"]["step_count"] == "0"
        for step in (1, 2):
            sharded_step(z, step)
        path = str(tmp_path / "sharded.safetensors")
        z.save_state(path, names, shapes)
        d = ag.safetensors_describe(path)
        assert sorted(d["entries"]) == sorted(f"buffer.{i}" for i in range(len(NUMELS)))
        assert d["metadata"]["step_count"] == "2" and '"Initialized":[true,true,true,true,true,true]' in d["metadata"]["optimizer"]
        # the unsharded optimizer over the same weights
        torch.cuda.synchronize()
        flat = z.master.cpu().numpy()
        params = [ag.Parameter(n, ag.Tensor(flat[o:o + k])) for n, o, k in zip(names, L.offsets, NUMELS)]
        u = ag.NewSGD(params, ag.SGDOptions(LR=1.0, Momentum=0.5, WeightDecay=5e-4))
        u.LoadSafeTensors(path)
        assert u.StepCount == 2 and u.LearningRate() == np.float32(hp["lr"])
        sharded_step(z, 3)
        for p, g in zip(params, _grads(0, 3)):
            p.Value.set_grad(g)
        u.StepClipped(HP["max_norm"])
        torch.cuda.synchronize()
        flat = z.master.cpu().numpy()
        for p, o, k in zip(params, L.offsets, NUMELS):
            assert np.array_equal(p.Value.to_host(), flat[o:o + k]), p.Name
        # and back: the unsharded file into a fresh sharded optimizer with other options
        back = str(tmp_path / "unsharded.safetensors")
        u.SaveSafeTensors(back)
        z2 = make("nccl", lr=9.0, momentum=0.5, nesterov=False)
        z2.master.copy_(z.master)
        z2.load_state(back, names, shapes)
        assert z2.step_count == 3 and np.float32(z2.lr) == np.float32(hp["lr"]) and z2.nesterov is True
        assert np.float32(z2.momentum) == np.float32(hp["momentum"])
        assert torch.equal(z2.buffer, z.buffer) and bool((z2.flags == 1).all())
        sharded_step(z, 4)
        sharded_step(z2, 4)
        torch.cuda.synchronize()
        assert torch.equal(z2.master, z.master) and torch.equal(z2.shadow_flat, z.shadow_flat)
        # reject before mutate
        kept = z2.buffer.clone()
        with pytest.raises(ValueError, match="state count"):
            z2.load_state(back, names[::-1], shapes)
        with pytest.raises(ValueError, match="unsupported SGD state format"):
            adamw_file = str(tmp_path / "adamw.safetensors")
            ag.safetensors_write(adamw_file, {}, {"format": "gograd-adamw", "version": "1"})
            z2.load_state(adamw_file, names, shapes)
        assert torch.equal(kept, z2.buffer) and z2.step_count == 4
        # the file from before the first step resets a stepped optimizer to "no buffer yet"
        z2.load_state(empty, names, shapes)
        assert z2.step_count == 0 and bool((z2.flags == 0).all())
        z.close()
        z2.close()
    finally:
        dist.destroy_process_group()


def _sgd_saving_rank_main(rank, world, port, out_dir, queue):
    import torch.distributed as dist
    from gograd_b200.zero1 import Zero1SGD
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    opt = Zero1SGD(NUMELS, GROUPS, SGD_HP["lr"], SGD_HP["momentum"], SGD_HP["dampening"], SGD_HP["nesterov"],
                   SGD_HP["maximize"], SGD_HP["max_norm"], rank, "peer")
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())
    for step in (1, 2):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))
        opt.step()
    names = [f"t{i}" for i in range(len(NUMELS))]
    path = os.path.join(out_dir, "sgd.safetensors")
    opt.save_state(path, names, [[n] for n in NUMELS])
    # a fresh pair of ranks reads the file back: every rank takes its own pieces
    fresh = Zero1SGD(NUMELS, GROUPS, 1.0, 0.5, 0.0, False, False, SGD_HP["max_norm"], rank, "nccl")
    fresh.load_state(path, names, [[n] for n in NUMELS])
    same = bool(torch.equal(fresh.buffer, opt.buffer)) and bool((fresh.flags[:len(fresh.my_pieces)] == 1).all())
    torch.cuda.synchronize()
    queue.put((rank, opt.lo, opt.buffer.cpu().numpy(), same, fresh.step_count))
    fresh.close()
    opt.close()
    dist.destroy_process_group()


def test_two_real_ranks_write_and_read_an_sgd_state_file(tmp_path):
    """Two ranks, tensors straddling the shard boundary: the file holds each tensor's whole momentum
    buffer assembled from both owners' pieces, with one flag per tensor, and splits again on load."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gograd_b200 import autograd as ag
    from gograd_b200.zero1 import ShardLayout
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_sgd_saving_rank_main, args=(r, world, port, str(tmp_path), queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    L = ShardLayout(NUMELS, world)
    flat = np.zeros(L.total, np.float32)
    for rank, lo, buffer, same, step_count in results:
        flat[lo:lo + buffer.size] = buffer
        assert same and step_count == 2
    ref = _oracle_sgd_run(world, 2)
    d = ag.safetensors_describe(str(tmp_path / "sgd.safetensors"))
    assert sorted(d["entries"]) == sorted(f"buffer.{i}" for i in range(len(NUMELS)))
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat[o:o + n], ref.buffers[i])
        want = ref.buffers[i].astype(np.float64)
        assert abs(d["entries"][f"buffer.{i}"]["sum"] - float(want.sum())) <= 1e-9 * float(np.abs(want).sum()) + 1e-30


def _absent_rank_main(rank, world, port, queue):
    """Two real ranks on the abi path. Both take step 1. Rank 1 then sits out step 2 (it stays alive,
    its buffers stay mapped, nothing of it is in flight); rank 0's step 2 therefore meets an exchange
    whose partner never announces itself."""
    import time

    import torch.distributed as dist
    from gograd_b200.engine import EngineError
    from gograd_b200.zero1 import Zero1AdamW
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    opt = Zero1AdamW(NUMELS, GROUPS, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["max_norm"], rank, comm="abi",
                     exchange_timeout_ms=1000)
    L = opt.layout
    weights = torch.zeros(L.total)
    for o, w in zip(L.offsets, _weights()):
        weights[o:o + w.size] = torch.from_numpy(w)
    opt.load_master(weights.cuda())

    def load(step):
        opt.grad_flat.zero_()
        for view, g in zip(opt.grads, _grads(rank, step)):
            view.copy_(torch.from_numpy(g))

    load(1)
    opt.step()
    torch.cuda.synchronize()
    assert opt.exchange_status() == 0
    dist.barrier()
    result = None
    if rank == 0:
        before = [t.clone() for t in (opt.master, opt.m, opt.v, opt.shadow_flat.view(torch.int16))]
        load(2)
        t0 = time.perf_counter()
        opt.step()                       # enqueues five launches; the first one waits for rank 1, in vain
        try:
            opt.exchange_status()
            result = "no error"
        except EngineError as e:
            waited = time.perf_counter() - t0
            after = (opt.master, opt.m, opt.v, opt.shadow_flat.view(torch.int16))
            same = all(bool(torch.equal(a, b)) for a, b in zip(before, after))
            probe = float((opt.master * 0 + 1).sum().item())      # the device still answers
            result = (e.code, "rank 1" in e.message, same, 0.9 <= waited < 20.0, probe == opt.master.numel())
    dist.barrier()                       # rank 1 waited here, on the host side of its own stream
    queue.put((rank, result))
    opt.close()
    dist.destroy_process_group()


def test_a_rank_that_sits_out_a_step_costs_a_time_out_not_a_hang():
    """The library-only sharded step on two real GPUs when one rank does not take part in a step: the
    other rank's exchange kernel gives up after its one-second limit, the status names the absent rank,
    the step's remaining launches do nothing (weights, moments and shadow unchanged), and both GPUs stay
    usable — the next collective between the two processes completes."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_absent_rank_main, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results[1] is None
    assert results[0] == (-6, True, True, True, True), results


def test_link_probes_touch_only_what_they_say():
    """The two link-rate probes on one GPU with two emulated ranks: the read probe stores no element (the
    output range keeps its canary) and leaves the sum of squares of the mean in the norm record; the store
    probe writes bf16 zeros over the given range of the OTHER rank's shadow only."""
    import gograd_b200 as eng
    eng.init(0)
    n = 3 * 4096
    rng = np.random.default_rng(11)
    g = [torch.from_numpy(rng.normal(0, 1e-3, 2 * n).astype(np.float32)).cuda() for _ in range(2)]
    keep = [x.clone() for x in g]
    p = torch.zeros(8, device="cuda")
    plan = eng.Plan([eng.TensorDesc(p, p)])
    plan.link_probe_reads([x.data_ptr() for x in g], n, n)
    _, sumsq = plan.read_norm()
    want = float((g[0][n:] + g[1][n:]).double().pow(2).sum().item())
    assert abs(sumsq - want) <= 1e-12 * want
    assert all(bool(torch.equal(a, b)) for a, b in zip(g, keep))
    shadows = [torch.full((2 * n,), -1, dtype=torch.int16, device="cuda") for _ in range(2)]
    deltas = [0, shadows[1].data_ptr() - shadows[0].data_ptr()]
    plan.link_probe_stores(shadows[0].data_ptr() + 2 * n, deltas, n)
    torch.cuda.synchronize()
    assert bool((shadows[0] == -1).all()), "the caller's own buffer is not a target"
    assert bool((shadows[1][:n] == -1).all()) and bool((shadows[1][n:] == 0).all())
    plan.close()
