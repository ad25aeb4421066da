"""Host-side checks of the sharded step: layout and partition arithmetic, and a world-size-2
run over gloo ranks on the CPU whose arithmetic is the oracle's. The sharded run must end
bit-identical to an unsharded oracle run on the mean gradient."""
import os
import socket

import numpy as np
import pytest

from gograd_b200.zero1 import ShardLayout, Zero1Schedule


def test_layout_partition_properties():
    rng = np.random.default_rng(0)
    for world in (1, 2, 3, 4, 8):
        for _ in range(20):
            numels = [int(x) for x in rng.integers(1, 20000, size=int(rng.integers(1, 12)))]
            L = ShardLayout(numels, world)
            assert L.total == L.shard_len * world and L.shard_len % 4096 == 0 and L.total >= L.used
            assert all(o % 8 == 0 for o in L.offsets)
            covered = np.zeros(L.total, np.int32)
            for r in range(world):
                lo, hi = L.shard_range(r)
                for pc in L.pieces(r):
                    assert lo <= pc.flat_offset and pc.flat_offset + pc.length <= hi
                    assert pc.flat_offset == L.offsets[pc.tensor] + pc.tensor_offset
                    assert pc.flat_offset % 8 == 0, "every piece keeps 128-bit alignment of fp32 and bf16"
                    covered[pc.flat_offset:pc.flat_offset + pc.length] += 1
            for a, b in L.padding_ranges():
                assert np.all(covered[a:b] == 0)
                covered[a:b] -= 1
            assert np.all(np.abs(covered) == 1), "every element is owned exactly once or is padding"
            per_tensor = [0] * len(numels)
            for r in range(world):
                for pc in L.pieces(r):
                    per_tensor[pc.tensor] += pc.length
            assert per_tensor == numels


def test_layout_8b_set_uses_64_bit_offsets():
    from gograd_b200 import paramsets
    ps = paramsets.get("llama8b")
    L = ShardLayout([s.numel for s in ps.params], 8)
    assert L.used >= ps.numel and L.total > 2 ** 32 and L.shard_len == 1_003_786_240
    assert sum(pc.length for r in range(8) for pc in L.pieces(r)) == ps.numel
    with pytest.raises(ValueError):
        ShardLayout([4, 0], 2)
    with pytest.raises(ValueError):
        ShardLayout([4], 0)


class OracleRank(Zero1Schedule):
    """A gloo rank whose arithmetic is the CPU oracle (test infrastructure)."""

    def __init__(self, numels, group_of, hp, rank, world, dist, weights):
        super().__init__(numels, group_of, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["max_norm"], rank, world)
        import torch
        self.dist, self.torch = dist, torch
        L = self.layout
        self.grad_flat = np.zeros(L.total, np.float32)
        self.shadow_flat = np.zeros(L.total, np.uint16)
        flat = np.zeros(L.total, np.float32)
        for o, w in zip(L.offsets, weights):
            flat[o:o + w.size] = w
        self.master = flat[self.lo:self.hi].copy()
        self.m = np.zeros(L.shard_len, np.float32)
        self.v = np.zeros(L.shard_len, np.float32)
        self.norm = 0.0

    def reduce_grads(self):
        t = self.torch.from_numpy(self.grad_flat.copy())
        self.dist.all_reduce(t)                     # two ranks: g0 + g1, commutative, one rounding
        mean = (t.numpy() * np.float32(1.0 / self.world)).astype(np.float32)
        self.grad_flat[self.lo:self.hi] = mean[self.lo:self.hi]
        from oracle import oracle
        self.sumsq = oracle.sum_squares([self.grad_flat[self.lo:self.hi]])

    def combine_sumsq(self):
        t = self.torch.tensor([self.sumsq], dtype=self.torch.float64)
        self.dist.all_reduce(t)
        self.norm = np.float32(np.sqrt(float(t.item())))

    def update(self):
        from oracle import oracle
        coef = oracle.clip_coefficient(float(self.norm), self.max_norm)
        bc1, bc2 = self.bias_corrections()
        for pc in self.my_pieces:
            a, b = pc.flat_offset - self.lo, pc.flat_offset - self.lo + pc.length
            g = self.grad_flat[pc.flat_offset:pc.flat_offset + pc.length].copy()
            oracle.scale_(g, float(coef))
            scale, decay = self.group_of[pc.tensor]
            step, dec = oracle.C.c_float(), oracle.C.c_float()
            oracle.lib().oracle_adamw_group_scale(self.lr, scale, decay, step, dec)
            p, m, v = self.master[a:b], self.m[a:b], self.v[a:b]
            oracle.lib().oracle_adamw_update(oracle._ptr(p), oracle._ptr(g), oracle._ptr(m), oracle._ptr(v), p.size,
                                             self.beta1, self.beta2, self.eps, step.value, dec.value, bc1, bc2)
            self.shadow_flat[pc.flat_offset:pc.flat_offset + pc.length] = oracle.f32_to_bf16(p)

    def gather_shadows(self):
        mine = self.torch.from_numpy(self.shadow_flat[self.lo:self.hi].astype(np.int32))
        out = [self.torch.zeros_like(mine) for _ in range(self.world)]
        self.dist.all_gather(out, mine)
        self.shadow_flat[:] = np.concatenate([x.numpy() for x in out]).astype(np.uint16)


NUMELS = [5000, 3, 4097, 12, 7001]
GROUPS = [(1.0, 0.1), (1.0, 0.0), (0.5, 0.1), (1.0, 0.0), (1.0, 0.1)]
HP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, max_norm=0.01)


def _inputs(rank, step):
    rng = np.random.default_rng(1000 * step + rank)
    return [rng.normal(0, 1e-3, n).astype(np.float32) for n in NUMELS]


def _weights():
    rng = np.random.default_rng(77)
    return [rng.normal(0, 0.02, n).astype(np.float32) for n in NUMELS]


def _worker(rank, world, port, queue):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    opt = OracleRank(NUMELS, GROUPS, HP, rank, world, dist, _weights())
    norms = []
    for step in range(1, 4):
        opt.grad_flat[:] = 0
        for o, g in zip(opt.layout.offsets, _inputs(rank, step)):
            opt.grad_flat[o:o + g.size] = g
        opt.step()
        norms.append(float(opt.norm))
    queue.put((rank, opt.lo, opt.master.copy(), opt.m.copy(), opt.v.copy(), opt.shadow_flat.copy(), norms))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_unsharded_oracle():
    import torch.multiprocessing as mp
    from oracle import oracle
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # unsharded oracle on the mean gradient
    weights = _weights()
    groups = [oracle.Group(f"g{i}", [i], s, d) for i, (s, d) in enumerate(GROUPS)]
    ref = oracle.OracleAdamW([w.copy() for w in weights], lr=HP["lr"], groups=groups, beta1=HP["beta1"],
                             beta2=HP["beta2"], eps=HP["eps"])
    want_norms = []
    for step in range(1, 4):
        g0, g1 = _inputs(0, step), _inputs(1, step)
        mean = [((a + b) * np.float32(0.5)).astype(np.float32) for a, b in zip(g0, g1)]
        norm, _ = oracle.clip_grad_norm(mean, HP["max_norm"])
        want_norms.append(float(norm))
        ref.step(mean)
    L = ShardLayout(NUMELS, world)
    flat_p = np.zeros(L.total, np.float32)
    flat_m = np.zeros(L.total, np.float32)
    flat_v = np.zeros(L.total, np.float32)
    for rank, lo, master, m, v, shadow, norms in results:
        flat_p[lo:lo + master.size], flat_m[lo:lo + m.size], flat_v[lo:lo + v.size] = master, m, v
        for a, b in zip(norms, want_norms):
            assert abs(a - b) <= 1e-6 * b
    for i, (o, n) in enumerate(zip(L.offsets, NUMELS)):
        assert np.array_equal(flat_p[o:o + n], ref.params[i]), f"p[{i}]"
        assert np.array_equal(flat_m[o:o + n], ref.m[i]) and np.array_equal(flat_v[o:o + n], ref.v[i])
        for rank, lo, master, m, v, shadow, norms in results:
            assert np.array_equal(shadow[o:o + n], oracle.f32_to_bf16(ref.params[i])), f"rank {rank} shadow[{i}]"


def _mismatch_worker(rank, world, port, queue):
    import torch.distributed as dist
    from gograd_b200.zero1 import layout_fingerprint, verify_same_layout
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    numels = list(NUMELS)
    if rank == 1:
        numels[2] += 1          # one rank was built from another model
    fp = layout_fingerprint(ShardLayout(numels, world), GROUPS, (1e-3, .9, .95, 1e-8, 1.0))
    try:
        verify_same_layout(dist, fp)
        queue.put((rank, "accepted"))
    except RuntimeError as e:
        queue.put((rank, str(e)))
    same = layout_fingerprint(ShardLayout(NUMELS, world), GROUPS, (1e-3, .9, .95, 1e-8, 1.0))
    verify_same_layout(dist, same)   # identical configurations pass
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_with_different_layouts_refuse_to_start():
    """A rank configured from another parameter list is detected on the host, on every rank, before
    any kernel could read the wrong ranges of a peer's buffer."""
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_mismatch_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all("ranks [1] were configured differently" in results[r] for r in range(world)), results


def _roll_call_worker(rank, world, port, queue):
    from datetime import timedelta

    import torch.distributed as dist
    from gograd_b200.zero1 import PeerLiveness, RankLost
    store = dist.TCPStore("127.0.0.1", port, is_master=False, timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world)
    opt = OracleRank(NUMELS, GROUPS, HP, rank, world, dist, _weights())
    opt.liveness = PeerLiveness(store, rank, world, timeout_s=2.0)

    def load(step):
        opt.grad_flat[:] = 0
        for o, g in zip(opt.layout.offsets, _inputs(rank, step)):
            opt.grad_flat[o:o + g.size] = g

    load(1)
    opt.step()
    if rank == 1:
        queue.put((rank, "left between steps"))   # no kernel, no collective of this rank is in flight
        return
    before = (opt.master.copy(), opt.m.copy(), opt.v.copy(), opt.shadow_flat.copy())
    load(2)
    try:
        opt.step()
        queue.put((rank, "stepped"))
    except RankLost as e:
        same = all(np.array_equal(a, b) for a, b in zip(before, (opt.master, opt.m, opt.v, opt.shadow_flat)))
        queue.put((rank, (e.missing, e.step, opt.step_count, same)))


def test_a_rank_that_left_is_found_on_the_host_before_the_next_step():
    """Three gloo ranks; rank 1 leaves after step 1. The others learn of it from the roll call in
    the key-value store within its limit: step 2 launches nothing, the step counter and the state
    keep their values, and the error names the missing rank."""
    from datetime import timedelta

    import torch.distributed as dist
    import torch.multiprocessing as mp
    world = 3
    server = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False, timeout=timedelta(seconds=30))
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_roll_call_worker, args=(r, world, server.port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[1] == "left between steps"
    for r in (0, 2):
        assert results[r] == ([1], 2, 1, True), results


def test_roll_call_passes_when_everyone_is_there():
    from datetime import timedelta

    import torch.distributed as dist
    from gograd_b200.zero1 import PeerLiveness
    server = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False, timeout=timedelta(seconds=30))
    # every participant talks to the store over a connection of its own, as ranks do: one client
    # object shared by two threads would interleave their requests on one socket
    client = dist.TCPStore("127.0.0.1", server.port, is_master=False, timeout=timedelta(seconds=30))
    a, b = PeerLiveness(server, 0, 2, 20.0), PeerLiveness(client, 1, 2, 20.0)
    import threading
    failures = []

    def other(step):
        try:
            b.arrive(step)
        except Exception as e:   # reported by the test's own assertion, not as a stray thread warning
            failures.append(e)

    for step in range(1, 6):
        t = threading.Thread(target=other, args=(step,))
        t.start()
        a.arrive(step)
        t.join()
    assert failures == []
    assert not server.check(["oe/alive/1/0"]) and server.check(["oe/alive/5/0"])
    with pytest.raises(ValueError):
        PeerLiveness(server, 0, 2, 0.0)


def _sgd_state_worker(rank, world, port, out_dir, queue):
    """A gloo rank that holds its shard of momentum buffers in CPU tensors and uses the sharded SGD's
    own save_state / load_state (the file code needs no GPU: only the tensors' home differs)."""
    import torch
    import torch.distributed as dist
    from gograd_b200.zero1 import Zero1Schedule, Zero1SGD

    class CpuSGDRank(Zero1SGD):
        def __init__(self, momentum):
            Zero1Schedule.__init__(self, NUMELS, GROUPS, 0.05, momentum, 0.0, 0.0, 1.0, rank, world)
            self.torch, self.dist, self.pg = torch, dist, None
            self.momentum, self.dampening, self.nesterov, self.maximize = momentum, 0.0, False, False
            self.buffer = torch.zeros(self.layout.shard_len)
            self.flags = torch.zeros(max(len(self.my_pieces), 1))
            self.loaded = 0

        def _device_sync(self):
            pass

        def _state_loaded(self):
            self.loaded += 1

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    names = [f"t{i}" for i in range(len(NUMELS))]
    shapes = [[n] for n in NUMELS]
    opt = CpuSGDRank(0.9)
    # tensor 1 (3 elements) never received a gradient: its buffer stays uninitialised
    full = [np.random.default_rng(50 + i).normal(0, 1, n).astype(np.float32) for i, n in enumerate(NUMELS)]
    for k, pc in enumerate(opt.my_pieces):
        if pc.tensor == 1:
            continue
        a = pc.flat_offset - opt.lo
        opt.buffer[a:a + pc.length] = torch.from_numpy(full[pc.tensor][pc.tensor_offset:pc.tensor_offset + pc.length])
        opt.flags[k] = 1.0
    opt.step_count = 7
    path = os.path.join(out_dir, "sgd.safetensors")
    opt.save_state(path, names, shapes)
    fresh = CpuSGDRank(0.5)
    fresh.load_state(path, names, shapes)
    same = bool(torch.equal(fresh.buffer, opt.buffer)) and bool(torch.equal(fresh.flags, opt.flags))
    errors = []
    kept = fresh.buffer.clone()
    for bad_names, bad_shapes in ((names[::-1], shapes), (names, [[n + 1] for n in NUMELS])):
        try:
            fresh.load_state(path, bad_names, bad_shapes)
            errors.append("accepted")
        except ValueError as e:
            errors.append(str(e))
    plain = CpuSGDRank(0.0)
    try:
        plain.load_state(path, names, shapes)
        errors.append("accepted")
    except ValueError as e:
        errors.append(str(e))
    untouched = bool(torch.equal(kept, fresh.buffer)) and fresh.loaded == 1 and plain.loaded == 0
    # a tensor whose pieces disagree about being initialised cannot be written
    torn = None
    if world > 1:
        split = CpuSGDRank(0.9)
        split.step_count = 1
        if rank == 0:
            split.flags[:] = 1.0
        try:
            split.save_state(os.path.join(out_dir, "torn.safetensors"), names, shapes)
            torn = "written"
        except ValueError as e:
            torn = str(e)
    queue.put((rank, same, fresh.step_count, float(np.float32(fresh.momentum)), errors, untouched, torn))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_write_and_read_a_sharded_sgd_state_file(tmp_path):
    """Sharded SGD state files on the CPU: two gloo ranks stream their pieces into one "gograd-sgd" file
    (one entry per initialised tensor, one flag per tensor reassembled from the pieces' flags), read it
    back piece by piece, reject files that do not fit before changing anything, and refuse to write a
    tensor that is initialised on one owner only."""
    import json

    import torch.multiprocessing as mp
    from gograd_b200 import autograd as ag
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_sgd_state_worker, args=(r, world, port, str(tmp_path), queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([queue.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, step_count, momentum, errors, untouched, torn in results:
        assert same and step_count == 7 and momentum == float(np.float32(0.9)) and untouched
        assert "state count" in errors[0] and "state count" in errors[1] and "disagree on momentum" in errors[2]
        assert "initialised on some ranks only" in torn
    d = ag.safetensors_describe(str(tmp_path / "sgd.safetensors"))
    assert sorted(d["entries"]) == sorted(f"buffer.{i}" for i in range(len(NUMELS)) if i != 1)
    cfg = json.loads(d["metadata"]["optimizer"])
    assert cfg["Initialized"] == [True, False, True, True, True] and cfg["StepCount"] == 7
    assert list(cfg) == ["StepCount", "Names", "Shapes", "Options", "Initialized", "Buffers", "Groups"]
    assert list(cfg["Options"]) == ["LR", "Momentum", "Dampening", "WeightDecay", "Nesterov", "Maximize"]
    for i, n in enumerate(NUMELS):
        if i == 1:
            continue
        want = np.random.default_rng(50 + i).normal(0, 1, n).astype(np.float32).astype(np.float64)
        assert d["entries"][f"buffer.{i}"]["shape"] == [n]
        assert abs(d["entries"][f"buffer.{i}"]["sum"] - float(want.sum())) <= 1e-9 * float(np.abs(want).sum())
    assert not (tmp_path / "torn.safetensors").exists()
