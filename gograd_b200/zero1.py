"""Sharded (ZeRO-1 style) AdamW step: one process per GPU, state partitioned over ranks.

The reference has no distributed code; this is the data-parallel form of its optimizer
step. Every rank holds a full flat fp32 gradient buffer (its own gradients, input) and a
full flat bf16 shadow buffer (output, what the next forward reads); master weights, m and
v exist only on the rank that owns their shard. One step:

    1. reduce-scatter the gradients (mean over ranks) into the owner's shard
    2. sum of squares of the shard -> all-reduce of one float64 -> global norm
    3. fused AdamW on the shard with the clip coefficient folded in
    4. all-gather of the bf16 shadows

Three ways to run it (`comm`):

  "peer"  hand-written kernels over peer-mapped memory (CUDA IPC, plain loads/stores):
          step 1+2 are ONE kernel (each rank pulls its shard from every rank, adds in
          ascending rank order, writes the mean and accumulates its squares), step 3+4 are
          ONE kernel (the update stores each bf16 value into every rank's shadow buffer).
          The only library collective is the 8-byte all-reduce, which also orders the
          ranks: nothing in the kernels waits on another GPU.
  "abi"   the same two kernels, but the three points where the ranks meet are the library's own
          exchange kernels too (oe_zero1_*: peer stores into an exchange area of every rank and a
          bounded wait): one C call per step and no torch.distributed call inside it — what a host
          without a collective library uses.
  "nccl"  ncclReduceScatter(avg) + the single-GPU kernels + ncclAllGather: the baseline
          the fused path is measured against.

`multicast=True` (peer and abi) allocates the shadow buffer as torch symmetric memory and lets the
update kernel send every 8-byte shadow vector once through the NVLink multicast mapping instead of
once per rank; values and layout are unchanged.

The flat layout and the partition live in `ShardLayout` (pure Python, tested on CPU with
gloo ranks); `Zero1AdamW` drives either path through torch.distributed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class Piece:
    """The part of one tensor that falls into one rank's shard."""
    tensor: int        # index in the parameter list
    tensor_offset: int  # first element inside the tensor
    flat_offset: int    # first element inside the flat buffer
    length: int


class ShardLayout:
    """Flat layout of a parameter list and its contiguous partition over `world` ranks.

    Tensor i starts at `offsets[i]`, a multiple of `align` elements (8 elements = 32 bytes of
    fp32 and 16 bytes of bf16, so both streams keep their 128-bit alignment); rank r owns
    [r*shard_len, (r+1)*shard_len) with shard_len a multiple of `shard_align`; the gaps and
    the tail are padding that must hold zeros in the gradient buffer. 64-bit offsets: the
    8B-parameter set's flat length exceeds 2^31."""

    def __init__(self, numels: Sequence[int], world: int, align: int = 8, shard_align: int = 4096):
        if world < 1:
            raise ValueError("world size must be positive")
        if align < 1 or shard_align % align != 0:
            raise ValueError("shard_align must be a multiple of align")
        if any(n <= 0 for n in numels):
            raise ValueError("tensors must not be empty")
        self.numels = [int(n) for n in numels]
        self.world = world
        self.align = align
        self.offsets: List[int] = []
        pos = 0
        for n in self.numels:
            pos = -(-pos // align) * align
            self.offsets.append(pos)
            pos += n
        self.used = pos
        per_rank = -(-pos // world)
        self.shard_len = max(shard_align, -(-per_rank // shard_align) * shard_align)
        self.total = self.shard_len * world

    def shard_range(self, rank: int) -> Tuple[int, int]:
        if not 0 <= rank < self.world:
            raise ValueError("rank out of range")
        return rank * self.shard_len, (rank + 1) * self.shard_len

    def pieces(self, rank: int) -> List[Piece]:
        lo, hi = self.shard_range(rank)
        out = []
        for i, (off, n) in enumerate(zip(self.offsets, self.numels)):
            a, b = max(off, lo), min(off + n, hi)
            if a < b:
                out.append(Piece(i, a - off, a, b - a))
        return out

    def padding_ranges(self) -> List[Tuple[int, int]]:
        """[start, end) ranges of the flat buffer that belong to no tensor."""
        gaps, pos = [], 0
        for off, n in zip(self.offsets, self.numels):
            if off > pos:
                gaps.append((pos, off))
            pos = off + n
        if pos < self.total:
            gaps.append((pos, self.total))
        return gaps

    def owner_of(self, flat_index: int) -> int:
        return flat_index // self.shard_len


def layout_fingerprint(layout: ShardLayout, group_of, hparams) -> str:
    """A digest of everything the ranks of a sharded step must agree on."""
    import hashlib
    h = hashlib.sha256()
    h.update(repr((layout.world, layout.align, layout.shard_len, layout.numels)).encode())
    h.update(repr([(float(a), float(b)) for a, b in group_of]).encode())
    h.update(repr([float(x) for x in hparams]).encode())
    return h.hexdigest()


def verify_same_layout(dist, fingerprint: str, group=None) -> None:
    """Every rank publishes its fingerprint; a rank that was built from another parameter list,
    other groups or other hyper-parameters would pull the wrong ranges of its peers' buffers, so
    all ranks raise (each naming the ranks that differ from rank 0) before any device work."""
    world = dist.get_world_size(group)
    everyone = [None] * world
    dist.all_gather_object(everyone, fingerprint, group=group)
    odd = [r for r, f in enumerate(everyone) if f != everyone[0]]
    if odd:
        raise RuntimeError(f"sharded optimizer: ranks {odd} were configured differently from rank 0 "
                           "(parameter sizes, groups or hyper-parameters); refusing to start")


class RankLost(RuntimeError):
    """A rank did not reach the step the others are about to launch."""

    def __init__(self, step: int, missing: Sequence[int], detail: str = ""):
        self.step, self.missing = step, list(missing)
        who = f"ranks {self.missing}" if self.missing else "a rank (the store no longer answers)"
        super().__init__(f"sharded optimizer: {who} did not reach step {step}; nothing was launched"
                         + (f" ({detail})" if detail else ""))


class PeerLiveness:
    """Host-side roll call before a sharded step.

    Every rank writes a key for the step it is about to launch into the job's key-value
    store and waits, with a short limit, for the keys of all the others. A rank that raised,
    exited or never joined is so found on the host, between steps, before any kernel reads a
    peer's buffer or a collective is enqueued that could never complete; the step counter
    and the optimizer state of the surviving ranks are left as they were. The wait is a host
    wait on the store: no GPU work is involved and nothing on a device can block on it."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "oe/alive"):
        if timeout_s <= 0:
            raise ValueError("timeout_s must be positive")
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def arrive(self, step: int) -> None:
        from datetime import timedelta
        keys = [self._key(step, r) for r in range(self.world)]
        try:
            self.store.set(keys[self.rank], "1")
            self.store.wait(keys, timedelta(seconds=self.timeout_s))
        except Exception as e:  # a timeout or a lost connection: find out who is missing
            missing = []
            try:
                missing = [r for r in range(self.world) if not self.store.check([keys[r]])]
            except Exception:
                pass
            raise RankLost(step, missing, type(e).__name__) from e
        if step > 2:  # every rank that passed step-1 has finished reading the keys of step-2
            try:
                self.store.delete_key(self._key(step - 2, self.rank))
            except Exception:
                pass


class _RawCuda:
    """Lets torch view a device address it does not own (the plan's norm record)."""

    def __init__(self, address: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (address, False),
                                         "version": 2}


class Zero1Schedule:
    """What every rank does in one sharded step, independent of where the arithmetic runs.

    Subclasses provide the four phases. `Zero1AdamW` runs them on the GPU through the C ABI;
    the CPU test-suite runs them over gloo ranks to check the layout, the partition and the
    sequencing against an unsharded run."""

    def __init__(self, numels: Sequence[int], group_of: Sequence[Tuple[float, float]], lr: float, beta1: float,
                 beta2: float, eps: float, max_norm: float, rank: int, world: int):
        if len(group_of) != len(numels):
            raise ValueError("one (lr_scale, weight_decay) pair per parameter")
        self.rank, self.world = rank, world
        self.group_of = list(group_of)
        self.lr, self.beta1, self.beta2, self.eps, self.max_norm = lr, beta1, beta2, eps, max_norm
        self.step_count = 0
        self.layout = ShardLayout(numels, world)
        self.lo, self.hi = self.layout.shard_range(rank)
        self.my_pieces = self.layout.pieces(rank)
        self.liveness: Optional[PeerLiveness] = None   # set one to have every step begin with a roll call
        self._lost = False

    def bias_corrections(self) -> Tuple[float, float]:
        from .workload import bias_corrections
        return bias_corrections(self.beta1, self.beta2, self.step_count)

    def step(self) -> None:
        if self.liveness is not None:
            try:
                self.liveness.arrive(self.step_count + 1)   # raises RankLost before anything is launched
            except RankLost:
                self._lost = True
                raise
        self.step_count += 1          # one shared counter, as AdamW.Step keeps (autograd/nn.go:492)
        self.reduce_grads()           # mean over ranks of this rank's shard + its sum of squares
        self.combine_sumsq()          # sum over ranks -> global norm
        self.update()                 # clip folded in, shard of p/m/v, bf16 of the shard
        self.gather_shadows()         # every rank ends with the full bf16 model

    def reduce_grads(self) -> None:
        raise NotImplementedError

    def combine_sumsq(self) -> None:
        raise NotImplementedError

    def update(self) -> None:
        raise NotImplementedError

    def gather_shadows(self) -> None:
        raise NotImplementedError


class Zero1AdamW(Zero1Schedule):
    """Sharded AdamW + clip + bf16 shadow over torch.distributed (NCCL), one rank per GPU.

    group_of[i] = (lr_scale, weight_decay) of parameter i. `comm` selects the path ("peer", "abi"
    or "nccl", see the module text); torch.distributed is used for set-up in every case (exchange
    of the IPC handles, the layout check) and, on the abi path, for nothing after that. Gradients
    are written by the caller into `self.grad_flat` (or the per-tensor views `self.grads`); after
    `step()` every rank's `self.shadow_flat` holds the bf16 weights of the whole model.
    `exchange_timeout_ms` bounds every wait of the abi path's exchange kernels (0 = 10 s).
    `ce_pull_sources` / `ce_push_targets` (abi path): how many peers' gradient ranges a copy stages
    before the pull kernel, and how many ranks get their shadow values from a copy after the update
    kernel; None leaves the choice to the library (by world size and shard size), 0 switches it off.
    The staging buffer (4 bytes x shard length per staged peer) is allocated here. `staging_writers`
    (default) maps every rank's staging on every GPU, so that the staged ranges are written by their
    owners (770 GB/s per GPU on B200 boxes) instead of read by the rank that reduces them (740)."""

    def __init__(self, numels: Sequence[int], group_of: Sequence[Tuple[float, float]], lr: float, beta1: float,
                 beta2: float, eps: float, max_norm: float, device: int, comm: str = "peer", process_group=None,
                 chunk_elems: int = 0, multicast: bool = False, exchange_timeout_ms: int = 0,
                 push_order: str = "ascending", ce_pull_sources: Optional[int] = None,
                 ce_push_targets: Optional[int] = None, staging_writers: bool = True):
        import torch
        import torch.distributed as dist

        from . import engine
        if comm not in ("peer", "nccl", "abi"):
            raise ValueError("comm must be 'peer', 'abi' or 'nccl'")
        if multicast and comm == "nccl":
            raise ValueError("multicast shadow stores belong to the peer and abi paths")
        if push_order not in ("ascending", "rotated"):
            raise ValueError("push_order must be 'ascending' or 'rotated'")
        self.torch, self.dist, self.engine = torch, dist, engine
        self.pg = process_group
        super().__init__(numels, group_of, lr, beta1, beta2, eps, max_norm, dist.get_rank(process_group),
                         dist.get_world_size(process_group))
        self.device = device
        self.comm = comm
        self.multicast = multicast
        self.push_order = push_order
        verify_same_layout(dist, layout_fingerprint(self.layout, group_of, (lr, beta1, beta2, eps, max_norm)),
                           process_group)
        # The peer path reads other ranks' gradient buffers directly: by default a tiny
        # stream-ordered all-reduce at the start of a step makes sure they are complete. A
        # caller that already synchronised its ranks after backward can switch it off.
        self.sync_before_pull = True
        L = self.layout
        dev = torch.device("cuda", device)
        self.grad_flat = torch.zeros(L.total, dtype=torch.float32, device=dev)
        self._symm = None
        if multicast:
            import torch.distributed._symmetric_memory as symm_mem
            self.shadow_flat = symm_mem.empty(L.total, dtype=torch.bfloat16, device=dev)
            self.shadow_flat.zero_()
            group = process_group if process_group is not None else dist.group.WORLD
            self._symm = symm_mem.rendezvous(self.shadow_flat, group)
            if not self._symm.multicast_ptr:
                raise RuntimeError("sharded optimizer: this system offers no NVLink multicast mapping")
        else:
            self.shadow_flat = torch.zeros(L.total, dtype=torch.bfloat16, device=dev)
        self.master = torch.zeros(L.shard_len, dtype=torch.float32, device=dev)
        self._allocate_state(dev)
        self.grads = [self.grad_flat[o:o + n] for o, n in zip(L.offsets, L.numels)]
        self.shadows = [self.shadow_flat[o:o + n] for o, n in zip(L.offsets, L.numels)]
        self.plan = engine.Plan(self._descs(), device, chunk_elems)
        self.sumsq = torch.as_tensor(_RawCuda(self.plan.norm_address(), (1,), "<f8"), device=dev)
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        self._imported: List[int] = []
        self._staging = None
        self.staging_bases: Optional[List[int]] = None
        self.grad_bases: Optional[List[int]] = None
        self.shadow_deltas: Optional[List[int]] = None
        self.mc_delta = 0
        self.ctx = None
        self._closed = False
        self._lost = False   # a roll call found a rank missing: nothing collective may follow
        if comm == "abi":
            # staging for the copy-assisted reduction: what an explicit request needs, else what the library
            # would use (all peers but one from four ranks on, shards of 64 MiB and more)
            if ce_pull_sources is None:
                staged = self.world - 2 if self.world >= 4 and 4 * L.shard_len >= (64 << 20) else 0
            else:
                staged = int(ce_pull_sources)
            self._staging_slot = -(-4 * L.shard_len // 256) * 256
            if staged:
                self._staging = torch.empty(staged * self._staging_slot, dtype=torch.uint8, device=dev)
        if comm in ("peer", "abi"):
            # the exchange area of the abi path: zeroed, exported like the other buffers
            self._sync = torch.zeros(engine.OE_ZERO1_SYNC_BYTES // 4, dtype=torch.int32, device=dev)
            self._map_peers(share_staging=staging_writers)
        if comm == "abi":
            def knob(value):
                return 0 if value is None else (engine.OE_ZERO1_CE_NONE if int(value) == 0 else int(value))

            staged_bytes = self._staging.numel() if self._staging is not None else 0
            self.ctx = engine.Zero1Context(self.plan, self.rank, self.world, self.lo, L.shard_len, self.grad_bases,
                                           self.shadow_deltas, self.sync_bases, self.mc_delta, exchange_timeout_ms,
                                           staging=self._staging.data_ptr() if staged_bytes else 0,
                                           staging_bytes=staged_bytes, ce_pull_sources=knob(ce_pull_sources),
                                           ce_push_targets=knob(ce_push_targets), staging_bases=self.staging_bases)

    def _allocate_state(self, dev) -> None:
        torch = self.torch
        self.m = torch.zeros(self.layout.shard_len, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.layout.shard_len, dtype=torch.float32, device=dev)

    def _descs(self):
        """One descriptor per piece of a tensor inside this rank's shard."""
        lo, descs = self.lo, []
        for pc in self.my_pieces:
            a, b = pc.flat_offset, pc.flat_offset + pc.length
            scale, decay = self.group_of[pc.tensor]
            descs.append(self.engine.TensorDesc(self.master[a - lo:b - lo], self.grad_flat[a:b], self.m[a - lo:b - lo],
                                                self.v[a - lo:b - lo], self.shadow_flat[a:b], scale, decay))
        return descs

    # ---- peer mapping (CUDA IPC through the C ABI) -------------------------------------
    def _map_peers(self, share_staging: bool = False) -> None:
        eng, dist = self.engine, self.dist
        mine = {"grad": eng.ipc_export(self.grad_flat.data_ptr(), self.device),
                "sync": eng.ipc_export(self._sync.data_ptr(), self.device)}
        if self._symm is None:
            mine["shadow"] = eng.ipc_export(self.shadow_flat.data_ptr(), self.device)
        own = {"grad": self.grad_flat.data_ptr(), "sync": self._sync.data_ptr(), "shadow": self.shadow_flat.data_ptr()}
        if share_staging and self._staging is not None:
            mine["staging"] = eng.ipc_export(self._staging.data_ptr(), self.device)
            own["staging"] = self._staging.data_ptr()
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.pg)
        opened = {}
        seen = {key: [] for key in own}
        for r, info in enumerate(everyone):
            for key in own:
                if r == self.rank:
                    seen[key].append(own[key])
                elif key not in info:       # symmetric memory: the rendezvous already mapped every rank's buffer
                    seen[key].append(int(self._symm.buffer_ptrs[r]))
                else:
                    handle, offset = info[key]
                    if handle not in opened:  # several buffers may live in one allocation
                        opened[handle] = eng.ipc_import(handle, self.device)
                        self._imported.append(opened[handle])
                    seen[key].append(opened[handle] + offset)
        self.grad_bases, self.sync_bases = seen["grad"], seen["sync"]
        self.staging_bases = seen.get("staging")
        self.shadow_deltas = [a - own["shadow"] for a in seen["shadow"]]
        if self._symm is not None:
            self.mc_delta = int(self._symm.multicast_ptr) - own["shadow"]
        dist.barrier(group=self.pg)

    def _push_deltas(self) -> List[int]:
        """The order in which the update kernel issues its plain shadow stores: ascending rank, or
        starting after this rank and ending with it, so that the ranks do not all store to the same
        GPU first."""
        if self.push_order == "ascending":
            return self.shadow_deltas
        return [self.shadow_deltas[(self.rank + 1 + j) % self.world] for j in range(self.world)]

    # ---- helpers --------------------------------------------------------------------------
    def zero_padding(self) -> None:
        for a, b in self.layout.padding_ranges():
            self.grad_flat[a:b].zero_()

    def load_master(self, flat_weights) -> None:
        """Every rank takes its shard out of a full flat fp32 weight tensor (same on all ranks)."""
        self.master.copy_(flat_weights[self.lo:self.hi])

    def _hparams(self, flags: int):
        b1, b2 = self.bias_corrections()
        return self.engine.AdamWHParams(self.lr, self.beta1, self.beta2, self.eps, b1, b2, self.max_norm, flags)

    def step(self) -> None:
        if self.comm != "abi":
            return super().step()
        # one C call enqueues the five launches of the step; no collective library is involved
        if self.liveness is not None:
            self._roll_call()
        self.step_count += 1
        self._abi_step()

    def _roll_call(self) -> None:
        try:
            self.liveness.arrive(self.step_count + 1)
        except RankLost:
            self._lost = True
            raise

    def _abi_step(self) -> None:
        from .engine import OE_WRITE_SHADOW
        self.ctx.adamw_step(self._hparams(OE_WRITE_SHADOW))

    def exchange_status(self) -> int:
        """abi path: waits for the stream and raises EngineError if a rank missed an exchange."""
        return self.ctx.status() if self.ctx is not None else 0

    # ---- the four phases; all work is enqueued on the current torch stream, no host sync ----
    def reduce_grads(self) -> None:
        from .engine import OE_PARTIAL_ONLY
        dist = self.dist
        own = self.grad_flat[self.lo:self.hi]
        if self.comm == "nccl":
            dist.reduce_scatter_tensor(own, self.grad_flat, op=dist.ReduceOp.AVG, group=self.pg)
            self.plan.grad_norm(OE_PARTIAL_ONLY)
            return
        if self.comm == "abi":
            self.ctx.exchange(0)
            self.ctx.reduce()      # staged copies, if the context uses them, then the pull kernel
            return
        if self.sync_before_pull:
            # every rank's gradients must be complete before anyone pulls them
            dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.pg)
        self.plan.peer_reduce_grads(self.grad_bases, self.lo, self.layout.shard_len, own.data_ptr(),
                                    1.0 / self.world, OE_PARTIAL_ONLY)

    def combine_sumsq(self) -> None:
        if self.comm == "abi":
            self.ctx.exchange(1)   # partial sums exchanged and added in rank order, norm finalised
            return
        # 8 bytes; on the peer path this is also the point after which every rank's pull is over
        self.dist.all_reduce(self.sumsq, op=self.dist.ReduceOp.SUM, group=self.pg)
        self.plan.norm_finalize()

    def update(self) -> None:
        from .engine import OE_WRITE_SHADOW
        hp = self._hparams(OE_WRITE_SHADOW)
        if self.comm == "nccl":
            self.plan.adamw_step(hp)
        elif self.comm == "abi":
            self.ctx.adamw_update(hp)   # shadow stores, then the shadow copies the context uses
        elif self.multicast:
            self.plan.adamw_step_multicast(hp, self.shadow_deltas, self.mc_delta)
        else:
            self.plan.adamw_step_peers(hp, self._push_deltas())

    def gather_shadows(self) -> None:
        dist = self.dist
        if self.comm == "abi":
            self.ctx.exchange(2)
        elif self.comm == "peer":
            # the update kernel already stored into every rank's buffer; once this tiny reduction
            # returns, every rank's stores are complete on every GPU
            dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.pg)
        else:
            dist.all_gather_into_tensor(self.shadow_flat, self.shadow_flat[self.lo:self.hi], group=self.pg)

    def grad_norm(self) -> float:
        return self.plan.read_norm()[0]

    # ---- checkpoint I/O in the reference's per-tensor layout -----------------------------
    def groups(self):
        """(name, member indexes, lr_scale, weight_decay) per distinct group value, in order of first
        appearance; a single group is called "default" as the flat constructors of the reference do."""
        seen = {}
        for i, key in enumerate(self.group_of):
            seen.setdefault(key, []).append(i)
        if len(seen) == 1:
            (scale, decay), members = next(iter(seen.items()))
            return [("default", members, scale, decay)]
        return [(f"group{k}", members, scale, decay) for k, ((scale, decay), members) in enumerate(seen.items())]

    def save_state(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]], streaming: bool = True) -> None:
        """Rank 0 writes the sharded moments as a "gograd-adamw" state file: entries m.<i> / v.<i> of
        shape [numel] per parameter plus the configuration metadata, the layout an unsharded AdamW
        reads back (autograd/optimizer_state.go:142-226).

        streaming (default): the file is written front to back in the order it stores its entries;
        for each entry the owners send their pieces to rank 0, which appends them, so rank 0 never
        holds more than one piece on the host. streaming=False gathers all of m and v on rank 0
        first (12 bytes of host memory per parameter of the model) and writes from memory; both
        produce the same bytes."""
        if not streaming:
            return self._save_state_gathered(path, names, shapes)
        groups = self.groups()
        stream = None
        if self.rank == 0:
            from . import autograd as host
            stream = host.AdamWStateStream(path, list(names), [list(s) for s in shapes], self.step_count, self.lr,
                                           groups[0][3], self.beta1, self.beta2, self.eps, groups)
        # every rank walks the same order: the file's (sorted entry names)
        order = sorted([f"{k}.{i}" for k in ("m", "v") for i in range(len(self.layout.numels))])
        self._stream_entries(stream, order, lambda key: self.m if key == "m" else self.v)

    def _stream_entries(self, stream, order: Sequence[str], shard_of) -> None:
        """Sends the entries `order` ("<key>.<tensor index>", in file order) to the writer on rank 0:
        for each entry the owners pass their pieces of `shard_of(key)` to rank 0, which appends them, so
        rank 0 holds one piece on the host at a time. `stream` is the writer on rank 0, None elsewhere."""
        torch, dist = self.torch, self.dist
        L = self.layout
        # who holds which part of every tensor: (rank, offset in the rank's shard, length), by rank
        holders: List[List[Tuple[int, int, int]]] = [[] for _ in L.numels]
        for r in range(self.world):
            lo, _ = L.shard_range(r)
            for pc in L.pieces(r):
                holders[pc.tensor].append((r, pc.flat_offset - lo, pc.length))
        try:
            bounce = None
            for entry in order:
                key, index = entry.split(".")
                shard = shard_of(key)
                for r, a, n in holders[int(index)]:
                    if self.rank == 0:
                        if r == 0:
                            piece = shard[a:a + n]
                        else:
                            if bounce is None or bounce.numel() < n:
                                bounce = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=shard.device)
                            piece = bounce[:n]
                            dist.recv(piece, src=r, group=self.pg)
                        stream.append(entry, piece.cpu().numpy())
                    elif self.rank == r:
                        dist.send(shard[a:a + n].contiguous(), dst=0, group=self.pg)
            if self.rank == 0:
                assert stream.next() is None
                stream.finish()
        except BaseException:
            if stream is not None:
                stream.abort()
            raise
        if self.world > 1:
            dist.barrier(group=self.pg)

    def _save_state_gathered(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]]) -> None:
        torch, dist = self.torch, self.dist
        gathered = {}
        for key, shard in (("m", self.m), ("v", self.v)):
            parts = [torch.empty_like(shard) for _ in range(self.world)] if self.rank == 0 else None
            if self.world > 1:
                dist.gather(shard, parts, dst=0, group=self.pg)
            else:
                parts = [shard]
            if self.rank == 0:
                gathered[key] = torch.cat(parts).cpu().numpy()
        if self.rank == 0:
            from . import autograd as host
            L = self.layout
            m = [gathered["m"][o:o + n] for o, n in zip(L.offsets, L.numels)]
            v = [gathered["v"][o:o + n] for o, n in zip(L.offsets, L.numels)]
            groups = self.groups()
            host.adamw_state_write(path, list(names), [list(s) for s in shapes], m, v, self.step_count, self.lr,
                                   groups[0][3], self.beta1, self.beta2, self.eps, groups)
        if self.world > 1:
            dist.barrier(group=self.pg)

    def load_state(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]]) -> None:
        """Every rank reads the file and takes its shard of m and v. The file is checked first
        (format, names, shapes, sizes, finite moments, v >= 0, group layout) and nothing is changed
        when a check fails (autograd/optimizer_state.go:228-259)."""
        import json
        import struct

        import numpy as np
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(hlen))
            base = 8 + hlen
            meta = header.pop("__metadata__", {})
            if meta.get("format") != "gograd-adamw" or meta.get("version") != "1":
                raise ValueError("autograd: not an optimizer state")
            cfg = json.loads(meta["optimizer"])
            n = len(self.layout.numels)
            if cfg["StepCount"] != int(meta["step_count"]) or len(header) != 2 * n:
                raise ValueError("autograd: optimizer state count or step mismatch")
            if list(cfg["Names"] or []) != list(names) or [list(s) for s in (cfg["Shapes"] or [])] != [list(s) for s in shapes]:
                raise ValueError("autograd: optimizer parameter name or shape mismatch")
            saved_groups = cfg.get("Groups") or []
            live = self.groups()
            if len(saved_groups) != len(live) or any(
                    [names[i] for i in g[1]] != sg["Names"] for g, sg in zip(live, saved_groups)):
                raise ValueError("autograd: saved parameter groups do not match the live optimizer")
            staged = {"m": np.zeros(self.layout.shard_len, np.float32), "v": np.zeros(self.layout.shard_len, np.float32)}
            for pc in self.my_pieces:
                for key in ("m", "v"):
                    entry = header.get(f"{key}.{pc.tensor}")
                    if entry is None or entry["dtype"] != "F32" or entry["shape"] != [self.layout.numels[pc.tensor]]:
                        raise ValueError(f"autograd: optimizer state is missing parameter {pc.tensor}")
                    f.seek(base + entry["data_offsets"][0] + 4 * pc.tensor_offset)
                    values = np.frombuffer(f.read(4 * pc.length), dtype="<f4")
                    if not np.all(np.isfinite(values)) or (key == "v" and np.any(values < 0)):
                        raise ValueError(f"autograd: invalid optimizer moment {pc.tensor}")
                    a = pc.flat_offset - self.lo
                    staged[key][a:a + pc.length] = values
        self.m.copy_(self.torch.from_numpy(staged["m"]))
        self.v.copy_(self.torch.from_numpy(staged["v"]))
        # the saved groups carry their own scale and decay (autograd/param_groups.go:225-251)
        for g, sg in zip(live, saved_groups):
            scale = float(np.float32(sg["LRScale"])) or 1.0
            for i in g[1]:
                self.group_of[i] = (scale, float(np.float32(sg["WeightDecay"])))
        self.plan.update(self._descs())
        self.step_count = int(cfg["StepCount"])
        self.lr, self.beta1, self.beta2, self.eps = (float(np.float32(cfg[k])) for k in ("LR", "Beta1", "Beta2", "Eps"))

    def close(self) -> None:
        """Releases the plan and unmaps the peers' buffers. Local and idempotent: no collective is
        enqueued, so a rank that survives a `RankLost` can call it. Nothing of another rank can still
        be touching this rank's buffers once its own stream has drained: a step ends with an exchange
        that every rank's stores precede, and a peer cannot begin the next pull without this rank.
        The buffers themselves are torch tensors; they go back to torch's allocator, not to the driver."""
        if self._closed:
            return
        self._closed = True
        self.torch.cuda.synchronize()
        if self.ctx is not None:
            self.ctx.close()
            self.ctx = None
        self.plan.close()
        for base in self._imported:
            self.engine.ipc_close(base, self.device)
        self._imported = []


class Zero1SGD(Zero1AdamW):
    """The sharded form of SGD.Step (autograd/sgd.go:192-225): same flat layout, reduction, norm and
    shadow exchange as `Zero1AdamW`; the owner of a shard keeps the momentum buffer of its pieces and
    one init flag per piece (the reference keeps one per tensor: a tensor that straddles two shards
    has a piece, and a flag, on each owner; state files carry the reference's one flag per tensor)."""

    def __init__(self, numels: Sequence[int], group_of: Sequence[Tuple[float, float]], lr: float, momentum: float,
                 dampening: float, nesterov: bool, maximize: bool, max_norm: float, device: int, comm: str = "peer",
                 process_group=None, chunk_elems: int = 0, **options):
        if nesterov and (not momentum > 0 or dampening != 0):
            raise ValueError("autograd: Nesterov momentum requires a positive momentum and zero dampening")
        self.momentum, self.dampening, self.nesterov, self.maximize = momentum, dampening, nesterov, maximize
        # the base class fingerprints (lr, beta1, beta2, eps, max_norm): momentum and dampening take
        # the places of the betas, the two switches the place of eps
        super().__init__(numels, group_of, lr, momentum, dampening, float(2 * int(nesterov) + int(maximize)), max_norm,
                         device, comm, process_group, chunk_elems, **options)

    def _allocate_state(self, dev) -> None:
        torch = self.torch
        self.buffer = torch.zeros(self.layout.shard_len, dtype=torch.float32, device=dev)
        self.flags = torch.zeros(max(len(self.my_pieces), 1), dtype=torch.float32, device=dev)

    def _descs(self):
        lo, descs = self.lo, []
        for k, pc in enumerate(self.my_pieces):
            a, b = pc.flat_offset, pc.flat_offset + pc.length
            scale, decay = self.group_of[pc.tensor]
            has_state = self.momentum > 0
            descs.append(self.engine.TensorDesc(self.master[a - lo:b - lo], self.grad_flat[a:b],
                                                self.buffer[a - lo:b - lo] if has_state else None,
                                                self.flags[k:k + 1] if has_state else None, self.shadow_flat[a:b], scale, decay))
        return descs

    def _sgd_hparams(self):
        from .engine import OE_MAXIMIZE, OE_NESTEROV, OE_WRITE_SHADOW
        flags = OE_WRITE_SHADOW | (OE_NESTEROV if self.nesterov else 0) | (OE_MAXIMIZE if self.maximize else 0)
        return self.engine.SGDHParams(self.lr, self.momentum, self.dampening, self.max_norm, flags)

    def update(self) -> None:
        hp = self._sgd_hparams()
        if self.comm == "nccl":
            self.plan.sgd_step(hp)
        elif self.comm == "abi":
            self.ctx.sgd_update(hp)
        elif self.multicast:
            self.plan.sgd_step_multicast(hp, self.shadow_deltas, self.mc_delta)
        else:
            self.plan.sgd_step_peers(hp, self._push_deltas())

    def _abi_step(self) -> None:
        self.ctx.sgd_step(self._sgd_hparams())

    def _device_sync(self) -> None:
        self.torch.cuda.synchronize()

    def _state_loaded(self) -> None:
        self.plan.update(self._descs())   # the groups' scale and decay live in the device table

    # ---- state files in the reference's "gograd-sgd" layout (autograd/sgd_state.go:27-194) --------
    def tensor_flags(self) -> List[bool]:
        """The reference keeps one "buffer initialised" flag per tensor; this class keeps one per piece.
        Every rank learns every piece's flag; a tensor is initialised when all of its pieces are. A
        tensor whose pieces disagree has no counterpart in the reference's state and is refused."""
        self._device_sync()
        mine = [bool(x) for x in self.flags[:len(self.my_pieces)].cpu().tolist()] if self.momentum > 0 else \
               [False] * len(self.my_pieces)
        everyone = [None] * self.world
        self.dist.all_gather_object(everyone, mine, group=self.pg)
        votes: List[List[bool]] = [[] for _ in self.layout.numels]
        for r, flags in enumerate(everyone):
            for pc, flag in zip(self.layout.pieces(r), flags):
                votes[pc.tensor].append(flag)
        for i, v in enumerate(votes):
            if any(v) != all(v):
                raise ValueError(f"autograd: SGD momentum buffer {i} is initialised on some ranks only")
        return [all(v) for v in votes]

    def save_state(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]]) -> None:
        """Rank 0 writes the sharded momentum buffers as a "gograd-sgd" state file: one entry buffer.<i>
        of shape [numel] per initialised parameter, the flags, options and groups in the metadata — the
        file an unsharded SGD reads back (autograd/sgd_state.go:150-194). Streamed like the sharded
        AdamW state: the owners send their pieces in file order, rank 0 appends them."""
        initialized = self.tensor_flags()
        groups = self.groups()
        stream = None
        if self.rank == 0:
            from . import autograd as host
            stream = host.SGDStateStream(path, list(names), [list(s) for s in shapes], self.step_count, self.lr,
                                         self.momentum, self.dampening, groups[0][3], self.nesterov, self.maximize,
                                         initialized, groups)
        order = sorted(f"buffer.{i}" for i, flag in enumerate(initialized) if flag)
        self._stream_entries(stream, order, lambda key: self.buffer)

    def load_state(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]]) -> None:
        """Every rank reads the file and takes its pieces of the momentum buffers and their flags. The
        whole file is checked first (format, names, shapes, options, flags against entries, finite
        values, group layout: autograd/sgd_state.go:68-100,166-194); nothing changes when a check fails."""
        import json
        import math
        import struct

        import numpy as np
        n = len(self.layout.numels)
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(hlen))
            base = 8 + hlen
            meta = header.pop("__metadata__", {})
            if meta.get("format") != "gograd-sgd" or meta.get("version") != "1":
                raise ValueError("autograd: unsupported SGD state format")
            cfg = json.loads(meta["optimizer"])
            opt = cfg["Options"]
            flags = list(cfg.get("Initialized") or [])
            if cfg["StepCount"] != int(meta["step_count"]) or cfg["StepCount"] < 0 or len(flags) != len(cfg["Names"] or []):
                raise ValueError("autograd: invalid SGD state metadata")
            for key in ("LR", "Momentum", "Dampening", "WeightDecay"):
                if not (math.isfinite(opt[key]) and opt[key] >= 0):
                    raise ValueError("autograd: invalid SGD configuration")
            if opt["Nesterov"] and (not opt["Momentum"] > 0 or opt["Dampening"] != 0):
                raise ValueError("autograd: Nesterov momentum requires a positive momentum and zero dampening")
            if len(flags) != n or list(cfg["Names"] or []) != list(names) or \
                    [list(s) for s in (cfg["Shapes"] or [])] != [list(s) for s in shapes]:
                raise ValueError("autograd: invalid SGD state count")
            if len(header) != sum(1 for b in flags if b):
                raise ValueError("autograd: unexpected SGD state entries")
            for i, flag in enumerate(flags):
                entry = header.get(f"buffer.{i}")
                if flag:
                    if not opt["Momentum"] > 0 or cfg["StepCount"] == 0 or entry is None or entry["dtype"] != "F32" \
                            or entry["shape"] != [self.layout.numels[i]]:
                        raise ValueError(f"autograd: invalid SGD momentum buffer {i}")
            if bool(opt["Momentum"] > 0) != bool(self.momentum > 0):
                raise ValueError("autograd: the saved state and the live optimizer disagree on momentum")
            saved_groups = cfg.get("Groups") or []
            live = self.groups()
            if len(saved_groups) != len(live) or any(
                    [names[i] for i in g[1]] != sg["Names"] for g, sg in zip(live, saved_groups)):
                raise ValueError("autograd: saved parameter groups do not match the live optimizer")
            staged = np.zeros(self.layout.shard_len, np.float32)
            piece_flags = np.zeros(max(len(self.my_pieces), 1), np.float32)
            for k, pc in enumerate(self.my_pieces):
                if not flags[pc.tensor]:
                    continue
                entry = header[f"buffer.{pc.tensor}"]
                f.seek(base + entry["data_offsets"][0] + 4 * pc.tensor_offset)
                values = np.frombuffer(f.read(4 * pc.length), dtype="<f4")
                if values.size != pc.length or not np.all(np.isfinite(values)):
                    raise ValueError("autograd: non-finite SGD momentum")
                a = pc.flat_offset - self.lo
                staged[a:a + pc.length] = values
                piece_flags[k] = 1.0
        if self.momentum > 0:
            self.buffer.copy_(self.torch.from_numpy(staged))
            self.flags.copy_(self.torch.from_numpy(piece_flags))
        for g, sg in zip(live, saved_groups):
            scale = float(np.float32(sg["LRScale"])) or 1.0
            for i in g[1]:
                self.group_of[i] = (scale, float(np.float32(sg["WeightDecay"])))
        self._state_loaded()
        self.step_count = int(cfg["StepCount"])
        self.lr, self.momentum, self.dampening = (float(np.float32(opt[k])) for k in ("LR", "Momentum", "Dampening"))
        self.nesterov, self.maximize = bool(opt["Nesterov"]), bool(opt["Maximize"])
