"""Python face of the C ABI: plans over torch tensors. No arithmetic happens here."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

from . import _lib
from ._lib import (OE_TUNE_PEER_PUSH_WARP_ROTATE, OE_TUNE_PEER_REDUCE_FIRST, OE_TUNE_PEER_REDUCE_GRID,
                   OE_TUNE_PEER_REDUCE_WARP_ROTATE,
                   OE_TUNE_PEER_UPDATE_GRID, OE_TUNE_PEER_UPDATE_VECTORS, OE_TUNE_STEP_GRID, OE_ZERO1_CE_NONE,
                   OE_ZERO1_NO_ENTRY_EXCHANGE, OE_ZERO1_SYNC_BYTES)
from ._lib import (OE_ACCUMULATE, OE_CLIP_DEVFORM, OE_MAXIMIZE, OE_NESTEROV, OE_PARTIAL_ONLY, OE_WRITE_SHADOW, OE_ZERO_GRAD,
                   EngineError, check, lib)

_initialised = set()


def init(device: int = 0) -> None:
    """oe_init once per device; raises EngineError without a driver or a B200."""
    if device not in _initialised:
        check(lib().oe_init(device))
        _initialised.add(device)


def _addr(t) -> int:
    return 0 if t is None else int(t.data_ptr())


def _stream(stream) -> int:
    if stream is None:
        import torch
        return int(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


@dataclass
class TensorDesc:
    """One parameter as the engine sees it (oe_tensor_desc). Tensors are torch CUDA
    tensors (fp32; shadow bf16 or int16/uint16) or None."""
    param: object
    grad: object = None
    state1: object = None
    state2: object = None
    shadow: object = None
    lr_scale: float = 1.0
    weight_decay: float = 0.0

    def to_c(self) -> _lib.oe_tensor_desc:
        return _lib.oe_tensor_desc(_addr(self.param), _addr(self.grad), _addr(self.state1), _addr(self.state2),
                                   _addr(self.shadow), int(self.param.numel()), self.lr_scale, self.weight_decay)


@dataclass
class AdamWHParams:
    lr: float
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    bc1: float = 1.0
    bc2: float = 1.0
    max_norm: float = 0.0
    flags: int = 0
    step_dev: int = 0
    lr_dev: int = 0

    def to_c(self) -> _lib.oe_adamw_hparams:
        return _lib.oe_adamw_hparams(self.lr, self.beta1, self.beta2, self.eps, self.bc1, self.bc2, self.max_norm,
                                     self.flags, self.step_dev, self.lr_dev)


@dataclass
class SGDHParams:
    lr: float
    momentum: float = 0.0
    dampening: float = 0.0
    max_norm: float = 0.0
    flags: int = 0
    step_dev: int = 0
    lr_dev: int = 0

    def to_c(self) -> _lib.oe_sgd_hparams:
        return _lib.oe_sgd_hparams(self.lr, self.momentum, self.dampening, self.max_norm, self.flags, 0,
                                   self.step_dev, self.lr_dev)


def _desc_array(descs: Sequence[TensorDesc]):
    arr = (_lib.oe_tensor_desc * max(len(descs), 1))()
    for i, d in enumerate(descs):
        arr[i] = d.to_c()
    return arr


class Plan:
    """oe_plan: device tables for one parameter list on one device."""

    def __init__(self, descs: Sequence[TensorDesc], device: int = 0, chunk_elems: int = 0):
        init(device)
        self.device = device
        self._descs = list(descs)  # keeps the tensors alive while the plan borrows them
        self._h = C.c_void_p()
        check(lib().oe_plan_create(device, _desc_array(descs), len(descs), chunk_elems, C.byref(self._h)))

    def update(self, descs: Sequence[TensorDesc], stream=None) -> None:
        self._descs = list(descs)
        check(lib().oe_plan_update(self._h, _desc_array(descs), len(descs), _stream(stream)))

    def info(self, what: int) -> int:
        return int(lib().oe_plan_info(self._h, what))

    @property
    def n_active(self) -> int:
        return self.info(0)

    @property
    def n_chunks(self) -> int:
        return self.info(1)

    @property
    def active_elems(self) -> int:
        return self.info(2)

    @property
    def uploads(self) -> int:
        return self.info(6)

    def norm_address(self) -> int:
        return int(lib().oe_plan_norm_address(self._h))

    def set_variant(self, name: str) -> None:
        check(lib().oe_plan_set_variant(self._h, name.encode()))

    def set_grad_scale(self, scale: float) -> None:
        """Norm and update kernels read every gradient element as float32(g * scale) from now on."""
        check(lib().oe_plan_set_grad_scale(self._h, C.byref(C.c_float(scale))))

    def grad_norm(self, flags: int = 0, stream=None) -> None:
        check(lib().oe_grad_norm(self._h, flags, _stream(stream)))

    def norm_finalize(self, stream=None) -> None:
        check(lib().oe_norm_finalize(self._h, _stream(stream)))

    def clip_grad_norm(self, max_norm: float, flags: int = 0, stream=None) -> None:
        mx = C.c_float(max_norm)
        check(lib().oe_clip_grad_norm(self._h, C.byref(mx), flags, _stream(stream)))

    def read_norm(self, stream=None):
        n, s = C.c_float(), C.c_double()
        check(lib().oe_read_norm(self._h, C.byref(n), C.byref(s), _stream(stream)))
        return n.value, s.value

    def adamw_step(self, hp: AdamWHParams, stream=None) -> None:
        c = hp.to_c()
        check(lib().oe_adamw_step(self._h, C.byref(c), _stream(stream)))

    def adamw_step_chunks(self, hp: AdamWHParams, first_chunk: int, n_chunks: int, stream=None) -> None:
        """The update over a contiguous range of the plan's work units (oe_adamw_step_chunks)."""
        c = hp.to_c()
        check(lib().oe_adamw_step_chunks(self._h, C.byref(c), first_chunk, n_chunks, _stream(stream)))

    def sgd_step(self, hp: SGDHParams, stream=None) -> None:
        c = hp.to_c()
        check(lib().oe_sgd_step(self._h, C.byref(c), _stream(stream)))

    def peer_reduce_grads(self, rank_bases: Sequence[int], first_elem: int, numel: int, out_address: int,
                          scale: float, flags: int = 0, stream=None) -> None:
        """Pull reduce-scatter + sum of squares over peer-mapped gradient buffers (oe_peer_reduce_grads)."""
        bases = (C.c_uint64 * len(rank_bases))(*rank_bases)
        sc = C.c_float(scale)
        check(lib().oe_peer_reduce_grads(self._h, bases, len(rank_bases), first_elem, numel, out_address,
                                         C.byref(sc), flags, _stream(stream)))

    def adamw_step_peers(self, hp: AdamWHParams, shadow_deltas: Sequence[int], stream=None) -> None:
        """AdamW step whose shadow stores go to every rank's shadow buffer (oe_adamw_step_peers)."""
        c = hp.to_c()
        deltas = (C.c_int64 * len(shadow_deltas))(*shadow_deltas)
        check(lib().oe_adamw_step_peers(self._h, C.byref(c), deltas, len(shadow_deltas), _stream(stream)))

    def sgd_step_peers(self, hp: SGDHParams, shadow_deltas: Sequence[int], stream=None) -> None:
        """SGD step whose shadow stores go to every rank's shadow buffer (oe_sgd_step_peers)."""
        c = hp.to_c()
        deltas = (C.c_int64 * len(shadow_deltas))(*shadow_deltas)
        check(lib().oe_sgd_step_peers(self._h, C.byref(c), deltas, len(shadow_deltas), _stream(stream)))

    def adamw_step_multicast(self, hp: AdamWHParams, shadow_deltas: Sequence[int], mc_delta: int, stream=None) -> None:
        """oe_adamw_step_peers with the 8-byte shadow vectors sent once through a multicast mapping."""
        c = hp.to_c()
        deltas = (C.c_int64 * len(shadow_deltas))(*shadow_deltas)
        check(lib().oe_adamw_step_multicast(self._h, C.byref(c), deltas, len(shadow_deltas),
                                            C.byref(C.c_int64(mc_delta)), _stream(stream)))

    def sgd_step_multicast(self, hp: SGDHParams, shadow_deltas: Sequence[int], mc_delta: int, stream=None) -> None:
        c = hp.to_c()
        deltas = (C.c_int64 * len(shadow_deltas))(*shadow_deltas)
        check(lib().oe_sgd_step_multicast(self._h, C.byref(c), deltas, len(shadow_deltas),
                                          C.byref(C.c_int64(mc_delta)), _stream(stream)))

    def link_probe_reads(self, rank_bases: Sequence[int], first_elem: int, numel: int, stream=None) -> None:
        """Every load of the pull-reduce over the range, no element stored (oe_link_probe_reads)."""
        bases = (C.c_uint64 * len(rank_bases))(*rank_bases)
        check(lib().oe_link_probe_reads(self._h, bases, len(rank_bases), first_elem, numel, _stream(stream)))

    def link_probe_stores(self, shadow_shard: int, shadow_deltas: Sequence[int], numel: int, stream=None) -> None:
        """bf16 zeros over the range of every other rank's shadow buffer (oe_link_probe_stores)."""
        deltas = (C.c_int64 * len(shadow_deltas))(*shadow_deltas)
        check(lib().oe_link_probe_stores(self._h, shadow_shard, deltas, len(shadow_deltas), numel, _stream(stream)))

    def set_tuning(self, what: int, value: int) -> None:
        """A launch-shape knob of the peer kernels (oe_plan_set_tuning); results never change."""
        check(lib().oe_plan_set_tuning(self._h, what, value))

    def zero_grads(self, stream=None) -> None:
        check(lib().oe_zero_grads(self._h, _stream(stream)))

    def adamw_step_from_host(self, hp: AdamWHParams, host_grads: Sequence[Optional[object]], stream=None) -> float:
        """host_grads: per parameter a CPU torch tensor / numpy array (ideally page-locked) or None."""
        n = len(host_grads)
        ptrs = (C.c_void_p * max(n, 1))()
        for i, g in enumerate(host_grads):
            if g is None:
                ptrs[i] = None
            elif hasattr(g, "data_ptr"):
                ptrs[i] = g.data_ptr()
            else:
                ptrs[i] = g.ctypes.data
        c = hp.to_c()
        norm = C.c_float()
        check(lib().oe_adamw_step_from_host(self._h, C.byref(c), ptrs, n, C.byref(norm), _stream(stream)))
        return norm.value

    def close(self) -> None:
        if self._h:
            check(lib().oe_plan_destroy(self._h))
            self._h = C.c_void_p()
            self._descs = []

    def __del__(self):  # best effort; explicit close() is the supported way
        try:
            if getattr(self, "_h", None):
                lib().oe_plan_destroy(self._h)
        except Exception:
            pass


def cast_bf16(src, dst, stream=None, device: int = 0) -> None:
    """Stand-alone fp32 -> bf16 cast of one tensor (oe_cast_bf16)."""
    init(device)
    check(lib().oe_cast_bf16(device, _addr(src), _addr(dst), int(src.numel()), _stream(stream)))


def ipc_export(address: int, device: int = 0):
    """(64-byte handle, offset) of the allocation containing a device address (oe_ipc_export)."""
    init(device)
    handle = (C.c_ubyte * 64)()
    offset = C.c_uint64()
    check(lib().oe_ipc_export(device, address, handle, C.byref(offset)))
    return bytes(handle), int(offset.value)


def ipc_import(handle: bytes, device: int = 0) -> int:
    """Maps a peer's allocation on this device and returns its base address (oe_ipc_import)."""
    init(device)
    buf = (C.c_ubyte * 64).from_buffer_copy(handle)
    base = C.c_uint64()
    check(lib().oe_ipc_import(device, buf, C.byref(base)))
    return int(base.value)


def ipc_close(base: int, device: int = 0) -> None:
    check(lib().oe_ipc_close(device, base))


class Zero1Context:
    """oe_zero1: a sharded step whose exchanges between the ranks are the library's own kernels."""

    def __init__(self, plan: Plan, rank: int, world: int, first_elem: int, numel: int, grad_bases: Sequence[int],
                 shadow_deltas: Sequence[int], sync_blocks: Sequence[int], mc_delta: int = 0, timeout_ms: int = 0,
                 flags: int = 0, staging: int = 0, staging_bytes: int = 0, ce_pull_sources: int = 0,
                 ce_push_targets: int = 0, staging_bases: Optional[Sequence[int]] = None):
        d = _lib.oe_zero1_desc()
        d.rank, d.world, d.first_elem, d.numel = rank, world, first_elem, numel
        for k in range(world):
            d.grad_bases[k], d.shadow_deltas[k], d.sync_blocks[k] = grad_bases[k], shadow_deltas[k], sync_blocks[k]
        d.shadow_mc_delta, d.timeout_ms, d.flags = mc_delta, timeout_ms, flags
        d.staging, d.staging_bytes = staging, staging_bytes
        d.ce_pull_sources, d.ce_push_targets = ce_pull_sources, ce_push_targets
        for k, base in enumerate(staging_bases or []):
            d.staging_bases[k] = base
        self._plan = plan  # the context borrows the plan
        self._h = C.c_void_p()
        check(lib().oe_zero1_create(plan._h, C.byref(d), C.byref(self._h)))

    def adamw_step(self, hp: AdamWHParams, stream=None) -> None:
        c = hp.to_c()
        check(lib().oe_zero1_adamw_step(self._h, C.byref(c), _stream(stream)))

    def sgd_step(self, hp: SGDHParams, stream=None) -> None:
        c = hp.to_c()
        check(lib().oe_zero1_sgd_step(self._h, C.byref(c), _stream(stream)))

    def exchange(self, phase: int, stream=None) -> None:
        check(lib().oe_zero1_exchange(self._h, phase, _stream(stream)))

    def copy_engine_use(self) -> Tuple[int, int]:
        """(peers staged by a copy in the reduce phase, ranks served by a shadow copy in the update phase)."""
        return int(lib().oe_zero1_info(self._h, 0)), int(lib().oe_zero1_info(self._h, 1))

    def staging_written_by_owners(self) -> bool:
        return int(lib().oe_zero1_info(self._h, 3)) == 1

    def reduce(self, stream=None) -> None:
        """The reduce phase alone: staged copies (if the context uses them) and the pull kernel."""
        check(lib().oe_zero1_reduce(self._h, _stream(stream)))

    def adamw_update(self, hp: AdamWHParams, stream=None) -> None:
        """The update phase alone: fused update with its shadow stores, then the shadow copies."""
        c = hp.to_c()
        check(lib().oe_zero1_adamw_update(self._h, C.byref(c), _stream(stream)))

    def sgd_update(self, hp: SGDHParams, stream=None) -> None:
        c = hp.to_c()
        check(lib().oe_zero1_sgd_update(self._h, C.byref(c), _stream(stream)))

    def status(self, stream=None) -> int:
        """Waits for the stream; 0 when every exchange completed, else raises EngineError (OE_ERR_DEVICE)."""
        word = C.c_uint32()
        check(lib().oe_zero1_status(self._h, C.byref(word), _stream(stream)))
        return int(word.value)

    def status_word(self, stream=None) -> int:
        """The raw status word, without raising."""
        word = C.c_uint32()
        code = lib().oe_zero1_status(self._h, C.byref(word), _stream(stream))
        if code not in (0, _lib.OE_ERR_DEVICE):
            check(code)
        return int(word.value)

    def close(self) -> None:
        if self._h:
            check(lib().oe_zero1_destroy(self._h))
            self._h = C.c_void_p()


def launch_count(name: Optional[str] = None) -> int:
    return int(lib().oe_launch_count(None if name is None else name.encode()))


def launch_count_reset() -> None:
    lib().oe_launch_count_reset()


__all__ = ["AdamWHParams", "SGDHParams", "TensorDesc", "Plan", "cast_bf16", "init", "launch_count",
           "launch_count_reset", "EngineError", "OE_CLIP_DEVFORM", "OE_WRITE_SHADOW", "OE_ZERO_GRAD", "OE_NESTEROV",
           "OE_MAXIMIZE", "OE_PARTIAL_ONLY", "OE_ACCUMULATE"]


def profile_enable(enabled: bool = True) -> None:
    """Per-launch timing like the reference's EnableGPUProfile: serialises every launch while on."""
    lib().oe_profile_enable(int(enabled))


def profile(name: Optional[str] = None):
    """(launch count, device milliseconds) of one kernel, or of all kernels."""
    count, ms = C.c_int64(), C.c_double()
    check(lib().oe_profile_get(None if name is None else name.encode(), C.byref(count), C.byref(ms)))
    return int(count.value), float(ms.value)
